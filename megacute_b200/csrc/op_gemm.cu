// Translation unit of MK_OP_GEMM.
#include "op_gemm.cuh"
#include "ops.cuh"

namespace mk {
__device__ void mk_op_gemm(const mk_op_desc* op, int a0, int a1, int a2) { op_gemm(op, a0, a1, a2, smem_map().work); }
}  // namespace mk
