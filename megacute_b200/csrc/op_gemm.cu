// Translation unit of MK_OP_GEMM.
#include "op_gemm.cuh"
#include "ops.cuh"

namespace mk {
__device__ void mk_op_gemm(const mk_op_desc* op, int a0, int a1, int a2) {
    // ops with at most 64 activation rows have a single m tile: hold 64 rows and stream deeper
    if (op->i[0] <= 64) {
        if ((op->i[2] / op->i[4]) % 64 == 0) op_gemm<64, 64, 3>(op, a0, a1, a2, smem_map().work);
        else op_gemm<64, 32, 6>(op, a0, a1, a2, smem_map().work);
    } else {
        op_gemm<128, 32, 4>(op, a0, a1, a2, smem_map().work);
    }
}
}  // namespace mk
