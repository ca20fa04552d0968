// Translation unit of MK_OP_ATTENTION.
#include "op_attention.cuh"
#include "ops.cuh"

namespace mk {
__device__ void mk_op_attention(const mk_op_desc* op, int a0, int a1, int a2) {
    uint8_t* work = smem_map().work;
    if (op->i[5] == 64) op_attention<64>(op, a0, a1, a2, work);
    else op_attention<128>(op, a0, a1, a2, work);
}
}  // namespace mk
