// Translation unit of MK_OP_ATTENTION.
#include "op_attention.cuh"
#include "ops.cuh"

namespace mk {
__device__ void mk_op_attention(const mk_op_desc* op, int a0, int a1, int a2) {
    uint8_t* work = smem_map().work;
    const bool f16 = op->i[8] == DT_F16;
    if (op->i[5] == 64) {
        if (f16) op_attention<64, true>(op, a0, a1, a2, work);
        else op_attention<64, false>(op, a0, a1, a2, work);
    } else {
        if (f16) op_attention<128, true>(op, a0, a1, a2, work);
        else op_attention<128, false>(op, a0, a1, a2, work);
    }
}
}  // namespace mk
