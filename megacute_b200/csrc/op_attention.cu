// Translation unit of MK_OP_ATTENTION.
#include "op_attention.cuh"
#include "ops.cuh"

namespace mk {
__device__ int mk_op_attention(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int seq, Sync sy) {
    const SmemMap m = smem_map();
    uint8_t* work = m.work;
    if (begin_op(p, m.ctrl, sy, seq)) return -1;
    const bool f16 = op->i[8] == DT_F16;
    if (op->i[5] == 64) {
        if (f16) op_attention<64, true>(op, a0, a1, a2, work);
        else op_attention<64, false>(op, a0, a1, a2, work);
    } else {
        if (f16) op_attention<128, true>(op, a0, a1, a2, work);
        else op_attention<128, false>(op, a0, a1, a2, work);
    }
    return end_op(p, m.ctrl, sy) ? -1 : 0;
}
}  // namespace mk
