// Translation unit of MK_OP_ATTENTION on tcgen05 (head_dim 64, tensor maps attached by the host library).
#include "op_attention_tc.cuh"
#include "ops.cuh"

namespace mk {
__device__ int mk_op_attention_tc(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int seq) {
    const SmemMap m = smem_map();
    return op_attention_tc(p, m.ctrl, m.work, op, a0, a1, a2, seq);
}
__device__ void mk_attention_feeder(const Params& p) {
    const SmemMap m = smem_map();
    const int lane = threadIdx.x & 31;
    uint32_t go = 0;                                          // parity of attn_go for the next such instruction
    // the whole warp walks the list (and leaves together: the kernel ends with CTA-wide barriers); lane 0 feeds
    for (int idx = blockIdx.x; idx < p.n_insts; idx += gridDim.x) {
        const Inst in = fetch_inst(p, idx);
        const int opi = in.opi - 1;
        if (opi < 0 || opi >= p.n_ops) return;
        const mk_op_desc* op = p.ops + opi;
        if (op->kind != MK_OP_ATTENTION || !op->ptr[11]) continue;
        int ok = 1;
        if (lane == 0) ok = attention_tc_feed(p, m.ctrl, m.work, op, in.a0, in.a1, in.a2, in.seq, go) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, ok, 0)) return;
        go ^= 1u;
    }
}
}  // namespace mk
