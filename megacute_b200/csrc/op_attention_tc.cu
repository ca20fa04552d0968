// Translation unit of MK_OP_ATTENTION on tcgen05 (head_dim 64, tensor maps attached by the host library).
#include "op_attention_tc.cuh"
#include "ops.cuh"

namespace mk {
__device__ int mk_op_attention_tc(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int seq) {
    const SmemMap m = smem_map();
    return op_attention_tc(p, m.ctrl, m.work, op, a0, a1, a2, seq);
}
__device__ bool mk_attention_tc_feed(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int seq, uint32_t go_parity) {
    const SmemMap m = smem_map();
    return attention_tc_feed(p, m.ctrl, m.work, op, a0, a1, a2, seq, go_parity);
}
}  // namespace mk
