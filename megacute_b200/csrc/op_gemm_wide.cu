// Translation unit of MK_OP_GEMM with 128 x 256 output tiles on the tcgen05 body (descriptor i 10 = 256 and tensor
// maps attached).  Separate from op_gemm.cu so that each tile shape gets its own register allocation: inlined side
// by side, the wider tile's extra live state spilled registers of the narrow tile's main loop (spills are L2 round
// trips here: batch-64 decode 7 % slower, the MLP block 14 %).
#include "op_gemm_tc_wide.cuh"
#include "ops.cuh"

namespace mk {
__device__ int mk_op_gemm_wide(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int seq, int packed_pos, Sync sy) {
    const SmemMap m = smem_map();
    if (begin_op(p, m.ctrl, sy, seq)) return -1;
    if (op_gemm_tc_wide(p, m.ctrl, m.ring, m.work, op, a0, a1, a2, seq) < 0) return -1;
    return end_op(p, m.ctrl, sy) ? -1 : packed_pos;
}
}  // namespace mk
