// Translation unit of MK_OP_GEMM with 128 x 256 output tiles on the tcgen05 body (descriptor i 10 = 256 and tensor
// maps attached).  Separate from op_gemm.cu so that each tile shape gets its own register allocation: inlined side
// by side, the wider tile's extra live state spilled registers of the narrow tile's main loop (spills are L2 round
// trips here: batch-64 decode 7 % slower, the MLP block 14 %).
#include "op_gemm_tc_wide.cuh"
#include "ops.cuh"
#include "walk.cuh"

namespace mk {
__device__ int mk_run_gemm_wide(const Params& p, int idx) {
    const SmemMap m = smem_map();
    return run_own_insts(
        p, m.ctrl, idx, [](const mk_op_desc* op) { return op->kind == MK_OP_GEMM && op->i[10] == 256 && op->ptr[11] != 0; },
        [&](const mk_op_desc* op, int a0, int a1, int a2, int seq) -> int {
            return op_gemm_tc_wide(p, m.ctrl, m.ring, m.work, op, a0, a1, a2, seq);
        });
}
}  // namespace mk
