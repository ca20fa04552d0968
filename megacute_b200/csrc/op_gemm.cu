// Translation unit of MK_OP_GEMM.
#include "op_gemm.cuh"
#include "op_gemm_tc.cuh"
#include "ops.cuh"
#include "walk.cuh"

namespace mk {
__device__ int mk_run_gemm(const Params& p, int idx) {
    const SmemMap m = smem_map();
    return run_own_insts(
        p, m.ctrl, idx,
        [](const mk_op_desc* op) { return op->kind == MK_OP_GEMM && !(op->i[10] == 256 && op->ptr[11]); },
        [&](const mk_op_desc* op, int a0, int a1, int a2, int seq) -> int {
            // the host library attached tensor maps: tcgen05 body, weights through the producer's ring
            // (the weight tiles have slots and barriers of their own: the ring position is untouched)
            // (128 x 256 tiles have a translation unit of their own, op_gemm_wide.cu: the kernel calls it directly)
            if (op->ptr[11]) return op_gemm_tc(p, m.ctrl, m.ring, m.work, op, a0, a1, a2, seq);
            // (a 256-wide output tile, i 10, is two 128-wide ones for this body)
            const int halves = op->i[10] == 256 ? 2 : 1;
            for (int hf = 0; hf < halves; ++hf) {
                const int n = a1 * halves + hf;
                // ops with at most 64 activation rows have a single m tile: hold 64 rows and stream deeper
                if (op->i[0] <= 64) {
                    if ((op->i[2] / op->i[4]) % 64 == 0) op_gemm<64, 64, 3>(op, a0, n, a2, m.work);
                    else op_gemm<64, 32, 6>(op, a0, n, a2, m.work);
                } else {
                    op_gemm<128, 32, 4>(op, a0, n, a2, m.work);
                }
            }
            return 0;
        });
}
}  // namespace mk
