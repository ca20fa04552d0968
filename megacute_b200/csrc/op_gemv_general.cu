// Translation unit of the general (2..8 row, or odd K) path of MK_OP_GEMV.
#include "op_gemv.cuh"
#include "ops.cuh"

namespace mk {

__device__ int mk_op_gemv_general(const Params& p, const mk_op_desc* op, int o0, int o1, int seq, int packed_pos) {
    const SmemMap m = smem_map();
    // bits 16.. of the packed position belong to the tensor-core path (hand-over barrier parities)
    const int r = gemv_general(p, m.ctrl, m.ring, m.work, op, o0, o1, seq, packed_pos & 0xff, (packed_pos >> 8) & 1);
    return (r & 0x1ff) | (packed_pos & ~0x1ff);
}

}  // namespace mk
