// Translation unit of the tensor-core streaming path of MK_OP_GEMV.
#include "op_gemv_mma.cuh"
#include "ops.cuh"

namespace mk {

__device__ int mk_op_gemv_units(const Params& p, const mk_op_desc* op, int o0, int o1, int seq, int packed_pos, int nwait, int wait_off) {
    const SmemMap m = smem_map();
    RingPos pos;
    pos.stage = packed_pos & 0xff;
    pos.phase = (uint32_t)(packed_pos >> 8);
    const int K = op->i[2];
    if (K == kSegElems) gemv_mma<1>(p, m.ctrl, m.ring, m.work, op, o0, o1, seq, pos, nwait, wait_off);
    else if (K == 2 * kSegElems) gemv_mma<2>(p, m.ctrl, m.ring, m.work, op, o0, o1, seq, pos, nwait, wait_off);
    else gemv_mma<0>(p, m.ctrl, m.ring, m.work, op, o0, o1, seq, pos, nwait, wait_off);
    return pos.stage | ((int)pos.phase << 8);
}

}  // namespace mk
