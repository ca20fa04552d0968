// Translation unit of the tensor-core streaming path of MK_OP_GEMV.
#include "op_gemv_mma.cuh"
#include "ops.cuh"

namespace mk {

__device__ int mk_op_gemv_units(const Params& p, const mk_op_desc* op, int o0, int o1, int seq, int packed_pos, int nwait, int wait_off,
                                int narrive, int arrive_off) {
    const SmemMap m = smem_map();
    RingPos pos;
    pos.stage = packed_pos & 0xff;
    pos.phase = (uint32_t)(packed_pos >> 8) & 1u;
    pos.comb = (uint32_t)(packed_pos >> 16) & 0x1fu;
    gemv_mma(p, m.ctrl, m.ring, m.work, op, o0, o1, seq, pos, nwait, wait_off);
    // The finisher warp has sent the first 32 arrivals (there are rarely more than two); what is left
    // is the barrier that ends the instruction, and any further arrivals.
    const int sent = narrive < 32 ? narrive : 32;
    if (publish(p, m.ctrl, narrive - sent, arrive_off < 0 ? arrive_off : arrive_off + sent)) return -1;
    return pos.stage | ((int)pos.phase << 8) | ((int)pos.comb << 16);
}

__device__ void mk_gemv_finisher(const Params& p) {
    const SmemMap m = smem_map();
    gemv_finisher(p, m.ctrl, m.work);
}

}  // namespace mk
