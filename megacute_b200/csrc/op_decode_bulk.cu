// Translation unit of the many-sequence form of MK_OP_DECODE_ATTN (compute-warp side; the copies are
// issued by the producer warp, op_gemv_common.cuh).
#include "op_decode_bulk.cuh"
#include "ops.cuh"

namespace mk {
__device__ bool mk_op_decode_bulk(const Params& p, const mk_op_desc* op, int b, int s, int nwait, int wait_off, int seq,
                                  int narrive, int arrive_off) {
    const SmemMap m = smem_map();
    const int G = op->i[1] / op->i[2];
    if (G <= 4) return op_decode_bulk<4>(p, m.ctrl, op, b, s, m.ring, nwait, wait_off, seq, narrive, arrive_off);
    return op_decode_bulk<8>(p, m.ctrl, op, b, s, m.ring, nwait, wait_off, seq, narrive, arrive_off);
}
}  // namespace mk
