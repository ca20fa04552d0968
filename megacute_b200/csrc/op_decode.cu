// Translation unit of MK_OP_DECODE_ATTN.
#include "op_decode.cuh"
#include "ops.cuh"

namespace mk {
__device__ bool mk_op_decode_attn(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int nwait, int wait_off,
                                  int seq, int narrive, int arrive_off) {
    const SmemMap m = smem_map();
    const int D = op->i[3], G = op->i[1] / op->i[2];
    if (op->i[11]) return mk_op_decode_bulk(p, op, a0, a2, nwait, wait_off, seq, narrive, arrive_off);
    if (op->i[10] > 1) {        // several kv heads per instruction (batched decode)
        if (D == 64) {
            if (G <= 4) return op_decode_attn_heads<64, 4>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
            return op_decode_attn_heads<64, 8>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
        }
        if (G <= 4) return op_decode_attn_heads<128, 4>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
        return op_decode_attn_heads<128, 8>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
    }
    if (D == 64) {
        if (G <= 4) return op_decode_attn<64, 4>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
        return op_decode_attn<64, 8>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
    } else {
        if (G <= 4) return op_decode_attn<128, 4>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
        return op_decode_attn<128, 8>(p, m.ctrl, op, a0, a1, a2, m.work, nwait, wait_off, seq, narrive, arrive_off);
    }
}
}  // namespace mk
