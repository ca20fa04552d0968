// Translation unit of the light ops: finalize, eltwise, norm, rope_append, increment, gather, argmax.
#include "op_pointwise.cuh"
#include "ops.cuh"

namespace mk {
__device__ int mk_op_pointwise(const Params& p, const mk_op_desc* op, int a0, int a1, int seq, Sync sy) {
    const SmemMap m = smem_map();
    if (begin_op(p, m.ctrl, sy, seq)) return -1;
    int unknown = 0;
    switch (op->kind) {
        case MK_OP_FINALIZE: op_finalize(op, a0, a1); break;
        case MK_OP_ELTWISE: op_eltwise(op, a0, a1); break;
        case MK_OP_NORM: op_norm(op, a0, m.work); break;
        case MK_OP_ROPE_APPEND: op_rope_append(op, a0); break;
        case MK_OP_INCREMENT: op_increment(op); break;
        case MK_OP_GATHER: op_gather(op, a0, a1); break;
        case MK_OP_ARGMAX: op_argmax(op, a0, a1, m.ctrl, m.work); break;
        default: unknown = 1; break;
    }
    return end_op(p, m.ctrl, sy) ? -1 : unknown;
}
}  // namespace mk
