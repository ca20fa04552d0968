// Translation unit of the light ops: finalize, eltwise, norm, rope_append, increment, gather, argmax.
#include "op_pointwise.cuh"
#include "ops.cuh"

namespace mk {
__device__ bool mk_op_pointwise(const mk_op_desc* op, int a0, int a1) {
    switch (op->kind) {
        case MK_OP_FINALIZE: op_finalize(op, a0, a1); return true;
        case MK_OP_ELTWISE: op_eltwise(op, a0, a1); return true;
        case MK_OP_NORM: op_norm(op, a0, smem_map().work); return true;
        case MK_OP_ROPE_APPEND: op_rope_append(op, a0); return true;
        case MK_OP_INCREMENT: op_increment(op); return true;
        case MK_OP_GATHER: op_gather(op, a0, a1); return true;
        case MK_OP_ARGMAX: op_argmax(op, a0, a1, smem_map().ctrl, smem_map().work); return true;
        default: return false;
    }
}
}  // namespace mk
