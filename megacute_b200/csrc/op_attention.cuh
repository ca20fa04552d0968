#pragma once
#include "mk_device.cuh"
namespace mk {
template <int D>
__device__ __forceinline__ void op_attention(const mk_op_desc*, const Inst&, uint8_t*) {}
}  // namespace mk
