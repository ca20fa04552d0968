// Greedy sampling: row-wise argmax of the logits, the last thing a decode step does before the
// next token's embedding is gathered (the reference's loop calls torch's argmax there,
// examples/llama/llama1b.py:105).  One CTA of 1024 threads per row: a row of 128 256 bf16 logits is
// 250 KB, read once with 16-byte loads; ties go to the lowest index.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/megacute_b200.h"

namespace {

struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {        // NaN never wins; equal values: lower index
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__global__ void __launch_bounds__(1024) argmax_rows(const void* logits, int dtype, int cols, long long ld, long long* out) {
    const int t = threadIdx.x;
    Best best{-__builtin_huge_valf(), 0x7fffffff};
    if (dtype == 0) {
        const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(logits) + (long long)blockIdx.x * ld;
        const int nvec = cols >> 3;                                // rows start 16-byte aligned (ld % 8 == 0)
        for (int v = t; v < nvec; v += 1024) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + v);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float x = __uint_as_float(e & 1 ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16));
                best = better(best, Best{x, v * 8 + e});
            }
        }
        for (int c = (nvec << 3) + t; c < cols; c += 1024) best = better(best, Best{__bfloat162float(row[c]), c});
    } else {
        const float* row = reinterpret_cast<const float*>(logits) + (long long)blockIdx.x * ld;
        for (int c = t; c < cols; c += 1024) best = better(best, Best{row[c], c});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    __shared__ float sv[32];
    __shared__ int si[32];
    if ((t & 31) == 0) { sv[t >> 5] = best.v; si[t >> 5] = best.i; }
    __syncthreads();
    if (t < 32) {
        best = Best{sv[t], si[t]};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (t == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
    }
}

}  // namespace

extern "C" int mk_argmax(const void* logits, int dtype, int rows, int cols, long long ld, long long* out, void* stream) {
    if (!logits || !out || rows <= 0 || cols <= 0 || (dtype != 0 && dtype != 1) || ld < cols) return MK_E_ARG;
    if (dtype == 0 && ((ld & 7) != 0 || (reinterpret_cast<uintptr_t>(logits) & 15) != 0)) return MK_E_ARG;
    argmax_rows<<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, dtype, cols, ld, out);
    return cudaGetLastError() == cudaSuccess ? MK_OK : MK_E_CUDA;
}
