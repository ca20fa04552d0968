// Greedy sampling: row-wise argmax of the logits, the last thing a decode step does before the
// next token's embedding is gathered (the reference's loop calls torch's argmax there,
// examples/llama/llama1b.py:105).  A row of 128 256 bf16 logits is 250 KB, read once with 16-byte
// loads by kSplit CTAs of 1024 threads; each leaves its best (value, index) in a static device
// array and the last CTA of a row to finish picks the winner (ties go to the lowest index).  Rows
// beyond the static array's capacity are handled by one CTA each.  Nothing is allocated.
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

constexpr int kSplit = 16;                 // CTAs per row
constexpr int kMaxSplitRows = 4096;        // rows the static scratch covers (512 KB + 16 KB per GPU)
__device__ float g_part_v[kMaxSplitRows * kSplit];
__device__ int g_part_i[kMaxSplitRows * kSplit];
__device__ int g_done[kMaxSplitRows];      // zero between launches: the last CTA of a row resets it

// grid (rows, nsplit): CTA (r, s) scans every nsplit-th 16-byte vector group of row r
__global__ void __launch_bounds__(1024) argmax_rows(const void* logits, int dtype, int cols, long long ld, long long* out) {
    const int t = threadIdx.x;
    const int nsplit = gridDim.y, part = blockIdx.y;
    const int stride = 1024 * nsplit, first = part * 1024 + t;
    Best best{-__builtin_huge_valf(), 0x7fffffff};
    if (dtype == 0) {
        const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(logits) + (long long)blockIdx.x * ld;
        const int nvec = cols >> 3;                                // rows start 16-byte aligned (ld % 8 == 0)
        for (int v = first; v < nvec; v += stride) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(row) + v);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float x = __uint_as_float(e & 1 ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16));
                best = better(best, Best{x, v * 8 + e});
            }
        }
        for (int c = (nvec << 3) + first; c < cols; c += stride) best = better(best, Best{__bfloat162float(row[c]), c});
    } else {
        const float* row = reinterpret_cast<const float*>(logits) + (long long)blockIdx.x * ld;
        for (int c = first; c < cols; c += stride) best = better(best, Best{row[c], c});
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
        if (nsplit == 1) {
            if (t == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
            return;
        }
        // several CTAs per row: leave this CTA's best, and let the last one to arrive reduce them
        __shared__ int last;
        if (t == 0) {
            g_part_v[blockIdx.x * kSplit + part] = best.v;
            g_part_i[blockIdx.x * kSplit + part] = best.i;
            __threadfence();
            last = atomicAdd(&g_done[blockIdx.x], 1) == nsplit - 1;
        }
        __syncwarp();
        if (!last) return;
        __threadfence();
        best = Best{-__builtin_huge_valf(), 0x7fffffff};
        if (t < nsplit) best = Best{__ldcg(&g_part_v[blockIdx.x * kSplit + t]), __ldcg(&g_part_i[blockIdx.x * kSplit + t])};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (t == 0) {
            out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
            g_done[blockIdx.x] = 0;
        }
    }
}

}  // namespace

extern "C" int mk_argmax(const void* logits, int dtype, int rows, int cols, long long ld, long long* out, void* stream) {
    if (!logits || !out || rows <= 0 || cols <= 0 || (dtype != 0 && dtype != 1) || ld < cols) return MK_E_ARG;
    if (dtype == 0 && ((ld & 7) != 0 || (reinterpret_cast<uintptr_t>(logits) & 15) != 0)) return MK_E_ARG;
    // few long rows: several CTAs per row (calls that may overlap on the GPU share the scratch: serialise them)
    const int nsplit = (rows <= 64 && rows <= kMaxSplitRows && cols >= 16 * 1024) ? kSplit : 1;
    argmax_rows<<<dim3(rows, nsplit), 1024, 0, (cudaStream_t)stream>>>(logits, dtype, cols, ld, out);
    return cudaGetLastError() == cudaSuccess ? MK_OK : MK_E_CUDA;
}
