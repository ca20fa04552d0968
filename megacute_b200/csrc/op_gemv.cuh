// Compute-warp side of MK_OP_GEMV (see op_gemv_common.cuh for the layout and the producer side).
#pragma once
#include "op_gemv_common.cuh"
#include "mma.cuh"

namespace mk {

// Compute warps: consume the stages of one GEMV instruction.  MB = compile-time bound on M.
template <int MB>
__device__ __forceinline__ RingPos gemv_compute(const Params& p, Ctrl* c, uint8_t* ring, uint8_t* work,
                                                const mk_op_desc* op, int o0, int o1, int seq, RingPos pos) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int M = op->i[0], K = op->i[2], act = op->i[3];
    const bool swi = op->flags & GEMV_F_SWIGLU;
    float* xs = reinterpret_cast<float*>(work);                          // [M][K] fp32
    float* red = reinterpret_cast<float*>(work + kXbufBytes);            // [2][8 warps][8 slots][MB]
    float* rowstat = red + 2 * kComputeWarps * 8 * MB;                   // [8 warps][MB] then [MB]

    // ---- stage the activation rows in shared memory (and normalise them) ----
    {
        const int xdt = op->i[4];
        const long long ldx = op->ld[0];
        const void* x = reinterpret_cast<const void*>(op->ptr[0]);
        const int vec_per_row = K >> 3;
        float ss[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) ss[m] = 0.f;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            if (m < M) {
                for (int v = t; v < vec_per_row; v += kComputeThreads) {
                    float f[8];
                    load8(x, m * ldx + v * 8, xdt, f);
                    float4* d = reinterpret_cast<float4*>(xs + m * K + v * 8);
                    d[0] = make_float4(f[0], f[1], f[2], f[3]);
                    d[1] = make_float4(f[4], f[5], f[6], f[7]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss[m] += f[e] * f[e];
                }
            }
        }
        if (op->flags & GEMV_F_RMS) {
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                float s = warp_sum(ss[m]);
                if (lane == 0) rowstat[warp * MB + m] = s;
            }
            compute_sync();
            const __nv_bfloat16* gain = reinterpret_cast<const __nv_bfloat16*>(op->ptr[5]);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                if (m < M) {
                    float s = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < kComputeWarps; ++w8) s += rowstat[w8 * MB + m];
                    const float rstd = rsqrt_approx(s / (float)K + op->f[0]);
                    for (int v = t; v < vec_per_row; v += kComputeThreads) {
                        float4* d = reinterpret_cast<float4*>(xs + m * K + v * 8);
                        float4 a = d[0], b = d[1];
                        float gq[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
                        if (gain) unpack8(*reinterpret_cast<const uint4*>(gain + v * 8), gq);
                        d[0] = make_float4(a.x * rstd * gq[0], a.y * rstd * gq[1], a.z * rstd * gq[2], a.w * rstd * gq[3]);
                        d[1] = make_float4(b.x * rstd * gq[4], b.y * rstd * gq[5], b.z * rstd * gq[6], b.w * rstd * gq[7]);
                    }
                }
            }
        }
        compute_sync();
    }

    const int per = swi ? 4 : 8;
    const int groups = (o1 - o0 + per - 1) / per;
    const int nkc = (K + kGemvKChunk - 1) / kGemvKChunk;
    int rb = 0;
    for (int g = 0; g < groups; ++g) {
        float acc[8][MB];
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
        for (int kc = 0; kc < nkc; ++kc) {
            const int k0 = kc * kGemvKChunk;
            const int kl = min(kGemvKChunk, K - k0);
            const bool active = t * 8 < kl;
            float xf[MB][8];
            if (active) {
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    if (m < M) {
                        const float4* s = reinterpret_cast<const float4*>(xs + m * K + k0 + t * 8);
                        float4 a = s[0], b = s[1];
                        xf[m][0] = a.x; xf[m][1] = a.y; xf[m][2] = a.z; xf[m][3] = a.w;
                        xf[m][4] = b.x; xf[m][5] = b.y; xf[m][6] = b.z; xf[m][7] = b.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) xf[m][e] = 0.f;
                    }
                }
            }
            const bool ok = wait_barrier(p, c, &c->full[pos.stage], pos.phase, seq, WHERE_RING_FULL);
            if (ok && active) {
                const uint4* st = reinterpret_cast<const uint4*>(ring + pos.stage * kStageBytes) + t;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    float wf[8];
                    unpack8(st[r * (kGemvKChunk / 8)], wf);
#pragma unroll
                    for (int m = 0; m < MB; ++m)
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[r][m] = fmaf(wf[e], xf[m][e], acc[r][m]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->empty[pos.stage]);
            pos.advance();
        }
        // ---- reduce the group across the CTA and write its outputs ----
        float* rbuf = red + rb * (kComputeWarps * 8 * MB);
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                float s = warp_sum(acc[r][m]);
                if (lane == 0) rbuf[(warp * 8 + r) * MB + m] = s;
            }
        compute_sync();
        if (t < per * MB) {
            const int j = t % per, m = t / per;
            const int o = o0 + g * per + j;
            if (o < o1 && m < M) {
                float a = 0.f, b = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < kComputeWarps; ++w8) {
                    a += rbuf[(w8 * 8 + j) * MB + m];
                    if (swi) b += rbuf[(w8 * 8 + j + 4) * MB + m];
                }
                float y;
                if (swi) {
                    y = a * sigmoidf_(a) * b;
                } else {
                    if (op->ptr[3]) a += load1(reinterpret_cast<const void*>(op->ptr[3]), o, 0);
                    y = apply_act(act, a);
                    if (op->ptr[4]) y += load1(reinterpret_cast<const void*>(op->ptr[4]), (long long)m * op->ld[4] + o, op->i[6]);
                }
                store1(reinterpret_cast<void*>(op->ptr[2]), (long long)m * op->ld[2] + o, op->i[5], y);
            }
        }
        rb ^= 1;
    }
    return pos;
}

// The general path behind one call: returns the advanced ring position packed as stage | phase << 8.
static __device__ __noinline__ int gemv_general(const Params& p, Ctrl* c, uint8_t* ring, uint8_t* work, const mk_op_desc* op,
                                        int o0, int o1, int seq, int stage, int phase) {
    RingPos pos;
    pos.stage = stage;
    pos.phase = (uint32_t)phase;
    const int M = op->i[0];
    if (M <= 1) pos = gemv_compute<1>(p, c, ring, work, op, o0, o1, seq, pos);
    else if (M <= 2) pos = gemv_compute<2>(p, c, ring, work, op, o0, o1, seq, pos);
    else if (M <= 4) pos = gemv_compute<4>(p, c, ring, work, op, o0, o1, seq, pos);
    else pos = gemv_compute<8>(p, c, ring, work, op, o0, o1, seq, pos);
    return pos.stage | ((int)pos.phase << 8);
}

}  // namespace mk
