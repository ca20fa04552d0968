// MK_OP_DECODE_ATTN: one query token per sequence against its KV cache, GQA, flash-decoding.
//
// One instruction = (sequence b, kv head j, split s of S).  The split owns a contiguous range of
// the cached keys, computed on the device from pos so that any context length spreads evenly over
// the S instructions.  Keys and values stream through a cp.async pipeline of 64-key tiles; the
// G query heads of the kv head are held in registers.  With S > 1 every split writes an
// unnormalised partial (O, running max, sum) and bumps an arrival count; the last split to arrive
// merges the S partials and writes the output (no extra dependency hop).
// Scores, probabilities and the rotated query stay fp32 (this path runs on CUDA cores, so the
// reference's bf16 rounding of P and q before its tensor-core products is not needed); the
// appended k and v are rounded to the cache's bf16 and the new token is scored with those values.
// Fused mode (rope_append folded in): q, k_new, v_new are the un-rotated columns of the QKV row;
// the op rotates q and k at pos, the last split also attends the new token from registers and
// appends k, v to cache row b * max_seq + pos (reference semantics: graph.py:412-418).
//
// ptr 0 q, 1 k_cache, 2 v_cache, 3 pos, 4 out, 5 k_new, 6 v_new, 7 cos, 8 sin, 9 part, 10 count
// i 0 B, 1 H, 2 KVH, 3 D, 4 max_seq, 5 splits, 6 fused, 7 dtype of q / k_new / v_new, 8 out dtype;  f 0 scale
// args: 0 b, 1 kv head, 2 split
#pragma once
#include "mk_device.cuh"

namespace mk {

constexpr int kDecTileKeys = 64;
constexpr int kMaxKvSplits = 32;          // config.py MAX_KV_SPLITS

template <int D, int GMAX>
__device__ __forceinline__ void decode_body(const Params& p, Ctrl* c, const mk_op_desc* op, int a0, int a1, int a2,
                                            uint8_t* work, int nwait, int wait_off, int seq) {
    constexpr int DP = D / 8;                         // threads per key (8 dims each)
    constexpr int KPP = kComputeThreads / DP;         // keys per pass
    constexpr int PASSES = kDecTileKeys / KPP;
    constexpr int TILE_BYTES = kDecTileKeys * D * 2;
    constexpr int NST = (D == 64) ? 4 : 2;
    constexpr int VPT = kDecTileKeys * DP / kComputeThreads;      // 16-byte vectors per thread per tile
    constexpr float NEG_INF = -__builtin_huge_valf();

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int dp = t % DP, kg = t / DP;
    const int H = op->i[1], KVH = op->i[2], L = op->i[4], S = op->i[5], qdt = op->i[7];
    const bool fused = op->i[6] != 0;
    const int G = H / KVH;
    const int b = a0, kvh = a1, s = a2;
    const int pos = *reinterpret_cast<const int*>(op->ptr[3]);
    const int n = fused ? pos : pos + 1;
    const int per = (n + S - 1) / S;
    const int k_begin = min(n, s * per), k_end = min(n, k_begin + per);
    const bool has_new = fused && s == S - 1;
    const int half = D / 2;

    uint8_t* kst = work;                                         // NST K tiles then NST V tiles (64 KB)
    uint8_t* vst = work + NST * TILE_BYTES;
    float* sS = reinterpret_cast<float*>(work + 2 * NST * TILE_BYTES);     // [GMAX][64]
    float* sP = sS + GMAX * kDecTileKeys;                                 // [GMAX][64]
    float* sM = sP + GMAX * kDecTileKeys;                                 // running max   [GMAX]
    float* sL = sM + GMAX;                                                // running sum   [GMAX]
    float* sA = sL + GMAX;                                                // rescale       [GMAX]
    float* snew = sA + GMAX;                                              // new token: k [D], v [D]
    float* ored = reinterpret_cast<float*>(work);                         // [KPP][G*D] after the loop

    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(op->ptr[2]);
    const long long ldk = op->ld[1], ldv = op->ld[2];
    const long long row0 = (long long)b * L;

    auto issue_tile = [&](int tile) {
        const int key0 = k_begin + tile * kDecTileKeys;
        const int st = tile % NST;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = t + i * kComputeThreads;
            const int key = key0 + v / DP, ch = v % DP;
            const bool valid = key < k_end;
            const long long r = row0 + (valid ? key : k_begin);
            cp_async16(kst + st * TILE_BYTES + v * 16, kc + r * ldk + kvh * D + ch * 8, valid);
            cp_async16(vst + st * TILE_BYTES + v * 16, vc + r * ldv + kvh * D + ch * 8, valid);
        }
    };

    const int ntiles = (k_end - k_begin + kDecTileKeys - 1) / kDecTileKeys;
    // Fused mode reads only cache rows below pos, which nothing in this launch writes: the first
    // tiles and the rope table row are requested before the dependency wait (the op waits for its
    // own dependencies).  Unfused mode may read the row a RopeAppend of this launch wrote, so it
    // waits first.
    if (!fused && wait_deps(p, c, nwait, wait_off, seq)) return;
#pragma unroll
    for (int i = 0; i < NST - 1; ++i) {
        if (i < ntiles) issue_tile(i);
        cp_async_commit();
    }
    const int pd = dp < DP / 2 ? dp * 8 + half : dp * 8 - half;     // partner chunk of the rotation
    const float sign = dp < DP / 2 ? -1.f : 1.f;
    float cs[8], sn[8];
    if (fused) {
        load8(reinterpret_cast<const __nv_bfloat16*>(op->ptr[7]) + (long long)pos * op->ld[7], dp * 8, 0, cs);
        load8(reinterpret_cast<const __nv_bfloat16*>(op->ptr[8]) + (long long)pos * op->ld[8], dp * 8, 0, sn);
    }
    if (t < GMAX) { sM[t] = NEG_INF; sL[t] = 0.f; }
    if (fused && wait_deps(p, c, nwait, wait_off, seq)) {
        cp_async_wait<0>();
        return;
    }
    if (t == 0 && p.trace_cap > 0) c->t_dep = (long long)globaltimer();

    // ---- query heads into registers (rotated when fused), pre-scaled to the log2 domain.  All
    // loads of a batch of four heads are issued before any is used: one L2 round trip per batch. ----
    float qf[GMAX][8];
    const float qscale = op->f[0] * kLog2e;
    {
        const void* q = reinterpret_cast<const void*>(op->ptr[0]);
        float kn[8], ko[8], vn[8];
        if (has_new && kg == 0) {          // only the first key slot's threads use the new token's k and v
            const long long ek = (long long)b * op->ld[5] + kvh * D, ev = (long long)b * op->ld[6] + kvh * D;
            load8(reinterpret_cast<const void*>(op->ptr[5]), ek + dp * 8, qdt, kn);
            load8(reinterpret_cast<const void*>(op->ptr[5]), ek + pd, qdt, ko);
            load8(reinterpret_cast<const void*>(op->ptr[6]), ev + dp * 8, qdt, vn);
        }
#pragma unroll
        for (int gb = 0; gb < GMAX; gb += 4) {
            float a[4][8], o[4][8];
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) {
                const int g = gb + g4;
                if (g < G) {
                    const long long e0 = (long long)b * op->ld[0] + (kvh * G + g) * D;
                    load8(q, e0 + dp * 8, qdt, a[g4]);
                    if (fused) load8(q, e0 + pd, qdt, o[g4]);
                }
            }
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) {
                const int g = gb + g4;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float v = 0.f;
                    if (g < G) v = fused ? a[g4][e] * cs[e] + sign * o[g4][e] * sn[e] : a[g4][e];
                    qf[g][e] = v * qscale;
                }
            }
        }
        if (has_new && kg == 0) {          // new token's rotated k and its v wait in shared memory
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                snew[dp * 8 + e] = round_bf16(kn[e] * cs[e] + sign * ko[e] * sn[e]);
                snew[D + dp * 8 + e] = round_bf16(vn[e]);
            }
        }
    }

    float oacc[GMAX][8];
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) oacc[g][e] = 0.f;

#pragma unroll 1
    for (int tile = 0; tile < ntiles; ++tile) {
        if (tile + NST - 1 < ntiles) issue_tile(tile + NST - 1);
        cp_async_commit();
        cp_async_wait<NST - 1>();
        compute_sync();
        const int st = tile % NST;
        const int key0 = k_begin + tile * kDecTileKeys;
        // ---- scores ----
#pragma unroll
        for (int ps = 0; ps < PASSES; ++ps) {
            const int key = ps * KPP + kg;
            float kf[8];
            unpack8(*reinterpret_cast<const uint4*>(kst + st * TILE_BYTES + (key * DP + dp) * 16), kf);
            float sc[GMAX];
#pragma unroll
            for (int g = 0; g < GMAX; ++g) {
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) a = fmaf(qf[g][e], kf[e], a);
#pragma unroll
                for (int o = 1; o < DP; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                sc[g] = a;
            }
            const bool in_range = key0 + key < k_end;
#pragma unroll
            for (int g = 0; g < GMAX; ++g)
                if (dp == g && g < G) sS[g * kDecTileKeys + key] = in_range ? sc[g] : NEG_INF;
        }
        compute_sync();
        // ---- online softmax: warp g owns query head g ----
        if (warp < G) {
            const float s0 = sS[warp * kDecTileKeys + lane], s1 = sS[warp * kDecTileKeys + lane + 32];
            const float mo = sM[warp];
            const float mn = fmaxf(mo, warp_max(fmaxf(s0, s1)));
            const float p0 = s0 == NEG_INF ? 0.f : ex2(s0 - mn);
            const float p1 = s1 == NEG_INF ? 0.f : ex2(s1 - mn);
            sP[warp * kDecTileKeys + lane] = p0;
            sP[warp * kDecTileKeys + lane + 32] = p1;
            const float sum = warp_sum(p0 + p1);
            if (lane == 0) {
                const float al = mo == NEG_INF ? 0.f : ex2(mo - mn);
                sA[warp] = al;
                sL[warp] = sL[warp] * al + sum;
                sM[warp] = mn;
            }
        }
        compute_sync();
        // ---- O += P V ----
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            if (g < G) {
                const float al = sA[g];
#pragma unroll
                for (int e = 0; e < 8; ++e) oacc[g][e] *= al;
            }
        }
#pragma unroll
        for (int ps = 0; ps < PASSES; ++ps) {
            const int key = ps * KPP + kg;
            float vf[8];
            unpack8(*reinterpret_cast<const uint4*>(vst + st * TILE_BYTES + (key * DP + dp) * 16), vf);
#pragma unroll
            for (int g = 0; g < GMAX; ++g) {
                if (g < G) {
                    const float pg = sP[g * kDecTileKeys + key];
#pragma unroll
                    for (int e = 0; e < 8; ++e) oacc[g][e] = fmaf(pg, vf[e], oacc[g][e]);
                }
            }
        }
        compute_sync();
    }
    cp_async_wait<0>();
    phase_mark(p, c, 0);

    // ---- the new token (fused mode, last split): attend it from registers and append it ----
    if (ntiles == 0) compute_sync();     // no tile loop ran: its barriers are what orders snew otherwise
    if (has_new) {
        float kn[8], vn[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) { kn[e] = snew[dp * 8 + e]; vn[e] = snew[D + dp * 8 + e]; }
        if (kg == 0) {
#pragma unroll
            for (int g = 0; g < GMAX; ++g) {
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) a = fmaf(qf[g][e], kn[e], a);
#pragma unroll
                for (int o = 1; o < DP; o <<= 1) a += __shfl_xor_sync((1u << DP) - 1u, a, o);
                if (dp == g && g < G) {
                    const float mo = sM[g];
                    const float mn = fmaxf(mo, a);
                    const float al = mo == NEG_INF ? 0.f : ex2(mo - mn);
                    const float pn = ex2(a - mn);
                    sA[g] = al;
                    sP[g * kDecTileKeys] = pn;
                    sL[g] = sL[g] * al + pn;
                    sM[g] = mn;
                }
            }
            const long long row = row0 + pos;
            store8(const_cast<__nv_bfloat16*>(kc), row * ldk + kvh * D + dp * 8, 0, kn);
            store8(const_cast<__nv_bfloat16*>(vc), row * ldv + kvh * D + dp * 8, 0, vn);
        }
        compute_sync();
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            if (g < G) {
                const float al = sA[g];
                const float pn = kg == 0 ? sP[g * kDecTileKeys] : 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) oacc[g][e] = fmaf(pn, vn[e], oacc[g][e] * al);
            }
        }
    }
    compute_sync();          // every tile has been consumed: the tile buffers can be reused

    // ---- reduce O over the KPP key slots ----
    const int GD = G * D;
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
        if (g < G) {
            float4* d = reinterpret_cast<float4*>(ored + kg * GD + g * D + dp * 8);
            d[0] = make_float4(oacc[g][0], oacc[g][1], oacc[g][2], oacc[g][3]);
            d[1] = make_float4(oacc[g][4], oacc[g][5], oacc[g][6], oacc[g][7]);
        }
    }
    compute_sync();
    const int pair = b * KVH + kvh;
    void* outp = reinterpret_cast<void*>(op->ptr[4]);
    const int odt = op->i[8];
    if (S == 1) {
        for (int idx = t; idx < GD; idx += kComputeThreads) {
            float a = 0.f;
#pragma unroll 8
            for (int k = 0; k < KPP; ++k) a += ored[k * GD + idx];
            const float l = sL[idx / D];
            store1(outp, (long long)b * op->ld[4] + kvh * GD + idx, odt, l == 0.f ? 0.f : a * rcp(l));
        }
        return;
    }
    float* part = reinterpret_cast<float*>(op->ptr[9]);
    const long long ldp = op->ld[9];
    {
        float* mine = part + ((long long)pair * S + s) * ldp;
        for (int idx = t; idx < GD; idx += kComputeThreads) {
            float a = 0.f;
#pragma unroll 8
            for (int k = 0; k < KPP; ++k) a += ored[k * GD + idx];
            mine[idx] = a;
        }
        if (t < G) { mine[GD + t] = sM[t]; mine[GD + G + t] = sL[t]; }
    }
    __threadfence();
    compute_sync();
    phase_mark(p, c, 1);
    int* count = reinterpret_cast<int*>(op->ptr[10]) + (long long)pair * op->ld[10];
    if (t == 0) {
        const int old = atomicAdd(count, 1);
        c->flag = (old == S - 1);
        if (old == S - 1) *count = 0;          // back to zero for the next launch
    }
    compute_sync();
    phase_mark(p, c, 2);
    if (!c->flag) return;
    __threadfence();
    // ---- last split to arrive: merge the S partials.  The S partial rows are copied into shared
    // memory with one wave of cp.async (one L2 round trip), then every thread merges one output. ----
    const float* base = part + (long long)pair * S * ldp;
    float* sp = reinterpret_cast<float*>(work);                 // [S][row_f] floats; tile buffers are free
    const int row_f = (GD + 2 * G + 3) & ~3;                    // floats per partial row, 16-byte multiple
    const int vec_per_row = row_f >> 2;
    for (int v = t; v < S * vec_per_row; v += kComputeThreads) {
        const int k = v / vec_per_row, j = v % vec_per_row;
        cp_async16(sp + k * row_f + j * 4, base + k * ldp + j * 4, true);
    }
    cp_async_commit();
    cp_async_wait<0>();
    compute_sync();
    for (int idx = t; idx < GD; idx += kComputeThreads) {
        const int g = idx / D;
        float mx = NEG_INF;
        for (int k = 0; k < S; ++k) mx = fmaxf(mx, sp[k * row_f + GD + g]);
        float a = 0.f, l = 0.f;
        for (int k = 0; k < S; ++k) {
            const float mk_ = sp[k * row_f + GD + g];
            const float w = mk_ == NEG_INF ? 0.f : ex2(mk_ - mx);
            a = fmaf(w, sp[k * row_f + idx], a);
            l = fmaf(w, sp[k * row_f + GD + G + g], l);
        }
        store1(outp, (long long)b * op->ld[4] + kvh * GD + idx, odt, l == 0.f ? 0.f : a * rcp(l));
    }
}

// The op waits for its own dependencies (see decode_body) and publishes its own arrivals, so the
// arrivals leave before the function's epilogue (callee-saved register restores come out of local
// memory, an L2 round trip here).  Returns whether the CTA is aborting.
template <int D, int GMAX>
static __device__ __noinline__ bool op_decode_attn(const Params& p, Ctrl* c, const mk_op_desc* op, int a0, int a1, int a2,
                                                   uint8_t* work, int nwait, int wait_off, int seq, int narrive,
                                                   int arrive_off) {
    decode_body<D, GMAX>(p, c, op, a0, a1, a2, work, nwait, wait_off, seq);
    return publish(p, c, narrive, arrive_off);
}

}  // namespace mk
