// MK_OP_DECODE_ATTN: one query token per sequence against its KV cache, GQA, flash-decoding.
//
// One instruction = (sequence b, kv head j, split s of S).  The split owns a contiguous range of
// the cached keys, computed on the device from pos so that any context length spreads evenly over
// the S instructions.  Keys and values stream through a two-stage cp.async pipeline of 128-key
// tiles (64 for head_dim 128).  S = Q K^T and O += P V run on tensor cores (mma.sync m16n8k16): the
// G <= 8 query heads of the kv head are the rows of the A operand, every warp works on its own 16
// keys of a tile with its own running max and sum, and the warps are merged once after the loop,
// so a tile costs two CTA barriers.  With S > 1 every split writes an unnormalised partial (O,
// running max, sum) and bumps an arrival count; the last split to arrive merges the S partials
// and writes the output (no extra dependency hop).
// q and P are each split into bf16 high + low parts so scores and probabilities keep ~16 mantissa
// bits where the reference rounds both to bf16 (megacute/ops/attention.py:293).  The low parts
// ride in rows 8..15 of the same A operand (heads take rows 0..7), so they cost no extra MMA: the
// two row halves of a result fragment are added in the lane that holds both.  The
// appended k and v are rounded to the cache's bf16 and the new token is scored with those values.
// Fused mode (rope_append folded in): q, k_new, v_new are the un-rotated columns of the QKV row;
// the op rotates q and k at pos, the last split also attends the new token from registers and
// appends k, v to cache row b * max_seq + pos (reference semantics: graph.py:412-418).
//
// ptr 0 q, 1 k_cache, 2 v_cache, 3 pos, 4 out, 5 k_new, 6 v_new, 7 cos, 8 sin, 9 part, 10 count; i 12 pos stride, 13 window
// i 0 B, 1 H, 2 KVH, 3 D, 4 max_seq, 5 splits, 6 fused, 7 dtype of q / k_new / v_new, 8 out dtype,
//   9 zero q / k_new / v_new after use (they are fp32 columns of a split-K workspace: the instruction that
//     writes the pair's output hands them back zeroed, as the SplitFinalize it replaces would),
//   10 kv heads per instruction, 11 many-sequence form (op_decode_bulk.cuh: all kv heads, whole rows by bulk copies);
//   f 0 scale
// args: 0 b, 1 kv head, 2 split
#pragma once
#include "mk_device.cuh"
#include "mma.cuh"

namespace mk {

template <int D>
constexpr int kDecTileKeys = D <= 64 ? 128 : 64;     // keys per tile; 16 per computing warp
constexpr int kMaxKvSplits = 32;          // config.py MAX_KV_SPLITS

template <int D, int GMAX>
__device__ __forceinline__ void decode_body(const Params& p, Ctrl* c, const mk_op_desc* op, int a0, int a1, int a2,
                                            uint8_t* work, int nwait, int wait_off, int seq) {
    constexpr int ROWB = D * 2 + 16;                   // padded tile row: conflict-free ldmatrix
    constexpr int TK = kDecTileKeys<D>;                // keys per tile; warp w owns keys 16w .. 16w + 15 of a tile
    constexpr int NW = TK / 16;                        // warps that compute
    constexpr int TILE_BYTES = TK * ROWB;              // one K or V tile
    constexpr int NST = 2;
    constexpr int CPR = D / 8;                         // 16-byte chunks per row
    constexpr int VPT = TK * CPR / kComputeThreads;    // chunks per thread per tile and tensor
    constexpr int WROW = D + 2;                        // per (warp, head) record of the intra-CTA merge: O, m, l
    constexpr float NEG_INF = -__builtin_huge_valf();
    static_assert(GMAX <= 8, "heads take rows 0..7 of the A operand, their low parts rows 8..15");
    static_assert(2 * NST * TILE_BYTES + 16 * ROWB + 4096 <= kWorkBytes, "decode tiles exceed the work area");
    static_assert(kComputeWarps * GMAX * WROW * 4 <= 2 * NST * TILE_BYTES, "merge records reuse the tile buffers");

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int dp = t % CPR;
    const int H = op->i[1], KVH = op->i[2], L = op->i[4], S = op->i[5], qdt = op->i[7];
    const bool fused = op->i[6] != 0;
    const int G = H / KVH;
    const int b = a0, kvh = a1, s = a2;
    // one position for the batch, or (i 12: stride) one per sequence; i 13: sliding window, the last `window` tokens
    // -- the new one included -- of the sequence (0: all of them)
    const int pos = reinterpret_cast<const int*>(op->ptr[3])[(long long)b * op->i[12]];
    const int n = fused ? pos : pos + 1;
    const int first = op->i[13] > 0 ? max(0, pos + 1 - op->i[13]) : 0;    // first cache row attended
    const int per = (n - first + S - 1) / S;
    const int k_begin = min(n, first + s * per), k_end = min(n, k_begin + per);
    const int nk = k_end - k_begin;                                       // cached keys of this split
    const bool has_new = fused && s == S - 1;
    const int half = D / 2;

    uint8_t* kst = work;                                                  // NST K tiles then NST V tiles
    uint8_t* vst = work + NST * TILE_BYTES;
    uint8_t* qs = work + 2 * NST * TILE_BYTES;                            // q [16][ROWB]: rows 0..7 high parts, 8..15 low parts
    float* sSc = reinterpret_cast<float*>(qs + 16 * ROWB);                // new token's score   [GMAX]
    float* snew = sSc + GMAX;                                             // new token: k [D], v [D] (bf16 values)
    float* wred = reinterpret_cast<float*>(work);                         // [8 warps][GMAX][WROW] after the loop

    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(op->ptr[2]);
    const long long ldk = op->ld[1], ldv = op->ld[2];
    const long long row0 = (long long)b * L;

    auto issue_tile = [&](int tile) {
        const int key0 = tile * TK;
        const int st = tile % NST;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = t + i * kComputeThreads;
            const int key = key0 + v / CPR, ch = v % CPR;
            const bool valid = key < nk;
            const long long r = row0 + k_begin + (valid ? key : 0);
            cp_async16(kst + st * TILE_BYTES + (v / CPR) * ROWB + ch * 16, kc + r * ldk + kvh * D + ch * 8, valid);
            cp_async16(vst + st * TILE_BYTES + (v / CPR) * ROWB + ch * 16, vc + r * ldv + kvh * D + ch * 8, valid);
        }
    };

    const int ntiles = (nk + TK - 1) / TK;
    // Fused mode reads only cache rows below pos, which nothing in this launch writes: the first
    // tile and the rope table row are requested before the dependency wait (the op waits for its
    // own dependencies).  Unfused mode may read the row a RopeAppend of this launch wrote, so it
    // waits first.
    if (!fused && wait_deps(p, c, nwait, wait_off, seq)) return;
    if (ntiles > 0) issue_tile(0);
    cp_async_commit();
    const int pd = dp < CPR / 2 ? dp * 8 + half : dp * 8 - half;         // partner chunk of the rotation
    const float sign = dp < CPR / 2 ? -1.f : 1.f;
    float cs[8], sn[8];
    if (fused) {
        load8(reinterpret_cast<const __nv_bfloat16*>(op->ptr[7]) + (long long)pos * op->ld[7], dp * 8, 0, cs);
        load8(reinterpret_cast<const __nv_bfloat16*>(op->ptr[8]) + (long long)pos * op->ld[8], dp * 8, 0, sn);
    }
    for (int v = t; v < 16 * ROWB / 16; v += kComputeThreads) reinterpret_cast<uint4*>(qs)[v] = make_uint4(0u, 0u, 0u, 0u);
    if (fused && wait_deps(p, c, nwait, wait_off, seq)) {
        cp_async_wait<0>();
        return;
    }
    if (!fused) compute_sync();                                           // the zero fill of qs, before the rows below land
    if (t == 0 && p.trace_cap > 0) c->t_dep = (long long)globaltimer();

    // ---- q (rotated when fused, pre-scaled to the log2 domain) as MMA A operand: rows = the G query
    // heads of this kv head, split into bf16 high and low parts so the scores keep ~16 mantissa bits.
    // One thread per 8-wide chunk; the new token's k and v take two more chunk rows. ----
    {
        const float qscale = op->f[0] * kLog2e;
        const int chunk = t / CPR;                                        // 0..G-1 q heads, G k_new, G+1 v_new
        if (chunk < G || (has_new && chunk < G + 2)) {
            const int which = chunk - G;                                  // < 0: q
            const void* src = reinterpret_cast<const void*>(which < 0 ? op->ptr[0] : op->ptr[5 + which]);
            const long long e0 = which < 0 ? (long long)b * op->ld[0] + (kvh * G + chunk) * D
                                           : (long long)b * op->ld[5 + which] + kvh * D;
            float a[8], o[8];
            load8(src, e0 + dp * 8, qdt, a);
            const bool rot = fused && which != 1;                         // v is not rotated
            if (rot) load8(src, e0 + pd, qdt, o);
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = rot ? a[e] * cs[e] + sign * o[e] * sn[e] : a[e];
            if (which < 0) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float y0 = y[2 * j] * qscale, y1 = y[2 * j + 1] * qscale;
                    const float h0 = round_bf16(y0), h1 = round_bf16(y1);
                    hi[j] = pack2(h0, h1);
                    lo[j] = pack2(y0 - h0, y1 - h1);
                }
                *reinterpret_cast<uint4*>(qs + chunk * ROWB + dp * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(qs + (8 + chunk) * ROWB + dp * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) snew[which * D + dp * 8 + e] = round_bf16(y[e]);     // the cache holds bf16
            }
        }
    }

    // ---- main loop: S = Q K^T and O += P V on tensor cores, every warp on its own 16 keys of the
    // tile with its own running max and sum (no barrier inside a tile) ----
    float oacc[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
    float mrow = NEG_INF, lrow = 0.f;                                     // head lane >> 2
    const uint32_t q_a = smem_u32(qs) + (lane & 15) * ROWB + (lane >> 4) * 16;

#pragma unroll 1
    for (int tile = 0; tile < ntiles; ++tile) {
        if (tile + 1 < ntiles) issue_tile(tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
        compute_sync();                                                   // tile (and, first time, q) visible to all
        const int kb0 = tile * TK + 16 * warp;                            // first key of this warp, relative to the split
        if (warp < NW && kb0 < nk) {
            const uint32_t kb = smem_u32(kst + (tile % NST) * TILE_BYTES) + 16 * warp * ROWB;
            const uint32_t vb = smem_u32(vst + (tile % NST) * TILE_BYTES) + 16 * warp * ROWB;
            float sc[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t a[4], b0, b1, b2, b3;
                ldmatrix_x4(q_a + kk * 32, a[0], a[1], a[2], a[3]);
                ldmatrix_x4(kb + ((lane & 7) + (lane >> 4) * 8) * ROWB + (kk * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
                mma_bf16(sc[0], a, b0, b1);
                mma_bf16(sc[1], a, b2, b3);
            }
            // score of head lane >> 2 = high-part row + low-part row; mask keys past the end of the split
            float mx = NEG_INF;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kb0 + j * 8 + (lane & 3) * 2 + e;
                    sc[j][e] = key >= nk ? NEG_INF : sc[j][e] + sc[j][e + 2];
                    mx = fmaxf(mx, sc[j][e]);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mnew = fmaxf(mrow, mx);                           // finite: the warp has at least one key
            const float alpha = mrow == NEG_INF ? 0.f : ex2(mrow - mnew);
            mrow = mnew;
            uint32_t pa[4];                                               // P as A operand: rows 0..7 high parts, 8..15 low parts
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float p0 = sc[j][0] == NEG_INF ? 0.f : ex2(sc[j][0] - mnew);
                const float p1 = sc[j][1] == NEG_INF ? 0.f : ex2(sc[j][1] - mnew);
                sum += p0 + p1;
                const float h0 = round_bf16(p0), h1 = round_bf16(p1);
                pa[j * 2] = pack2(h0, h1);                                // head lane >> 2, keys j * 8 + ...
                pa[j * 2 + 1] = pack2(p0 - h0, p1 - h1);
            }
            lrow = lrow * alpha + sum;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) oacc[j][e] *= alpha;
            }
#pragma unroll
            for (int jp = 0; jp < D / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vb + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (jp * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
                mma_bf16(oacc[jp * 2], pa, b0, b1);
                mma_bf16(oacc[jp * 2 + 1], pa, b2, b3);
            }
        }
        compute_sync();                                                   // the stage is overwritten by the next issue
    }
    cp_async_wait<0>();
    if (ntiles == 0) compute_sync();                                      // q and snew visible without the loop's barriers
    phase_mark(p, c, 0);

    // ---- the new token (fused mode, last split): its score per head from the q parts in shared
    // memory, and its k, v appended to the cache ----
    if (has_new) {
        if (warp < G) {
            float a = 0.f;
            for (int d = lane; d < D; d += 32) {
                const float qv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(qs + warp * ROWB + d * 2)) +
                                 __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(qs + (8 + warp) * ROWB + d * 2));
                a = fmaf(qv, snew[d], a);
            }
            a = warp_sum(a);
            if (lane == 0) sSc[warp] = a;
        }
        if (t < CPR) {
            float kn[8], vn[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) { kn[e] = snew[t * 8 + e]; vn[e] = snew[D + t * 8 + e]; }
            const long long row = row0 + pos;
            store8(const_cast<__nv_bfloat16*>(kc), row * ldk + kvh * D + t * 8, 0, kn);
            store8(const_cast<__nv_bfloat16*>(vc), row * ldv + kvh * D + t * 8, 0, vn);
        }
    }
    // ---- per-warp results to shared memory (the tile buffers are free: every warp passed the
    // loop's last barrier) ----
    lrow += __shfl_xor_sync(0xffffffffu, lrow, 1);
    lrow += __shfl_xor_sync(0xffffffffu, lrow, 2);
    {
        const int g = lane >> 2;
        if (g < G) {
            float* rec = wred + (warp * GMAX + g) * WROW;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {                             // high-part rows + low-part rows
                rec[j * 8 + (lane & 3) * 2] = oacc[j][0] + oacc[j][2];
                rec[j * 8 + (lane & 3) * 2 + 1] = oacc[j][1] + oacc[j][3];
            }
            if ((lane & 3) == 0) { rec[D] = mrow; rec[D + 1] = lrow; }
        }
    }
    compute_sync();

    // ---- merge the warps (and the new token) per output element: `acc` is this split's
    // unnormalised O, with its running max and sum ----
    const int GD = G * D;
    auto merged = [&](int idx, float& mx_out, float& l_out) {
        const int g = idx / D, d = idx % D;
        float mx = has_new ? sSc[g] : NEG_INF;
#pragma unroll
        for (int w = 0; w < kComputeWarps; ++w) mx = fmaxf(mx, wred[(w * GMAX + g) * WROW + D]);
        float a = 0.f, l = 0.f;
        if (mx != NEG_INF) {
#pragma unroll
            for (int w = 0; w < kComputeWarps; ++w) {
                const float* rec = wred + (w * GMAX + g) * WROW;
                const float wgt = rec[D] == NEG_INF ? 0.f : ex2(rec[D] - mx);
                a = fmaf(wgt, rec[d], a);
                l = fmaf(wgt, rec[D + 1], l);
            }
            if (has_new) {
                const float pn = ex2(sSc[g] - mx);
                a = fmaf(pn, snew[D + d], a);
                l += pn;
            }
        }
        mx_out = mx;
        l_out = l;
        return a;
    };
    const int pair = b * KVH + kvh;
    // every instruction of the pair has read q (and the one with the new token k_new, v_new) by the
    // time one of them writes the pair's output
    auto zero_inputs = [&]() {
        if (!op->i[9]) return;
        float* q = reinterpret_cast<float*>(op->ptr[0]) + (long long)b * op->ld[0] + kvh * GD;
        for (int idx = t; idx < GD; idx += kComputeThreads) q[idx] = 0.f;
        if (t < 2 * D) {
            const int which = t / D;
            reinterpret_cast<float*>(op->ptr[5 + which])[(long long)b * op->ld[5 + which] + kvh * D + t % D] = 0.f;
        }
    };
    void* outp = reinterpret_cast<void*>(op->ptr[4]);
    const int odt = op->i[8];
    if (S == 1) {
        for (int idx = t; idx < GD; idx += kComputeThreads) {
            float mx, l;
            const float a = merged(idx, mx, l);
            store1(outp, (long long)b * op->ld[4] + kvh * GD + idx, odt, l == 0.f ? 0.f : a * rcp(l));
        }
        zero_inputs();
        return;
    }
    float* part = reinterpret_cast<float*>(op->ptr[9]);
    const long long ldp = op->ld[9];
    {
        float* mine = part + ((long long)pair * S + s) * ldp;
        for (int idx = t; idx < GD; idx += kComputeThreads) {
            float mx, l;
            mine[idx] = merged(idx, mx, l);
            if (idx % D == 0) { mine[GD + idx / D] = mx; mine[GD + G + idx / D] = l; }
        }
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
    zero_inputs();
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

// i 10 > 1 (unsplit batched decode): kv heads a1 .. a1 + i10 - 1 of the sequence, one after the other;
// fetch, dependency wait and arrival are paid once per instruction.  A function of its own: in the
// single-head function the loop's extra live state costs registers (spills are L2 round trips here).
template <int D, int GMAX>
static __device__ __noinline__ void decode_one_head(const Params& p, Ctrl* c, const mk_op_desc* op, int a0, int a1, int a2,
                                                    uint8_t* work, int nwait, int wait_off, int seq) {
    decode_body<D, GMAX>(p, c, op, a0, a1, a2, work, nwait, wait_off, seq);
}
template <int D, int GMAX>
static __device__ __noinline__ bool op_decode_attn_heads(const Params& p, Ctrl* c, const mk_op_desc* op, int a0, int a1, int a2,
                                                         uint8_t* work, int nwait, int wait_off, int seq, int narrive,
                                                         int arrive_off) {
    const int hp = op->i[10];
#pragma unroll 1
    for (int j = 0; j < hp; ++j) {
        if (j) compute_sync();                                  // the previous head's merge reads the tile buffers
        decode_one_head<D, GMAX>(p, c, op, a0, a1 + j, a2, work, j ? 0 : nwait, wait_off, seq);
        if (*(volatile int*)&c->abort) break;
    }
    return publish(p, c, narrive, arrive_off);
}

}  // namespace mk
