// MK_OP_DECODE_ATTN, many-sequence form (descriptor i 11 = 1): one instruction = (sequence b, KV split s)
// over ALL kv heads of the sequence, head_dim 64.
//
// The cache rows of a sequence are contiguous in memory (a row holds every kv head: KVH x 64 bf16), so
// a tile of 16 consecutive rows is fetched with plain bulk copies of whole rows -- four copies of four
// rows (4 KB with 8 kv heads) per tensor and tile -- where the per-head form (op_decode.cuh) gathers
// 128-byte row pieces with cp.async.  An SM draws ~33 GB/s through cp.async pieces and ~45 GB/s through
// bulk copies of 4 KB and more, so with every SM streaming the KV cache moves at the HBM rate.
//
// Roles.  The producer warp issues the copies (op_gemv_common.cuh, producer_loop): for every instruction
// of this form on its walk down the CTA's instruction list it streams the split's K and V tiles through
// seven 16 KB slots in the ring's memory (kv_full / kv_empty barriers) -- ahead of the compute warps and
// across instruction boundaries, like weights: in the fused form the rows read (below pos) are written
// by nothing in the launch, so the KV stream keeps running through dependency hops.  (The unfused form
// also reads the row a RopeAppend of this launch appended: there the producer waits on kv_go, which the
// compute warps signal once the instruction's dependencies are met.)  Compute warp w owns kv head w for
// the whole split: its own running max, sum and output accumulators, so nothing is merged across warps;
// the S splits of a sequence are merged by the last one to arrive, as in the per-head form.
// Bytes in flight are what sets the rate: with five slots (80 KB, ~3 in flight) the stream ran at
// ~29 GB/s per SM, no faster than the cp.async form.
//
// Shared-memory reads without bank conflicts.  Rows of a tile are 128 x KVH bytes apart, a multiple
// of 128: the same 16-byte slot of every row falls into the same banks, and an MMA fragment needs
// eight different keys at one offset.  Three freedoms of the contraction are used instead of padding:
//   * the four-row groups of a tile are stored 32 bytes apart beyond their size, so rows of different
//     groups differ by two 16-byte slots per group;
//   * S = Q K^T sums over head_dim in any order: thread (n, q) of a warp reads, of key n, the 16-byte
//     chunks q and q + 4 (dims 8q .. 8q+7 and 32+8q .. 32+8q+7) -- even n the low chunk first, odd n the
//     high chunk first, so the eight lanes of a quarter warp hit eight different slots -- and q is laid
//     out in registers in the matching order; rotate-half partners (d, d + 32) sit in one thread;
//   * O = P V sums over keys in any order and its columns can be any permutation of the dims: MMA key
//     index 2q, 2q+1, 2q+8, 2q+9 of lane (n, q) are tile rows 4q .. 4q+3 (one row of each group per
//     load), and column n of the j-th 8-column block is dim 8n + j, so a lane reads one 16-byte chunk
//     (dims 8n .. 8n+7) of each of its four rows and builds the transposed fragments with byte permutes.
//     A lane ends up holding 16 consecutive dims of its head's output.
//
// Numerics as in op_decode.cuh: scores in the log2 domain, q and P as bf16 high + low parts in rows
// 0..7 / 8..15 of the A operand, appended k and v rounded to the cache's bf16.
#pragma once
#include "mk_device.cuh"
#include "mma.cuh"

namespace mk {

__device__ __forceinline__ uint4 kv_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

struct KvPos {
    int slot = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance() {
        if (++slot == kKvSlots) { slot = 0; phase ^= 1u; }
    }
};

// ---- compute warps ----
// All compute threads call this.  Returns after the instruction's global writes (the caller publishes).
template <int GMAX>
__device__ __forceinline__ void decode_bulk_body(const Params& p, Ctrl* c, const mk_op_desc* op, int b, int s, uint8_t* ring,
                                                 int nwait, int wait_off, int seq) {
    constexpr int D = 64;
    constexpr float NEG_INF = -__builtin_huge_valf();
    static_assert(GMAX <= 8, "heads take rows 0..7 of the A operand, their low parts rows 8..15");
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int g = lane >> 2, q4 = lane & 3;                           // MMA row / column group of this lane
    const int H = op->i[1], KVH = op->i[2], L = op->i[4], S = op->i[5], qdt = op->i[7], odt = op->i[8];
    const bool fused = op->i[6] != 0;
    const int G = H / KVH;
    const int rb = KVH * D * 2;
    const bool head = warp < KVH;                                     // this warp owns kv head `warp`
    const bool hrow = head && g < G;                                  // this lane's MMA row is a query head
    const int pos = reinterpret_cast<const int*>(op->ptr[3])[(long long)b * op->i[12]];      // (i 12: 0, or the stride of per-sequence positions)
    int k_begin, k_end;
    kv_split_range(fused ? pos : pos + 1, S, s, k_begin, k_end);
    const int nk = k_end - k_begin;
    const int ntiles = (nk + kKvTileRows - 1) / kKvTileRows;
    const bool has_new = fused && s == S - 1;
    KvPos kp;
    kp.slot = (int)(c->kv_cons & 0xffu);
    kp.phase = (c->kv_cons >> 8) & 1u;

    // Fused mode reads only cache rows below pos, which nothing in this launch writes: the tiles
    // stream while this instruction waits for its dependencies.  Unfused mode waits first and tells
    // the producer warp.
    if (!fused) {
        if (wait_deps(p, c, nwait, wait_off, seq)) return;
        if (t == 0) mbar_arrive(&c->kv_go);
    }
    // rope table row of pos: the chunks q4 and q4 + 4 of cos and sin
    float cs[16], sn[16];
    if (fused) {
        const __nv_bfloat16* cr = reinterpret_cast<const __nv_bfloat16*>(op->ptr[7]) + (long long)pos * op->ld[7];
        const __nv_bfloat16* sr = reinterpret_cast<const __nv_bfloat16*>(op->ptr[8]) + (long long)pos * op->ld[8];
        load8(cr, q4 * 8, 0, cs); load8(cr, 32 + q4 * 8, 0, cs + 8);
        load8(sr, q4 * 8, 0, sn); load8(sr, 32 + q4 * 8, 0, sn + 8);
    }
    if (fused && wait_deps(p, c, nwait, wait_off, seq)) return;
    if (t == 0 && p.trace_cap > 0) c->t_dep = (long long)globaltimer();

    // ---- q of head (warp, g): chunks q4 and q4 + 4, rotated at pos when fused, scaled into the log2
    // domain, split into bf16 high and low parts = the A fragments of the four k-steps ----
    uint32_t qa[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) qa[i][e] = 0u;
    float s_new = NEG_INF;                                            // score of the new token (fused, last split)
    uint32_t vnew[8];                                                 // its v, dims 16 q4 .. 16 q4 + 15, as bf16 pairs
#pragma unroll
    for (int i = 0; i < 8; ++i) vnew[i] = 0u;
    if (hrow) {
        const float qscale = op->f[0] * kLog2e;
        float x[16];
        const long long e0 = (long long)b * op->ld[0] + (warp * G + g) * D;
        load8(reinterpret_cast<const void*>(op->ptr[0]), e0 + q4 * 8, qdt, x);
        load8(reinterpret_cast<const void*>(op->ptr[0]), e0 + 32 + q4 * 8, qdt, x + 8);
        float y[16];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            y[e] = fused ? x[e] * cs[e] - x[8 + e] * sn[e] : x[e];
            y[8 + e] = fused ? x[8 + e] * cs[8 + e] + x[e] * sn[8 + e] : x[8 + e];
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) y[e] *= qscale;
        // k-step i covers chunk (i >> 1) words 2 (i & 1), 2 (i & 1) + 1: k = 2 q4 + j <-> y[8 (i >> 1) + 4 (i & 1) + j],
        // k = 2 q4 + 8 + j <-> y[... + 2 + j]
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float* v = y + 8 * (i >> 1) + 4 * (i & 1);
            const float h0 = round_bf16(v[0]), h1 = round_bf16(v[1]), h2 = round_bf16(v[2]), h3 = round_bf16(v[3]);
            qa[i][0] = pack2(h0, h1);
            qa[i][1] = pack2(v[0] - h0, v[1] - h1);
            qa[i][2] = pack2(h2, h3);
            qa[i][3] = pack2(v[2] - h2, v[3] - h3);
        }
        if (has_new) {
            // the new token: rotated k (rounded to the cache's bf16) scored against this head's q; k and v appended
            float kx[16], kr[16];
            const long long k0 = (long long)b * op->ld[5] + warp * D, v0 = (long long)b * op->ld[6] + warp * D;
            load8(reinterpret_cast<const void*>(op->ptr[5]), k0 + q4 * 8, qdt, kx);
            load8(reinterpret_cast<const void*>(op->ptr[5]), k0 + 32 + q4 * 8, qdt, kx + 8);
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                kr[e] = round_bf16(kx[e] * cs[e] - kx[8 + e] * sn[e]);
                kr[8 + e] = round_bf16(kx[8 + e] * cs[8 + e] + kx[e] * sn[8 + e]);
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) dot = fmaf(y[e], kr[e], dot);
            s_new = dot;
            float vx[16];
            load8(reinterpret_cast<const void*>(op->ptr[6]), v0 + q4 * 16, qdt, vx);
            load8(reinterpret_cast<const void*>(op->ptr[6]), v0 + q4 * 16 + 8, qdt, vx + 8);
#pragma unroll
            for (int i = 0; i < 8; ++i) vnew[i] = pack2(vx[2 * i], vx[2 * i + 1]);
            if (g == 0) {                                             // one lane group per head appends
                const long long row = (long long)b * L + pos;
                __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(op->ptr[1]);
                __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(op->ptr[2]);
                store8(kc, row * op->ld[1] + warp * D + q4 * 8, 0, kr);
                store8(kc, row * op->ld[1] + warp * D + 32 + q4 * 8, 0, kr + 8);
                *reinterpret_cast<uint4*>(vc + row * op->ld[2] + warp * D + q4 * 16) = make_uint4(vnew[0], vnew[1], vnew[2], vnew[3]);
                *reinterpret_cast<uint4*>(vc + row * op->ld[2] + warp * D + q4 * 16 + 8) = make_uint4(vnew[4], vnew[5], vnew[6], vnew[7]);
            }
        }
    }
    if (has_new) {                                                    // the four lanes of a row hold partial dots
        s_new += __shfl_xor_sync(0xffffffffu, s_new, 1);
        s_new += __shfl_xor_sync(0xffffffffu, s_new, 2);
        if (!hrow) s_new = NEG_INF;
    }

    // ---- main loop over the split's tiles ----
    float oacc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
    float mrow = NEG_INF, lrow = 0.f;
    // byte offsets inside a slot.  K: key n = g of block 0 is tile row 4 (g >> 1) + (g & 1), of block 1 two rows further
    const int krow = 4 * (g >> 1) + (g & 1);
    const uint32_t k_off = (uint32_t)((krow >> 2) * (kKvGroupRows * rb + kKvGroupSkew) + (krow & 3) * rb + warp * (D * 2));
    const uint32_t k_first = (uint32_t)((q4 + 4 * (g & 1)) * 16), k_second = (uint32_t)((q4 + 4 * ((g & 1) ^ 1)) * 16);
    // V: rows 4 q4 .. 4 q4 + 3 (group q4), chunk g
    const uint32_t v_off = (uint32_t)(q4 * (kKvGroupRows * rb + kKvGroupSkew) + warp * (D * 2) + g * 16);
    const uint32_t work_s = smem_u32(ring);
    bool ok = true;
#pragma unroll 1
    for (int tile = 0; tile < ntiles; ++tile) {
        // ---- K tile: S = Q K^T ----
        ok = wait_barrier(p, c, &c->kv_full[kp.slot], kp.phase, seq, WHERE_RING_FULL) && ok;
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
        if (ok && head) {
            const uint32_t base = work_s + kp.slot * kKvSlotBytes + k_off;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint4 a = kv_lds128(base + j * 2 * rb + k_first), bq = kv_lds128(base + j * 2 * rb + k_second);
                const bool odd = g & 1;
                const uint4 lo = odd ? bq : a, hi = odd ? a : bq;    // chunk q4, chunk q4 + 4
                mma_bf16(sc[j], qa[0], lo.x, lo.y);
                mma_bf16(sc[j], qa[1], lo.z, lo.w);
                mma_bf16(sc[j], qa[2], hi.x, hi.y);
                mma_bf16(sc[j], qa[3], hi.z, hi.w);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->kv_empty[kp.slot]);
        kp.advance();
        // ---- online softmax over the tile's 16 keys: this lane has rows 4 q4 .. 4 q4 + 3 of head g ----
        uint32_t pa[4] = {0u, 0u, 0u, 0u};
        float alpha = 1.f;
        if (head) {
            const int key0 = tile * kKvTileRows + 4 * q4;             // relative to the split
            float mx = NEG_INF;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + 2 * j + e;
                    sc[j][e] = key >= nk ? NEG_INF : sc[j][e] + sc[j][e + 2];
                    mx = fmaxf(mx, sc[j][e]);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mnew = fmaxf(mrow, mx);                       // finite: a tile has at least one key of the split
            alpha = mrow == NEG_INF ? 0.f : ex2(mrow - mnew);
            mrow = mnew;
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float p0 = sc[j][0] == NEG_INF ? 0.f : ex2(sc[j][0] - mnew);
                const float p1 = sc[j][1] == NEG_INF ? 0.f : ex2(sc[j][1] - mnew);
                sum += p0 + p1;
                const float h0 = round_bf16(p0), h1 = round_bf16(p1);
                pa[j * 2] = pack2(h0, h1);
                pa[j * 2 + 1] = pack2(p0 - h0, p1 - h1);
            }
            lrow = lrow * alpha + sum;
        }
        // ---- V tile: O += P V ----
        ok = wait_barrier(p, c, &c->kv_full[kp.slot], kp.phase, seq, WHERE_RING_FULL) && ok;
        if (ok && head) {
            const uint32_t base = work_s + kp.slot * kKvSlotBytes + v_off;
            const uint4 r0 = kv_lds128(base), r1 = kv_lds128(base + rb), r2 = kv_lds128(base + 2 * rb), r3 = kv_lds128(base + 3 * rb);
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) oacc[j][e] *= alpha;
            const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w}, w1[4] = {r1.x, r1.y, r1.z, r1.w};
            const uint32_t w2[4] = {r2.x, r2.y, r2.z, r2.w}, w3[4] = {r3.x, r3.y, r3.z, r3.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {                             // word u: dims 8 g + 2u (low half), 8 g + 2u + 1 (high half)
                mma_bf16(oacc[2 * u], pa, prmt(w0[u], w1[u], 0x5410u), prmt(w2[u], w3[u], 0x5410u));
                mma_bf16(oacc[2 * u + 1], pa, prmt(w0[u], w1[u], 0x7632u), prmt(w2[u], w3[u], 0x7632u));
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->kv_empty[kp.slot]);
        kp.advance();
    }
    if (t == 0) c->kv_cons = (uint32_t)kp.slot | (kp.phase << 8);     // (read again behind the barrier that ends the instruction)
    phase_mark(p, c, 0);
    // (a failed wait has raised the CTA's abort flag; the code below then writes meaningless values to
    // valid addresses and publish() ends the instruction without arrivals -- no thread leaves early,
    // so every thread passes the same barriers)

    // ---- this split's result for (head warp, query head g): 16 consecutive dims 16 q4 .. per lane ----
    lrow += __shfl_xor_sync(0xffffffffu, lrow, 1);
    lrow += __shfl_xor_sync(0xffffffffu, lrow, 2);
    float o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {                                     // high-part rows + low-part rows
        o[j] = oacc[j][0] + oacc[j][2];
        o[8 + j] = oacc[j][1] + oacc[j][3];
    }
    if (has_new && hrow) {
        const float mnew = fmaxf(mrow, s_new);
        const float a = mrow == NEG_INF ? 0.f : ex2(mrow - mnew), pn = ex2(s_new - mnew);
        lrow = lrow * a + pn;
        mrow = mnew;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[2 * i] = fmaf(pn, bf16_lo(vnew[i]), o[2 * i] * a);
            o[2 * i + 1] = fmaf(pn, bf16_hi(vnew[i]), o[2 * i + 1] * a);
        }
    }
    const int GD = G * D;
    // every split of the sequence has read q (and the one with the new token k_new, v_new) by the
    // time one of them writes the sequence's output
    auto zero_inputs = [&]() {
        if (!op->i[9]) return;
        float* qz = reinterpret_cast<float*>(op->ptr[0]) + (long long)b * op->ld[0];
        for (int i = t; i < H * D; i += kComputeThreads) qz[i] = 0.f;
        for (int i = t; i < 2 * KVH * D; i += kComputeThreads) {
            const int which = i / (KVH * D);
            reinterpret_cast<float*>(op->ptr[5 + which])[(long long)b * op->ld[5 + which] + i % (KVH * D)] = 0.f;
        }
    };
    void* outp = reinterpret_cast<void*>(op->ptr[4]);
    const long long oe = (long long)b * op->ld[4] + (warp * G + g) * D + q4 * 16;
    if (S == 1) {
        if (hrow) {
            const float inv = lrow == 0.f ? 0.f : rcp(lrow);
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] *= inv;
            store8(outp, oe, odt, o);
            store8(outp, oe + 8, odt, o + 8);
        }
        zero_inputs();
        return;
    }
    float* part = reinterpret_cast<float*>(op->ptr[9]);
    const long long ldp = op->ld[9];
    if (hrow) {
        float* mine = part + ((long long)(b * KVH + warp) * S + s) * ldp;
#pragma unroll
        for (int e = 0; e < 16; e += 4)
            *reinterpret_cast<float4*>(mine + g * D + q4 * 16 + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
        if (q4 == 0) { mine[GD + g] = mrow; mine[GD + G + g] = lrow; }
    }
    __threadfence();
    compute_sync();
    phase_mark(p, c, 1);
    int* count = reinterpret_cast<int*>(op->ptr[10]) + (long long)(b * KVH) * op->ld[10];
    if (t == 0) {
        const int old = atomicAdd(count, 1);
        c->flag = (old == S - 1);
        if (old == S - 1) *count = 0;          // back to zero for the next launch
    }
    compute_sync();
    phase_mark(p, c, 2);
    if (!c->flag) return;
    __threadfence();
    // ---- last split to arrive: merge the S partials of every head (warp w: head w), straight from L2.
    // The loads of different splits are independent of each other: the loops are unrolled and free of
    // branches so that many are in flight at once (one split per L2 round trip costs ~1 us each). ----
    if (hrow) {
        const float* base = part + (long long)(b * KVH + warp) * S * ldp;
        float mx = NEG_INF;
#pragma unroll 8
        for (int k = 0; k < S; ++k) mx = fmaxf(mx, __ldcg(base + k * ldp + GD + g));
        float acc[16], l = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = 0.f;
#pragma unroll 4
        for (int k = 0; k < S; ++k) {
            const float mk_ = __ldcg(base + k * ldp + GD + g);
            const float lk = __ldcg(base + k * ldp + GD + G + g);
            float4 v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = __ldcg(reinterpret_cast<const float4*>(base + k * ldp + g * D + q4 * 16 + 4 * e));
            const float w = mk_ == NEG_INF ? 0.f : ex2(mk_ - mx);        // (a split without keys wrote zeros)
            l = fmaf(w, lk, l);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[4 * e] = fmaf(w, v[e].x, acc[4 * e]); acc[4 * e + 1] = fmaf(w, v[e].y, acc[4 * e + 1]);
                acc[4 * e + 2] = fmaf(w, v[e].z, acc[4 * e + 2]); acc[4 * e + 3] = fmaf(w, v[e].w, acc[4 * e + 3]);
            }
        }
        const float inv = l == 0.f ? 0.f : rcp(l);
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] *= inv;
        store8(outp, oe, odt, acc);
        store8(outp, oe + 8, odt, acc + 8);
    }
    zero_inputs();
}

// Waits for its own dependencies and publishes its own arrivals.  Returns whether the CTA is aborting.
template <int GMAX>
static __device__ __noinline__ bool op_decode_bulk(const Params& p, Ctrl* c, const mk_op_desc* op, int b, int s, uint8_t* ring,
                                                   int nwait, int wait_off, int seq, int narrive, int arrive_off) {
    decode_bulk_body<GMAX>(p, c, op, b, s, ring, nwait, wait_off, seq);
    return publish(p, c, narrive, arrive_off);
}

}  // namespace mk
