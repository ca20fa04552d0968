// MK_OP_ATTENTION on the 5th-generation tensor cores (tcgen05 + tensor memory), head_dim 64.
// One instruction = (batch b, head h, 128-query tile), as the mma.sync body (op_attention.cuh); the host
// library selects this body by attaching three tensor maps (q, k, v: {columns, rows} bf16, boxes of 64
// columns x 128 rows, 128-byte swizzle, zero fill) through ptr 11.
//
//   S = Q K_j^T      tcgen05.mma 128 x 128 x 16 (x 4 for head_dim 64): Q and the 128-key tile K_j are K-major
//                    operands in shared memory; S lives in tensor memory, columns 0..127, fp32
//   softmax          all eight compute warps, two threads per query row: a tensor-memory lane is a query row and a
//                    warp reaches the 32 lanes of its quarter (warp & 3), so warps w and w + 4 share 32 rows and take
//                    64 of the block's 128 score columns each (read from tensor memory once for the maximum and once
//                    for the exponentials, 32 at a time: 64 held at once spill under the kernel's register cap).  The two threads of a row agree on the maximum
//                    through shared memory (bf16 values: any common reference near the maximum will do, see the
//                    lazy rescale) and add their partial row sums at the end.  Log2 domain, scale * log2(e) folded
//                    into the subtraction; P rounded to the operand type and written to shared memory as the
//                    K-major A operand of the second product (a thread's 64 keys are one 128-byte row of one tile).
//                    The running maximum is only raised when it grows by more than 2^8 (the reference's lazy
//                    rescale, megacute/ops/attention.py:37,252-262): then the row's sum and its O row in tensor
//                    memory are scaled down.  (One thread per row, four warps: one warp per scheduler, issue-active
//                    18 %, 8.8 us per 128-key block against 0.4 us of MMA; the mma.sync body took 4.3 us.)
//   O += P V_j       tcgen05.mma 128 x 64 x 16 (x 8 for 128 keys): V_j as loaded ([key][64 dims], dims
//                    contiguous) is the MN-major B operand; O lives in tensor memory, columns 256..319
//   out = O / l      read back with tcgen05.ld, half a row per thread; a fully masked row yields 0
//
// Tile requests and MMA issue are ONE thread of the feeder warp (mk_attention_feeder walks the CTA's instruction list
// for these ops): it polls the barriers without blocking (mbarrier.test_wait costs ~1 ns) and does
// whatever is possible next -- K_j into two buffers, V_j into one, each refilled as soon as the product that read
// it has completed; S of block j + 1 (two S tiles in tensor memory) ahead of P V of block j, so the tensor core works
// on the next scores while the softmax of this block runs.  The compute warps tell it through `attn_go` that the
// instruction's dependencies are met and its barriers initialised (nothing of the previous instruction is pending:
// every copy was waited for and the last commit of an instruction arrives behind all earlier ones).  Every wait is
// bounded.  head_dim 128 and operands the tensor maps cannot describe run the mma.sync body.
//
// ptr 0 q, 1 k, 2 v, 3 out, 11 tensor maps; i 0 batch, 1 seq_q, 2 seq_k, 3 heads, 4 kv_heads, 5 head_dim,
// 6 causal, 7 out dtype, 8 dtype of q, k, v; f 0 scale.  args: 0 b, 1 h, 2 query tile.
#pragma once
#include "mk_device.cuh"
#include "op_gemm_tc.cuh"

namespace mk {

constexpr int kAtQOff = kTcXOff;                              // shared-memory map of the work area (1024-byte aligned tiles)
constexpr int kAtKOff = kAtQOff + kTcTileBytes;               // two K buffers
constexpr int kAtVOff = kAtKOff + 2 * kTcTileBytes;
constexpr int kAtPOff = kAtVOff + kTcTileBytes;               // P: two 128 x 64 K-major tiles (keys 0..63, 64..127)
static_assert(kAtPOff + 2 * kTcTileBytes <= kWorkBytes, "attention tiles exceed the work area");
constexpr uint32_t kAtSCol = 0, kAtOCol = 256;                // tensor-memory columns: S buffers at 0 and 128, O at 256
static_assert(kAtOCol + 64 <= kTcCols, "attention accumulators exceed the tensor memory held");
constexpr float kAtRescale = 8.0f;                            // raise the running maximum only past 2^8

// instruction descriptors, kind::f16, fp32 accumulator, M = 128; operand format bits 7-9 / 10-12: 1 = bf16, 0 = fp16
// (q, k, v -- and with them P -- are bf16, or fp16 when they are runtime-private activations)
__device__ __forceinline__ uint32_t at_idesc_s(bool f16) {      // N = 128, A and B K-major
    const uint32_t f = f16 ? 0u : 1u;
    return (1u << 4) | (f << 7) | (f << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ uint32_t at_idesc_o(bool f16) {      // N = 64, B MN-major
    const uint32_t f = f16 ? 0u : 1u;
    return (1u << 4) | (f << 7) | (f << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
}

// 2-D tiled bulk tensor copy global -> shared without a cache hint
__device__ __forceinline__ void tma_load_2d_plain(void* dst, const void* tmap, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// 32 consecutive fp32 columns of this thread's lane, tensor memory <- registers
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n\t"
        "tcgen05.wait::st.sync.aligned;" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tc_mma_i(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// barrier of the two warps (w, w + 4) that share the query rows of tensor-memory quarter q
__device__ __forceinline__ void at_pair_sync(int q) { asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory"); }

// Tile requests and MMA issue of one instruction: one thread of the feeder warp.  Returns false when aborting.
__device__ __forceinline__ bool attention_tc_feed(const Params& p, Ctrl* c, uint8_t* work, const mk_op_desc* op, int b, int h, int qi,
                                                  int seq, uint32_t go_parity) {
    constexpr int D = 64;
    const int Sq = op->i[1], Sk = op->i[2], H = op->i[3], KVH = op->i[4];
    const bool causal = op->i[6] != 0, f16 = op->i[8] == DT_F16;
    const int hk = h / (H / KVH);
    const int q0 = qi * 128;
    const int kend = causal ? min(Sk, q0 + 128) : Sk;
    const int nb = (kend + 127) / 128;
    const uint8_t* tmaps = reinterpret_cast<const uint8_t*>(op->ptr[11]);
    AttnBars* a = &c->attn;
    // the compute warps have met the dependencies, initialised the barriers and (first time) allocated tensor memory;
    // they may be busy with earlier instructions for a long time: twice the time limit, so that a stuck wait there reports first
    if (!wait_barrier(p, c, &c->attn_go, go_parity, seq, WHERE_DEP, 2)) return false;
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t*)&c->tmem_base;
    uint8_t* qs = work + kAtQOff;
    uint8_t* ks = work + kAtKOff;
    uint8_t* vs = work + kAtVOff;
    uint8_t* ps = work + kAtPOff;
    // earlier instructions wrote the work area through the generic proxy
    asm volatile("fence.proxy.async;" ::: "memory");
    const int qrow = b * Sq + q0, krow = b * Sk;
    mbar_arrive_expect_tx(&a->q_full, (uint32_t)kTcTileBytes);
    tma_load_2d_plain(qs, tmaps, h * D, qrow, &a->q_full);
    const uint64_t qd = tc_smem_desc(smem_u32(qs));
    const uint64_t vd = tc_smem_desc(smem_u32(vs));       // V as MN-major operand: 8-key groups 1024 bytes apart; 16 keys further = 2048 bytes
    const uint64_t pd0 = tc_smem_desc(smem_u32(ps)), pd1 = tc_smem_desc(smem_u32(ps + kTcTileBytes));
    const uint32_t idesc_s = at_idesc_s(f16), idesc_o = at_idesc_o(f16);
    // Block j uses K and S buffer j & 1, for the (j >> 1)-th time: a "full" barrier of a buffer completes with parity
    // (j >> 1) & 1; before the buffer is used again its "empty" barrier must have completed with the parity of the previous use.
    int kl = 0, vl = 0, si = 0, pi = 0;                   // K tiles requested, V tiles requested, S products issued, P V products issued
    bool q_ready = false;
    uint32_t idle = 0;
    unsigned long long t0 = 0;
    while (pi < nb) {
        bool progress = false;
        if (kl < nb && (kl < 2 || mbar_test_wait(&a->k_empty[kl & 1], (uint32_t)((kl - 2) >> 1) & 1u))) {
            const int u = kl & 1;
            mbar_arrive_expect_tx(&a->k_full[u], (uint32_t)kTcTileBytes);
            tma_load_2d_plain(ks + u * kTcTileBytes, tmaps + 128, hk * D, krow + kl * 128, &a->k_full[u]);
            ++kl;
            progress = true;
        }
        if (vl < nb && (vl == 0 || mbar_test_wait(&a->v_empty, (uint32_t)(vl - 1) & 1u))) {
            mbar_arrive_expect_tx(&a->v_full, (uint32_t)kTcTileBytes);
            tma_load_2d_plain(vs, tmaps + 256, hk * D, krow + vl * 128, &a->v_full);
            ++vl;
            progress = true;
        }
        if (!q_ready) q_ready = mbar_test_wait(&a->q_full, 0u);
        // S of block si (at most one block ahead of the P V products), into tensor-memory buffer si & 1
        if (q_ready && si < nb && si <= pi + 1 && si < kl && mbar_test_wait(&a->k_full[si & 1], (uint32_t)(si >> 1) & 1u) &&
            (si < 2 || mbar_test_wait(&a->s_empty[si & 1], (uint32_t)((si - 2) >> 1) & 1u))) {
            const int u = si & 1;
            tc_fence_after();
            const uint64_t kd = tc_smem_desc(smem_u32(ks + u * kTcTileBytes));
#pragma unroll
            for (int k16 = 0; k16 < D / 16; ++k16) tc_mma_i(tmem + kAtSCol + 128 * u, qd + 2 * k16, kd + 2 * k16, idesc_s, k16 ? 1u : 0u);
            tc_commit(&a->k_empty[u]);
            tc_commit(&a->s_full[u]);
            ++si;
            progress = true;
        }
        if (pi < si && pi < vl && mbar_test_wait(&a->p_full, (uint32_t)pi & 1u) && mbar_test_wait(&a->v_full, (uint32_t)pi & 1u)) {
            tc_fence_after();
#pragma unroll
            for (int k16 = 0; k16 < 8; ++k16) {
                const uint64_t pd = (k16 < 4 ? pd0 : pd1) + 2 * (k16 & 3);       // 16 keys further inside a 64-key tile: 32 bytes
                tc_mma_i(tmem + kAtOCol, pd, vd + 128 * k16, idesc_o, (pi > 0 || k16 > 0) ? 1u : 0u);   // 16 keys of V: 2048 bytes
            }
            tc_commit(&a->v_empty);
            tc_commit(&a->pv_done);
            ++pi;
            progress = true;
        }
        if (progress) { idle = 0; t0 = 0; continue; }
        if ((++idle & 1023u) == 0) {                       // nothing to do: the time limit of every other wait applies
            if (*(volatile int*)&c->abort) return false;
            if (ld_volatile(&p.status[MK_ST_CODE]) != 0) { c->abort = 1; return false; }
            const unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.timeout_ns) {
                report(p, c, MK_DEV_TIMEOUT_BARRIER, seq, WHERE_RING_FULL, (int)(&a->p_full - c->full), pi, si);
                return false;
            }
        }
    }
    return true;
}

// All compute threads call this (the instruction's dependencies are met).  Returns 0, or -1 when aborting.
__device__ __forceinline__ int op_attention_tc(const Params& p, Ctrl* c, uint8_t* work, const mk_op_desc* op, int b, int h, int qi,
                                               int seq) {
    constexpr int D = 64;
    constexpr float NEG_INF = -__builtin_huge_valf();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int Sq = op->i[1], Sk = op->i[2], odt = op->i[7];
    const bool causal = op->i[6] != 0, f16 = op->i[8] == DT_F16;
    const int q0 = qi * 128;
    const int kend = causal ? min(Sk, q0 + 128) : Sk;
    const int nb = (kend + 127) / 128;                                   // 128-key blocks
    AttnBars* a = &c->attn;

    // ---- tensor memory (shared with the tile GEMM; allocated once per launch) and this instruction's barriers ----
    const bool first_use = *(volatile uint32_t*)&c->tmem_ready == 0;     // (written behind the barrier below: the same for every thread)
    if (first_use) {
        if (warp == 0) {
            __syncwarp();          // (.sync.aligned: the whole warp, converged)
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&c->tmem_base)), "r"(kTcCols)
                         : "memory");
        }
        tc_fence_before();
    }
    if (t == 0) {
        mbar_init(&a->q_full, 1);
        for (int u = 0; u < 2; ++u) {
            mbar_init(&a->k_full[u], 1); mbar_init(&a->k_empty[u], 1);
            mbar_init(&a->s_full[u], 1); mbar_init(&a->s_empty[u], kComputeWarps);
        }
        mbar_init(&a->v_full, 1); mbar_init(&a->v_empty, 1);
        mbar_init(&a->p_full, kComputeWarps); mbar_init(&a->pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    compute_sync();
    tc_fence_after();
    if (t == 0 && first_use) c->tmem_ready = 1;
    if (t == 0) mbar_arrive(&c->attn_go);                               // the feeding thread (feeder warp) may start
    const uint32_t tmem = *(volatile uint32_t*)&c->tmem_base;
    uint8_t* ps = work + kAtPOff;
    __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(work);          // 512 bytes in front of the tiles: 2 x 128 row maxima (bf16),
    float* xf = reinterpret_cast<float*>(work);                          // at the end 128 partial row sums
    int ok = 1;

    // ---- softmax, rescale, read-back: thread = (query row r, column half) ----
    const int qd = warp & 3, half = warp >> 2;
    const int r = qd * 32 + lane;
    const int qrow = q0 + r;                                             // position in the sequence
    const uint32_t tl = tmem + ((uint32_t)(qd * 32) << 16);
    const float sl2 = op->f[0] * kLog2e;
    float m_used = NEG_INF, l = 0.f;
    uint8_t* prow = ps + half * kTcTileBytes + r * 128;                  // this thread's 64 keys: row r of P tile `half`
    for (int j = 0; j < nb; ++j) {
        const int u = j & 1;
        ok = wait_barrier(p, c, &a->s_full[u], (uint32_t)(j >> 1) & 1u, seq, WHERE_COMBINE) && ok;
        tc_fence_after();
        if (p.trace_cap > 0 && t == 0 && j == 0) c->t_phase[0] = (long long)globaltimer();      // first scores ready
        // Two passes over the thread's 64 scores, 32 at a time (held all at once they do not fit the kernel's
        // 168-register cap beside the exponentials: 80 registers spilled).  Tensor memory is read twice instead.
        const uint32_t scol = tl + kAtSCol + 128 * u + half * 64;
        const int key0 = j * 128 + half * 64;
        const bool edge = key0 + 64 > kend || (causal && key0 + 64 > q0);      // a block with masked keys: those count as -inf
        float m4[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
            float s[32];
            tc_ld32(scol + ch * 32, s);
            if (edge) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int key = key0 + ch * 32 + e;
                    if (key >= kend || (causal && key > qrow)) s[e] = NEG_INF;
                }
            }
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                m4[0] = fmaxf(m4[0], s[e]); m4[1] = fmaxf(m4[1], s[e + 1]); m4[2] = fmaxf(m4[2], s[e + 2]); m4[3] = fmaxf(m4[3], s[e + 3]);
            }
        }
        // the row's maximum over both halves, as a value both threads of the row compute alike
        const __nv_bfloat16 mine = __float2bfloat16_rn(fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl2);
        xb[half * 128 + r] = mine;
        at_pair_sync(qd);
        const float mx = fmaxf(__bfloat162float(mine), __bfloat162float(xb[(half ^ 1) * 128 + r]));
        at_pair_sync(qd);                                                // (the slot is written again in the next block)
        // lazy rescale: keep the old maximum unless the new one is more than 2^8 above it
        float factor = 1.f;
        if (mx > m_used + kAtRescale || (m_used == NEG_INF && mx != NEG_INF)) {
            factor = m_used == NEG_INF ? 0.f : ex2(m_used - mx);
            m_used = mx;
        }
        // the P buffer and (for a rescale) O are free once the previous block's P V has completed
        if (j > 0) ok = wait_barrier(p, c, &a->pv_done, (uint32_t)(j - 1) & 1u, seq, WHERE_COMBINE) && ok;
        tc_fence_after();
        if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {           // (both warps of a row see the same factors)
            l *= factor;
            float o[32];
            tc_ld32(tl + kAtOCol + half * 32, o);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] *= factor;
            tc_st32(tl + kAtOCol + half * 32, o);
        }
        // P = 2^(s * scale - m), rounded to the operand type, into the swizzled K-major tile; partial row sums
        const float mm = m_used == NEG_INF ? 0.f : m_used;               // (a row without a live key so far: every s is -inf)
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
            float s[32];
            tc_ld32(scol + ch * 32, s);
            if (edge) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int key = key0 + ch * 32 + e;
                    if (key >= kend || (causal && key > qrow)) s[e] = NEG_INF;           // 2^-inf = 0
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {                                // 8 keys = one 16-byte chunk
                float pe[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    pe[e] = ex2(fmaf(s[q * 8 + e], sl2, -mm));
                    l4[e & 3] += pe[e];
                }
                uint4 w;
                if (f16) w = make_uint4(pack2h(pe[0], pe[1]), pack2h(pe[2], pe[3]), pack2h(pe[4], pe[5]), pack2h(pe[6], pe[7]));
                else w = make_uint4(pack2(pe[0], pe[1]), pack2(pe[2], pe[3]), pack2(pe[4], pe[5]), pack2(pe[6], pe[7]));
                *reinterpret_cast<uint4*>(prow + (((ch * 4 + q) ^ (r & 7)) << 4)) = w;
            }
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        // S has been read (the next block's S may overwrite it); P is in shared memory for the tensor core
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&a->s_empty[u]);
            mbar_arrive(&a->p_full);
        }
    }
    if (p.trace_cap > 0 && t == 0) c->t_phase[1] = (long long)globaltimer();                        // last P handed over
    // ---- out = O / l ----
    if (nb > 0) ok = wait_barrier(p, c, &a->pv_done, (uint32_t)(nb - 1) & 1u, seq, WHERE_COMBINE) && ok;
    tc_fence_after();
    if (half == 1) xf[r] = l;
    at_pair_sync(qd);
    if (half == 0) { l += xf[r]; xf[r] = l; }
    at_pair_sync(qd);
    if (half == 1) l = xf[r];
    const float inv = l == 0.f ? 0.f : rcp(l);
    {
        uint8_t* O = reinterpret_cast<uint8_t*>(op->ptr[3]) + (((long long)b * Sq + qrow) * op->ld[3] + h * D + half * 32) * 2;
        float o[32];
        if (nb > 0) {
            tc_ld32(tl + kAtOCol + half * 32, o);
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0.f;
        }
        if (ok && qrow < Sq) {
#pragma unroll
            for (int e = 0; e < 32; e += 8)
                *reinterpret_cast<uint4*>(O + e * 2) =
                    make_uint4(pack2t(odt, o[e] * inv, o[e + 1] * inv), pack2t(odt, o[e + 2] * inv, o[e + 3] * inv),
                               pack2t(odt, o[e + 4] * inv, o[e + 5] * inv), pack2t(odt, o[e + 6] * inv, o[e + 7] * inv));
        }
    }
    tc_fence_before();
    const bool aborting = compute_sync_or(!ok || *(volatile int*)&c->abort);
    phase_mark(p, c, 2);                                                                               // output written
    return aborting ? -1 : 0;
}

}  // namespace mk
