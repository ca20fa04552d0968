// MK_OP_ATTENTION on the 5th-generation tensor cores (tcgen05 + tensor memory), head_dim 64.
// One instruction = (batch b, head h, 128-query tile), as the mma.sync body (op_attention.cuh); the host
// library selects this body by attaching three tensor maps (q, k, v: {columns, rows} bf16, boxes of 64
// columns x 128 rows, 128-byte swizzle, zero fill) through ptr 11.
//
//   S = Q K_j^T      tcgen05.mma 128 x 128 x 16 (x 4 for head_dim 64): Q and the 128-key tile K_j are K-major
//                    operands in shared memory; S lives in tensor memory, columns 0..127, fp32
//   softmax          four warps, one thread per query row (a tensor-memory lane is a query row, so a row's
//                    maximum and sum need no exchange between threads): log2 domain, scale * log2(e)
//                    applied before the maximum; P rounded to bf16 and written to shared memory as the
//                    K-major A operand of the second product.  The running maximum is only raised when it
//                    grows by more than 2^8 (the reference's lazy rescale, megacute/ops/attention.py:37,
//                    252-262): then the row's sum and its O row in tensor memory are scaled down
//   O += P V_j       tcgen05.mma 128 x 64 x 16 (x 8 for 128 keys): V_j as loaded ([key][64 dims], dims
//                    contiguous) is the MN-major B operand; O lives in tensor memory, columns 128..191
//   out = O / l      read back with tcgen05.ld, one row per thread; a fully masked row yields 0
//
// Roles inside the compute warps: one thread requests the tiles (Q once; K_j into two buffers, V_j into one,
// each refilled as soon as the product that read it has completed), one thread issues the MMAs -- S of
// block j + 1 (two S tiles in tensor memory) ahead of P V of block j, so the tensor core works on the next
// scores while the softmax of this block runs -- and warps 4..7 run the softmax, the rescale and the final
// read-back.  (A first version with single K and S buffers was a chain of latencies -- tile request,
// product, softmax, product -- of ~9 us per block; the mma.sync body was 2.7 x faster.)  The instruction's barriers are
// re-initialised at its start (nothing of the previous instruction is pending: every copy was waited for
// and the last commit of an instruction arrives behind all earlier ones).  Every wait is bounded.
// head_dim 128 and operands the tensor maps cannot describe run the mma.sync body.
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

// All compute threads call this (the instruction's dependencies are met).  Returns 0, or -1 when aborting.
__device__ __forceinline__ int op_attention_tc(const Params& p, Ctrl* c, uint8_t* work, const mk_op_desc* op, int b, int h, int qi,
                                               int seq) {
    constexpr int D = 64;
    constexpr float NEG_INF = -__builtin_huge_valf();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int Sq = op->i[1], Sk = op->i[2], H = op->i[3], KVH = op->i[4], odt = op->i[7];
    const bool causal = op->i[6] != 0, f16 = op->i[8] == DT_F16;
    const int hk = h / (H / KVH);
    const int q0 = qi * 128;
    const int kend = causal ? min(Sk, q0 + 128) : Sk;
    const int nb = (kend + 127) / 128;                                   // 128-key blocks
    const uint8_t* tmaps = reinterpret_cast<const uint8_t*>(op->ptr[11]);
    AttnBars* a = &c->attn;

    // ---- tensor memory (shared with the tile GEMM; allocated once per launch) and this instruction's barriers ----
    if (*(volatile uint32_t*)&c->tmem_base == kTcNoTmem) {
        if (warp == 0)
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&c->tmem_base)), "r"(kTcCols)
                         : "memory");
        tc_fence_before();
    }
    if (t == 0) {
        mbar_init(&a->q_full, 1);
        for (int u = 0; u < 2; ++u) {
            mbar_init(&a->k_full[u], 1); mbar_init(&a->k_empty[u], 1);
            mbar_init(&a->s_full[u], 1); mbar_init(&a->s_empty[u], 4);
        }
        mbar_init(&a->v_full, 1); mbar_init(&a->v_empty, 1);
        mbar_init(&a->p_full, 4); mbar_init(&a->pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    compute_sync();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t*)&c->tmem_base;
    uint8_t* qs = work + kAtQOff;
    uint8_t* ks = work + kAtKOff;
    uint8_t* vs = work + kAtVOff;
    uint8_t* ps = work + kAtPOff;
    int ok = 1;

    // Block j uses K and S buffer j & 1, for the (j >> 1)-th time: a "full" barrier of a buffer is waited with parity
    // (j >> 1) & 1; before the buffer is used again its "empty" barrier is waited with the parity of the previous use.
    if (warp == 0 && lane == 0) {
        // ---- tile requests.  Earlier instructions wrote the work area through the generic proxy. ----
        asm volatile("fence.proxy.async;" ::: "memory");
        const int qrow = b * Sq + q0, krow = b * Sk;
        auto load_k = [&](int j) {
            const int u = j & 1;
            mbar_arrive_expect_tx(&a->k_full[u], (uint32_t)kTcTileBytes);
            tma_load_2d_plain(ks + u * kTcTileBytes, tmaps + 128, hk * D, krow + j * 128, &a->k_full[u]);
        };
        mbar_arrive_expect_tx(&a->q_full, (uint32_t)kTcTileBytes);
        tma_load_2d_plain(qs, tmaps, h * D, qrow, &a->q_full);
        load_k(0);
        if (nb > 1) load_k(1);
        mbar_arrive_expect_tx(&a->v_full, (uint32_t)kTcTileBytes);
        tma_load_2d_plain(vs, tmaps + 256, hk * D, krow, &a->v_full);
        for (int j = 1; j < nb; ++j) {
            if (j + 1 < nb) {                      // K of block j + 1 into the buffer block j - 1 used
                if (!wait_barrier(p, c, &a->k_empty[(j + 1) & 1], (uint32_t)((j - 1) >> 1) & 1u, seq, WHERE_RING_EMPTY)) break;
                load_k(j + 1);
            }
            if (!wait_barrier(p, c, &a->v_empty, (uint32_t)(j - 1) & 1u, seq, WHERE_RING_EMPTY)) break;
            mbar_arrive_expect_tx(&a->v_full, (uint32_t)kTcTileBytes);
            tma_load_2d_plain(vs, tmaps + 256, hk * D, krow + j * 128, &a->v_full);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMAs ----
        bool good = wait_barrier(p, c, &a->q_full, 0u, seq, WHERE_RING_FULL);
        const uint64_t qd = tc_smem_desc(smem_u32(qs));
        // V as MN-major operand: 8-key groups 1024 bytes apart; 16 keys further = 2048 bytes
        const uint64_t vd = tc_smem_desc(smem_u32(vs));
        const uint64_t pd0 = tc_smem_desc(smem_u32(ps)), pd1 = tc_smem_desc(smem_u32(ps + kTcTileBytes));
        const uint32_t idesc_s = at_idesc_s(f16), idesc_o = at_idesc_o(f16);
        auto issue_s = [&](int j) -> bool {        // S of block j into tensor-memory buffer j & 1
            const int u = j & 1;
            if (!wait_barrier(p, c, &a->k_full[u], (uint32_t)(j >> 1) & 1u, seq, WHERE_RING_FULL)) return false;
            if (j >= 2 && !wait_barrier(p, c, &a->s_empty[u], (uint32_t)((j - 2) >> 1) & 1u, seq, WHERE_COMBINE)) return false;
            tc_fence_after();
            const uint64_t kd = tc_smem_desc(smem_u32(ks + u * kTcTileBytes));
#pragma unroll
            for (int k16 = 0; k16 < D / 16; ++k16) tc_mma_i(tmem + kAtSCol + 128 * u, qd + 2 * k16, kd + 2 * k16, idesc_s, k16 ? 1u : 0u);
            tc_commit(&a->k_empty[u]);
            tc_commit(&a->s_full[u]);
            return true;
        };
        good = good && issue_s(0);
        for (int j = 0; j < nb && good; ++j) {
            if (j + 1 < nb) good = issue_s(j + 1);                               // the next block's scores, ahead of this block's P V
            const uint32_t par = (uint32_t)j & 1u;
            good = good && wait_barrier(p, c, &a->p_full, par, seq, WHERE_COMBINE) && wait_barrier(p, c, &a->v_full, par, seq, WHERE_RING_FULL);
            if (!good) break;
            tc_fence_after();
#pragma unroll
            for (int k16 = 0; k16 < 8; ++k16) {
                const uint64_t pd = (k16 < 4 ? pd0 : pd1) + 2 * (k16 & 3);       // 16 keys further inside a 64-key tile: 32 bytes
                tc_mma_i(tmem + kAtOCol, pd, vd + 128 * k16, idesc_o, (j > 0 || k16 > 0) ? 1u : 0u);   // 16 keys of V: 2048 bytes
            }
            tc_commit(&a->v_empty);
            tc_commit(&a->pv_done);
        }
    }
    __syncwarp();

    if (warp >= 4) {
        // ---- softmax, rescale, read-back: thread = query row (tensor-memory lane 32 (warp & 3) + lane) ----
        const int r = (warp & 3) * 32 + lane;
        const int qrow = q0 + r;                                           // position in the sequence
        const uint32_t tl = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const float sl2 = op->f[0] * kLog2e;
        float m_used = NEG_INF, l = 0.f;
        uint8_t* prow = ps + r * 128;                                      // row r of both P tiles
        for (int j = 0; j < nb; ++j) {
            const uint32_t scol = kAtSCol + 128 * (j & 1);
            ok = wait_barrier(p, c, &a->s_full[j & 1], (uint32_t)(j >> 1) & 1u, seq, WHERE_COMBINE) && ok;
            tc_fence_after();
            if (p.trace_cap > 0 && t == 128 && j == 0) c->t_phase[0] = (long long)globaltimer();      // first scores ready
            const int key0 = j * 128;
            const bool edge = key0 + 128 > kend || (causal && key0 + 128 > q0);
            // pass 1: the row's maximum over the block
            float mx = NEG_INF;
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                float s[32];
                tc_ld32(tl + scol + ch * 32, s);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int key = key0 + ch * 32 + e;
                    const bool dead = edge && (key >= kend || (causal && key > qrow));
                    mx = fmaxf(mx, dead ? NEG_INF : s[e] * sl2);
                }
            }
            // lazy rescale: keep the old maximum unless the new one is more than 2^8 above it
            float factor = 1.f;
            if (mx > m_used + kAtRescale || (m_used == NEG_INF && mx != NEG_INF)) {
                factor = m_used == NEG_INF ? 0.f : ex2(m_used - mx);
                m_used = mx;
            }
            // the P buffer and (for a rescale) O are free once the previous block's P V has completed
            if (j > 0) ok = wait_barrier(p, c, &a->pv_done, (uint32_t)(j - 1) & 1u, seq, WHERE_COMBINE) && ok;
            tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                l *= factor;
#pragma unroll 1
                for (int ch = 0; ch < D / 32; ++ch) {
                    float o[32];
                    tc_ld32(tl + kAtOCol + ch * 32, o);
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] *= factor;
                    tc_st32(tl + kAtOCol + ch * 32, o);
                }
            }
            // pass 2: P = 2^(s - m), rounded to bf16, into the swizzled K-major tiles; row sum
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                float s[32];
                tc_ld32(tl + scol + ch * 32, s);
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float pv[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int key = key0 + ch * 32 + e + u;
                        const bool dead = (edge && (key >= kend || (causal && key > qrow))) || m_used == NEG_INF;
                        const float pe = dead ? 0.f : ex2(s[e + u] * sl2 - m_used);
                        pv[u] = f16 ? round_f16(pe) : round_bf16(pe);
                        l += pv[u];
                    }
                    pk[e >> 1] = f16 ? pack2h(pv[0], pv[1]) : pack2(pv[0], pv[1]);
                }
                // 32 keys = 64 bytes = four 16-byte chunks of tile (ch >> 1), chunk index 4 (ch & 1) + q, swizzled with the row
                uint8_t* tile = prow + (ch >> 1) * kTcTileBytes;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<uint4*>(tile + ((((ch & 1) * 4 + q) ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            }
            // S has been read (the next block's S may overwrite it); P is in shared memory for the tensor core
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&a->s_empty[j & 1]);
                mbar_arrive(&a->p_full);
            }
        }
        if (p.trace_cap > 0 && t == 128) c->t_phase[1] = (long long)globaltimer();                    // last P handed over
        // ---- out = O / l ----
        if (nb > 0) ok = wait_barrier(p, c, &a->pv_done, (uint32_t)(nb - 1) & 1u, seq, WHERE_COMBINE) && ok;
        tc_fence_after();
        const float inv = l == 0.f ? 0.f : rcp(l);
        __nv_bfloat16* O = reinterpret_cast<__nv_bfloat16*>(op->ptr[3]) + ((long long)b * Sq + qrow) * op->ld[3] + h * D;
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
            float o[32];
            if (nb > 0) {
                tc_ld32(tl + kAtOCol + ch * 32, o);
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = 0.f;
            }
            if (ok && qrow < Sq) {
#pragma unroll
                for (int e = 0; e < 32; e += 8)
                    *reinterpret_cast<uint4*>(O + ch * 32 + e) =
                        make_uint4(pack2t(odt, o[e] * inv, o[e + 1] * inv), pack2t(odt, o[e + 2] * inv, o[e + 3] * inv),
                                   pack2t(odt, o[e + 4] * inv, o[e + 5] * inv), pack2t(odt, o[e + 6] * inv, o[e + 7] * inv));
            }
        }
    }
    tc_fence_before();
    const bool aborting = compute_sync_or(!ok || *(volatile int*)&c->abort);
    phase_mark(p, c, 2);                                                                               // output written
    return aborting ? -1 : 0;
}

}  // namespace mk
