// MK_OP_ATTENTION: prefill flash attention, one instruction = (batch b, head h, 128-query tile).
//   out = softmax(q k^T * scale [+ causal mask]) v,   GQA: query head h reads kv head h / (H / KVH)
// 8 warps x 16 query rows.  K and V stream through a 2-stage cp.async pipeline of 64-key tiles;
// S = Q K^T and O += P V are warp-level mma.sync m16n8k16 bf16 -> fp32 with the online softmax
// kept in registers in the log2 domain; P is rounded to bf16 before P V (as the reference's
// kernel does, megacute/ops/attention.py:293).  A fully masked row yields 0.  This is the
// portable first implementation; the tcgen05 / TMEM version is the planned replacement.
//
// ptr 0 q, 1 k, 2 v, 3 out; i 0 batch, 1 seq_q, 2 seq_k, 3 heads, 4 kv_heads, 5 head_dim,
// 6 causal, 7 out dtype (DT_BF16 or DT_F16), 8 dtype of q, k and v (DT_BF16 or DT_F16); f 0 scale.  args: 0 b, 1 h, 2 query tile.
#pragma once
#include "mk_device.cuh"
#include "mma.cuh"

namespace mk {

constexpr int kAttnBQ = 128, kAttnBK = 64;

// F16: q, k and v (runtime-private activations, see passes.promote_temps) are fp16 instead of bf16; P is then
// rounded to fp16 too, since one MMA takes one operand type.
template <int D, bool F16>
static __device__ __noinline__ void op_attention(const mk_op_desc* op, int a0, int a1, int a2, uint8_t* work) {
    constexpr int ROWB = D * 2 + 16;                       // padded row: conflict-free ldmatrix
    constexpr int KT_BYTES = kAttnBK * ROWB;               // one K or V tile
    constexpr int CPR = D / 8;                             // 16-byte chunks per row
    constexpr float NEG_INF = -__builtin_huge_valf();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int Sq = op->i[1], Sk = op->i[2], H = op->i[3], KVH = op->i[4];
    const bool causal = op->i[6] != 0;
    const int b = a0, h = a1, qi = a2;
    const int hk = h / (H / KVH);
    const float sl2 = op->f[0] * kLog2e;
    const __nv_bfloat16* Q = reinterpret_cast<const __nv_bfloat16*>(op->ptr[0]) + (long long)b * Sq * op->ld[0] + h * D;
    const __nv_bfloat16* Kp = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]) + (long long)b * Sk * op->ld[1] + hk * D;
    const __nv_bfloat16* Vp = reinterpret_cast<const __nv_bfloat16*>(op->ptr[2]) + (long long)b * Sk * op->ld[2] + hk * D;
    __nv_bfloat16* O = reinterpret_cast<__nv_bfloat16*>(op->ptr[3]) + (long long)b * Sq * op->ld[3] + h * D;
    const int q0 = qi * kAttnBQ;
    const int kend = causal ? min(Sk, q0 + kAttnBQ) : Sk;
    const int ntiles = (kend + kAttnBK - 1) / kAttnBK;

    // ---- Q tile -> shared -> A fragments in registers ----
    for (int v = t; v < kAttnBQ * CPR; v += kComputeThreads) {
        const int r = v / CPR, ch = v % CPR;
        const bool ok = q0 + r < Sq;
        cp_async16(work + r * ROWB + ch * 16, Q + (long long)(ok ? q0 + r : q0) * op->ld[0] + ch * 8, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    compute_sync();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(smem_u32(work) + (warp * 16 + (lane & 15)) * ROWB + (kk * 16 + (lane >> 4) * 8) * 2, qf[kk][0],
                    qf[kk][1], qf[kk][2], qf[kk][3]);
    compute_sync();                                         // Q smem is reused by the K/V pipeline

    uint8_t* ks = work;                                     // 2 K tiles then 2 V tiles
    uint8_t* vs = work + 2 * KT_BYTES;
    auto issue = [&](int tile) {
        const int st = tile & 1, key0 = tile * kAttnBK;
        for (int v = t; v < kAttnBK * CPR; v += kComputeThreads) {
            const int r = v / CPR, ch = v % CPR;
            const bool ok = key0 + r < kend;
            const long long row = ok ? key0 + r : 0;
            cp_async16(ks + st * KT_BYTES + r * ROWB + ch * 16, Kp + row * op->ld[1] + ch * 8, ok);
            cp_async16(vs + st * KT_BYTES + r * ROWB + ch * 16, Vp + row * op->ld[2] + ch * 8, ok);
        }
    };

    float oacc[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
    float mrow[2] = {NEG_INF, NEG_INF}, lrow[2] = {0.f, 0.f};
    const int qrow0 = q0 + warp * 16 + (lane >> 2);         // this thread's two query rows: qrow0, qrow0 + 8

    issue(0);
    cp_async_commit();
    for (int tile = 0; tile < ntiles; ++tile) {
        if (tile + 1 < ntiles) issue(tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
        compute_sync();
        const uint32_t kb = smem_u32(ks + (tile & 1) * KT_BYTES), vb = smem_u32(vs + (tile & 1) * KT_BYTES);
        const int key0 = tile * kAttnBK;
        // ---- S = Q K^T (16 x 64 per warp) ----
        float s[kAttnBK / 8][4];
#pragma unroll
        for (int j = 0; j < kAttnBK / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < kAttnBK / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kb + (jp * 16 + (lane & 7) + (lane >> 4) * 8) * ROWB + (kk * 16 + ((lane >> 3) & 1) * 8) * 2,
                            b0, b1, b2, b3);
                if (F16) { mma_f16(s[jp * 2], qf[kk], b0, b1); mma_f16(s[jp * 2 + 1], qf[kk], b2, b3); }
                else { mma_bf16(s[jp * 2], qf[kk], b0, b1); mma_bf16(s[jp * 2 + 1], qf[kk], b2, b3); }
            }
        }
        // ---- mask + online softmax (log2 domain) ----
        const bool edge = (key0 + kAttnBK > kend) || (causal && key0 + kAttnBK > q0 + warp * 16);
        float mx[2] = {NEG_INF, NEG_INF};
#pragma unroll
        for (int j = 0; j < kAttnBK / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * sl2;
                if (edge) {
                    const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    const int qr = qrow0 + (e >> 1) * 8;
                    if (key >= kend || (causal && key > qr)) v = NEG_INF;
                }
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], mnew[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            mnew[r] = fmaxf(mrow[r], mx[r]);
            alpha[r] = (mrow[r] == NEG_INF) ? 0.f : ex2(mrow[r] - mnew[r]);
            mrow[r] = mnew[r];
        }
        float sum[2] = {0.f, 0.f};
        uint32_t pf[kAttnBK / 16][4];
#pragma unroll
        for (int j = 0; j < kAttnBK / 8; ++j) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float m = mnew[e >> 1];
                p[e] = (s[j][e] == NEG_INF || m == NEG_INF) ? 0.f : (F16 ? round_f16(ex2(s[j][e] - m)) : round_bf16(ex2(s[j][e] - m)));
                sum[e >> 1] += p[e];
            }
            pf[j >> 1][(j & 1) * 2] = F16 ? pack2h(p[0], p[1]) : pack2(p[0], p[1]);          // rows r
            pf[j >> 1][(j & 1) * 2 + 1] = F16 ? pack2h(p[2], p[3]) : pack2(p[2], p[3]);      // rows r + 8
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * alpha[r] + sum[r];
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            oacc[j][0] *= alpha[0]; oacc[j][1] *= alpha[0];
            oacc[j][2] *= alpha[1]; oacc[j][3] *= alpha[1];
        }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < kAttnBK / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < D / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vb + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (jp * 16 + (lane >> 4) * 8) * 2,
                                  b0, b1, b2, b3);
                if (F16) { mma_f16(oacc[jp * 2], pf[kk], b0, b1); mma_f16(oacc[jp * 2 + 1], pf[kk], b2, b3); }
                else { mma_bf16(oacc[jp * 2], pf[kk], b0, b1); mma_bf16(oacc[jp * 2 + 1], pf[kk], b2, b3); }
            }
        }
        compute_sync();                                      // the stage is overwritten by the next issue
    }
    cp_async_wait<0>();
    // ---- normalise and store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qr = qrow0 + r * 8;
        if (qr >= Sq) continue;
        const float inv = lrow[r] == 0.f ? 0.f : rcp(lrow[r]);
#pragma unroll
        for (int j = 0; j < D / 8; ++j)
            *reinterpret_cast<uint32_t*>(O + (long long)qr * op->ld[3] + j * 8 + (lane & 3) * 2) =
                pack2t(op->i[7], oacc[j][r * 2] * inv, oacc[j][r * 2 + 1] * inv);
    }
    compute_sync();
}

}  // namespace mk
