// MK_OP_GEMM, warp-level mma.sync body: tiled linear for more than 8 activation rows.
//   out[128 x 128 tile] = act(x @ w^T + bias) + residual        (one instruction per output tile)
//   ws += x[:, Kj] @ w[:, Kj]^T                                  (split-K partial: reduce-add)
// The tcgen05 body (op_gemm_tc.cuh) runs the ops the host library binds to it; this one takes the
// rest: a K range per instruction that is not a multiple of 64, operands not aligned for 16-byte
// accesses, launches whose descriptors the library never saw (mk_launch_noalloc).
// Operands stream through a cp.async pipeline of 32- or 64-wide k-tiles; the math is mma.sync
// m16n8k16 bf16 -> fp32 (8 warps as 2 x 4); with fp16 activations (descriptor i 9) the weight fragments are
// converted to fp16 in registers and the fp16 form of the instruction is used.  Two shapes: 128 activation rows per tile with 4 stages
// (warp tile 64 x 32), and, when the op has at most 64 rows (batched decode, where the op is bound
// by streaming the weights), 64 rows per tile (warp tile 32 x 32): no MMAs on padding rows and more
// weight bytes in flight.
//
// ptr 0 x, 1 w, 2 out (or ws), 3 bias, 4 residual
// i 0 M, 1 N (weight rows), 2 K, 3 act, 4 splits, 5 out dtype, 6 accumulate, 7 residual dtype,
//   8 swiglu (weight tile = 64 gate rows then 64 up rows; the tile writes 64 output columns),
//   9 x dtype (DT_BF16 or DT_F16), 10 weight rows per output tile (128, or 256: the n tile argument then
//   names a pair of 128-row tiles)
// args: 0 m tile, 1 n tile, 2 k split
#pragma once
#include "mk_device.cuh"
#include "mma.cuh"

namespace mk {

constexpr int kGemmBM = 128, kGemmBN = 128;                    // kGemmBM: rows per m tile in the schedule (config.py GEMM_BM)

// BM: activation rows held per tile (128, or 64 when M <= 64); MI = 16-row fragments per warp.
template <int BM, int kGemmBK, int kGemmStages>
static __device__ __noinline__ void op_gemm(const mk_op_desc* op, int a0, int a1, int a2, uint8_t* work) {
    constexpr int kGemmRowBytes = kGemmBK * 2 + 16;            // padded: conflict-free ldmatrix
    constexpr int CPRW = kGemmBK / 8;                          // 16-byte chunks per row
    constexpr int MI = BM / 32;
    constexpr int kATileBytes = BM * kGemmRowBytes, kBTileBytes = kGemmBN * kGemmRowBytes;
    static_assert(kGemmStages * (kATileBytes + kBTileBytes) <= kWorkBytes, "GEMM stages exceed the work area");
    const int M = op->i[0], N = op->i[1], K = op->i[2], act = op->i[3], splits = op->i[4];
    const int odt = op->i[5], accum = op->i[6], rdt = op->i[7], swi = op->i[8];
    const bool xh = op->i[9] == DT_F16;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int wm = warp >> 2, wn = warp & 3;
    const int m0 = a0 * kGemmBM, n0 = a1 * kGemmBN;
    const int kc = K / splits, kbeg = a2 * kc, nk = kc / kGemmBK;
    const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(op->ptr[0]);
    const __nv_bfloat16* Wt = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]);
    const long long ldx = op->ld[0], ldw = op->ld[1];
    uint8_t* sa = work;
    uint8_t* sb = work + kGemmStages * kATileBytes;

    auto issue = [&](int kt) {
        const int st = kt % kGemmStages;
        const int k0 = kbeg + kt * kGemmBK;
#pragma unroll
        for (int i = 0; i < kGemmBN * CPRW / kComputeThreads; ++i) {
            const int v = t + i * kComputeThreads;
            const int r = v / CPRW, ch = v % CPRW;
            if (r < BM) {
                const bool va = m0 + r < M;
                cp_async16(sa + st * kATileBytes + r * kGemmRowBytes + ch * 16,
                           X + (long long)(va ? m0 + r : m0) * ldx + k0 + ch * 8, va);
            }
            const bool vb = n0 + r < N;
            cp_async16(sb + st * kBTileBytes + r * kGemmRowBytes + ch * 16,
                       Wt + (long long)(vb ? n0 + r : n0) * ldw + k0 + ch * 8, vb);
        }
    };

    float acc[MI][4][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < kGemmStages - 1; ++s) {
        if (s < nk) issue(s);
        cp_async_commit();
    }
    // weight-tile row of the first of each pair of n-fragments owned by this warp
    const int brow0 = swi ? wn * 16 : wn * 32, brow1 = swi ? 64 + wn * 16 : wn * 32 + 16;
    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<kGemmStages - 2>();
        compute_sync();
        if (kt + kGemmStages - 1 < nk) issue(kt + kGemmStages - 1);
        cp_async_commit();
        const uint32_t a_base = smem_u32(sa + (kt % kGemmStages) * kATileBytes);
        const uint32_t b_base = smem_u32(sb + (kt % kGemmStages) * kBTileBytes);
#pragma unroll
        for (int kk = 0; kk < kGemmBK / 16; ++kk) {
            uint32_t af[MI][4], bf[4][2];
#pragma unroll
            for (int i = 0; i < MI; ++i)
                ldmatrix_x4(a_base + (wm * (BM / 2) + i * 16 + (lane & 15)) * kGemmRowBytes + (kk * 16 + (lane >> 4) * 8) * 2,
                            af[i][0], af[i][1], af[i][2], af[i][3]);
#pragma unroll
            for (int pr = 0; pr < 2; ++pr) {
                const int row = (pr ? brow1 : brow0) + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(b_base + row * kGemmRowBytes + (kk * 16 + ((lane >> 3) & 1) * 8) * 2, bf[pr * 2][0],
                            bf[pr * 2][1], bf[pr * 2 + 1][0], bf[pr * 2 + 1][1]);
            }
            if (xh) {
#pragma unroll
                for (int j = 0; j < 4; ++j) { bf[j][0] = bf16x2_to_f16x2(bf[j][0]); bf[j][1] = bf16x2_to_f16x2(bf[j][1]); }
#pragma unroll
                for (int i = 0; i < MI; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_f16(acc[i][j], af[i], bf[j][0], bf[j][1]);
            } else {
#pragma unroll
                for (int i = 0; i < MI; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j][0], bf[j][1]);
            }
        }
    }
    cp_async_wait<0>();

    // ---- epilogue: thread holds rows (lane/4, +8) and column pairs 2*(lane%4) of each fragment ----
    const int n_out = swi ? N / 2 : N;
    const int col_base = swi ? a1 * 64 + wn * 16 : n0 + wn * 32;
    void* O = reinterpret_cast<void*>(op->ptr[2]);
    const long long ldo = op->ld[2];
#pragma unroll
    for (int i = 0; i < MI; ++i) {
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int r = m0 + wm * (BM / 2) + i * 16 + (lane >> 2) + hrow * 8;
            if (r >= M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (swi && j >= 2) continue;
                const int col = col_base + j * 8 + (lane & 3) * 2;
                if (col >= n_out) continue;
                float v0 = acc[i][j][hrow * 2], v1 = acc[i][j][hrow * 2 + 1];
                if (swi) {
                    const float u0 = acc[i][j + 2][hrow * 2], u1 = acc[i][j + 2][hrow * 2 + 1];
                    v0 = v0 * sigmoidf_(v0) * u0;
                    v1 = v1 * sigmoidf_(v1) * u1;
                } else if (!accum) {
                    if (op->ptr[3]) {
                        const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(op->ptr[3]);
                        v0 += __bfloat162float(bias[col]);
                        v1 += __bfloat162float(bias[col + 1]);
                    }
                    v0 = apply_act(act, v0);
                    v1 = apply_act(act, v1);
                    if (op->ptr[4]) {
                        const void* R = reinterpret_cast<const void*>(op->ptr[4]);
                        v0 += load1(R, (long long)r * op->ld[4] + col, rdt);
                        v1 += load1(R, (long long)r * op->ld[4] + col + 1, rdt);
                    }
                }
                const long long e = (long long)r * ldo + col;
                if (accum) {
                    if (odt == 1) red_add_f32x2(reinterpret_cast<float*>(O) + e, v0, v1);
                    else red_add_bf16x2(reinterpret_cast<__nv_bfloat16*>(O) + e, v0, v1);
                } else if (odt == 1) {
                    *reinterpret_cast<float2*>(reinterpret_cast<float*>(O) + e) = make_float2(v0, v1);
                } else {
                    *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(O) + e) = pack2t(odt, v0, v1);
                }
            }
        }
    }
    compute_sync();          // the tile buffers are free for the next instruction
}

}  // namespace mk
