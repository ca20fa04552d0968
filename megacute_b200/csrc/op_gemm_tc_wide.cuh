// MK_OP_GEMM on tcgen05 with 128 x 256 output tiles (descriptor i 10 = 256): the body of op_gemm_tc.cuh with two
// accumulator halves of 128 columns in tensor memory.  One activation k-tile feeds two weight tiles, which halves
// the activation bytes per flop: the main loop of a tile GEMM is bound by the operand bytes an SM draws from L2
// (~64 GB/s measured: 0.5 us per 32 KB k-tile of a 128 x 128 tile, 0.75 us per 48 KB of a 128 x 256 one with
// twice the flops).  The two weight tiles of a k-tile travel through the same single-tile ring slots, one after
// the other (the producer warp knows the shape: op_gemv_common.cuh); the epilogue handles the halves in turn,
// each exactly as the narrow tile's.  A body of its own (and a translation unit of its own, op_gemm_wide.cu)
// rather than a parameter of the narrow one: sharing the code cost the narrow tile's main loop spilled registers.
#pragma once
#include "op_gemm_tc.cuh"

namespace mk {

__device__ __forceinline__ int op_gemm_tc_wide(const Params& p, Ctrl* c, uint8_t* ring, uint8_t* work, const mk_op_desc* op, int a0,
                                          int a1, int a2, int seq) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int M = op->i[0], N = op->i[1], K = op->i[2], splits = op->i[4];
    const int swi = op->i[8];
    constexpr int halves = 2;                                             // 128-column accumulator halves of the output tile
    const int m0 = a0 * 128, n0 = a1 * 128 * halves;
    const int kc = K / splits, kbeg = a2 * kc, nk = kc / 64;
    const uint8_t* tmaps = reinterpret_cast<const uint8_t*>(op->ptr[11]);
    uint8_t* xs = work + kTcXOff;
    // activation stages: whole 128-row tiles, or twice as many 64-row half tiles
    const int xbytes = M <= 64 ? kTcTileBytes / 2 : kTcTileBytes;
    const uint32_t xstages = M <= 64 ? kTcXHalfStages : kTcXStages;

    // Tensor memory is allocated by the CTA's first tile GEMM instruction and kept until the kernel
    // ends (the kernel frees it on every path); the permit to allocate is never relinquished.
    // (the test is on a word that only changes behind a barrier, so every thread takes the same branch -- not on the
    // address itself, which the allocation writes while the other warps are still arriving at the test)
    const uint32_t uses = *(volatile uint32_t*)&c->acc_uses;
    if (*(volatile uint32_t*)&c->tmem_ready == 0) {            // (the attention op may have allocated it already)
        if (warp == 0) {
            __syncwarp();          // (.sync.aligned: the whole warp, converged)
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&c->tmem_base)), "r"(kTcCols)
                         : "memory");
        }
        tc_fence_before();
        compute_sync();
        tc_fence_after();
        if (t == 0) c->tmem_ready = 1;                          // (read again only behind the barrier that ends this instruction)
    }
    const uint32_t tmem = *(volatile uint32_t*)&c->tmem_base;
    const uint32_t apar = uses & 1u;

    phase_mark(p, c, 0);
    const uint32_t xpar0 = c->x_par;
    const uint32_t ws0 = c->ww_slot, wph0 = c->ww_phase;
    if (warp == 2 && lane < 2) {
        // ---- activation tiles: {64 K-elements, 128 rows} at (kbeg + 64 kt, m0) ---- (as in the narrow tile)
        asm volatile("fence.proxy.async;" ::: "memory");
        unsigned long long keep;
        asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(keep));
        // (two lanes, every other k-tile each: one lane's wait / expect / copy sequence takes as long as a k-tile's MMAs)
        uint32_t s = lane, round = 1;
        for (int kt = lane; kt < nk; kt += 2) {
            if (!wait_barrier(p, c, &c->x_empty[s], ((xpar0 >> s) & 1u) ^ round, seq, WHERE_RING_EMPTY)) break;
            if (!check_phase(p, c, &c->x_full[s], ((xpar0 >> s) & 1u) ^ round ^ 1u, seq, WHERE_CHECK_ARM)) break;
            mbar_arrive_expect_tx(&c->x_full[s], (uint32_t)xbytes);
            tma_load_2d(xs + s * xbytes, tmaps, kbeg + kt * 64, m0, &c->x_full[s], keep);
            s += 2;
            if (s >= xstages) { s -= xstages; round ^= 1u; }
        }
    } else if ((warp == 3 || warp == 1) && lane == 0) {
        // ---- MMAs: accumulator[128 activation rows][256 weight rows] += x tile . w slot^T ----
        // Two issuing threads as in the narrow tile, each with a 256-column accumulator (columns 256 i ..) and every
        // other k-tile.  A k-tile is one activation stage and one 32 KB weight slot (the producer warp puts both weight
        // tiles of the k-tile there, one barrier): one N = 256 instruction per 16 K-elements.
        const uint32_t i = warp == 3 ? 0u : 1u;
        const uint32_t idesc = tc_idesc_n(op->i[9] == DT_F16, 256);
        const uint64_t ad0 = tc_smem_desc(smem_u32(xs)), bd0 = tc_smem_desc(smem_u32(ring));
        const uint32_t xunits = (uint32_t)xbytes >> 4;
        const uint32_t acc_at = tmem + 256 * i;
        uint32_t acc = 0, s = i, round = 0;
        uint32_t ws = ws0 + i, wph = wph0;
        if (ws >= kTcWideSlots) { ws -= kTcWideSlots; wph ^= 1u; }
        for (int kt = (int)i; kt < nk; kt += kTcIssuers) {
            if (!wait_barrier(p, c, &c->ww_full[ws], wph, seq, WHERE_RING_FULL) ||
                !wait_barrier(p, c, &c->x_full[s], ((xpar0 >> s) & 1u) ^ round, seq, WHERE_RING_FULL))
                break;
            tc_fence_after();
            const uint64_t ad = ad0 + s * xunits, bd = bd0 + ws * (2 * kTcTileBytes >> 4);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
                tc_mma(acc_at, ad + 2 * k16, bd + 2 * k16, idesc, acc);
                acc = 1;
            }
            if (!check_phase(p, c, &c->x_empty[s], ((xpar0 >> s) & 1u) ^ round, seq, WHERE_CHECK_RELEASE) ||
                !check_phase(p, c, &c->ww_empty[ws], wph, seq, WHERE_CHECK_RELEASE))
                break;
            tc_commit(&c->x_empty[s]);
            tc_commit(&c->ww_empty[ws]);
            s += kTcIssuers;
            if (s >= xstages) { s -= xstages; round ^= 1u; }
            ws += kTcIssuers;
            if (ws >= kTcWideSlots) { ws -= kTcWideSlots; wph ^= 1u; }
        }
        tc_commit(&c->acc_full);
        if (p.trace_cap > 0 && i == 0) c->t_phase[1] = (long long)globaltimer();     // last MMA issued
    }
    __syncwarp();

    // ---- epilogue: warp w owns lanes 32 (w & 3) .. +31 (activation rows) and column half w >> 2 ----
    int ok = 1;
    if (lane == 0) ok = wait_barrier(p, c, &c->acc_full, apar, seq, WHERE_COMBINE) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    tc_fence_after();
    phase_mark(p, c, 2);                                                    // accumulator complete
    __syncwarp();                                                           // (the tensor-memory loads below are .sync.aligned: whole warp, converged)
    // Per 128-column accumulator half -- first: tensor memory -> shared memory.  Warp w reads lanes
    // 32 (w & 3) .. +31 (activation rows) and column half w >> 2; the activation stages are free now
    // (every MMA has completed).  Then row-contiguous global accesses from shared memory.
    const int qd = warp & 3, h = warp >> 2;
    float* stage = reinterpret_cast<float*>(work + kTcXOff);
    const int rows = min(128, M - m0);
    const uint32_t two = nk > 1 ? 256u : 0u;                               // columns to the second issuing thread's accumulator, if it has a part
#pragma unroll 1
    for (int hf = 0; hf < halves; ++hf) {
        const int nh = n0 + 128 * hf;                                        // first weight row of this half
        if (hf) compute_sync();                                              // the previous half's rows have been read
        if (ok && qd * 32 < rows) {
            const uint32_t tl = tmem + ((uint32_t)(qd * 32) << 16) + 128 * hf;
            float* srow = stage + (qd * 32 + lane) * kTcStagePitch;
            float v[32];
            if (swi) {
                // gate columns 32 h .. +31 and the up columns 64 further of the same outputs
                float u[32];
                tc_ld32_sum(tl + h * 32, two, v);
                tc_ld32_sum(tl + 64 + h * 32, two, u);
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(srow + h * 32 + j) =
                        make_float4(v[j] * sigmoidf_(v[j]) * u[j], v[j + 1] * sigmoidf_(v[j + 1]) * u[j + 1],
                                    v[j + 2] * sigmoidf_(v[j + 2]) * u[j + 2], v[j + 3] * sigmoidf_(v[j + 3]) * u[j + 3]);
            } else {
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    const int tcol = h * 64 + ch * 32;
                    if (nh + tcol >= N) break;
                    tc_ld32_sum(tl + tcol, two, v);
#pragma unroll
                    for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(srow + tcol + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
        }
        tc_fence_before();
        compute_sync();
        if (ok) {
            if (swi) tc_write_rows(op, stage, m0, rows, 64, nh / 2, N / 2);
            else if (op->i[6]) tc_write_rows(op, stage, m0, rows, 128, nh, N);          // split-K partial: reduce-add
            else tc_store_rows(op, stage, m0, rows, nh, N);
        }
    }
    tc_fence_before();
    const bool aborting = compute_sync_or(!ok || *(volatile int*)&c->abort);
    if (t == 0) tc_finish_state(c, uses, xpar0, ws0, wph0, nk, xstages, true);
    if (aborting) return -1;
    return 0;
}

}  // namespace mk
