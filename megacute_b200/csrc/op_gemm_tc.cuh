// MK_OP_GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory), compute-warp side.
//   out[128 x 128 tile] = act(x @ w^T + bias) + residual        (one instruction per output tile)
//   ws += x[:, Kj] @ w[:, Kj]^T                                  (split-K partial: reduce-add)
// Same instructions, descriptor and epilogue semantics as the mma.sync body (op_gemm.cuh); the host
// library selects this body by putting the address of two tensor maps in ptr 11 (activations, then
// weights 128 bytes further: {K, rows} bf16, 128-byte swizzle, zero fill; boxes of 64 columns x 128
// rows, or x 64 rows for the activations of an op with at most 64 of them) and, when it has packed
// the weights into tile images, the packed array in ptr 10.
//
// Operands are K-major 128-row x 64-column tiles (16 KB).  The 128 activation rows of the m tile are
// the MMA's M side, so an accumulator row (a tensor-memory lane) is an activation row and a thread of
// the epilogue holds whole output rows: swiglu (gate columns 0..63, up columns 64..127 of the weight
// tile) pairs values of one thread.  Rows beyond M are zero-filled by the copy and never stored.
//   weights      producer warp -> eight single-tile slots in the ring's memory, across instruction
//                boundaries: they depend on nothing in the launch, so the next instruction's first
//                128 KB are already on their way while this one waits for its dependencies
//   activations  one compute thread -> single-tile stages in the work area, after the instruction's
//                dependencies are met: 6 stages of 128 rows, or 10 of 64 rows when the op has at most
//                64 (the MMA still reads 128 rows: the upper 64 accumulator rows are never looked at)
//   MMA          one compute thread: 4 x tcgen05.mma (128 x 128 x 16) per k-tile; tcgen05.commit
//                returns the activation stage and the ring slot when the MMAs that read them are done
//   epilogue     all 8 compute warps: tensor memory -> shared memory (warp w reads lanes 32 (w & 3) .. +31,
//                column half w >> 2), then row-contiguous global stores / reductions from there
// Every wait is bounded (wait_barrier); tensor memory is allocated by the first such instruction of a
// CTA and freed by the kernel before it exits, on every path.
#pragma once
#include "mk_device.cuh"
#include "mma.cuh"
#include "op_gemv_common.cuh"

namespace mk {

// instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A format (bits 7-9) and B format (bits 10-12):
// 0 = fp16, 1 = bf16, both K-major, N = 128 (bits 17-22 = N / 8), M = 128 (bits 24-28 = M / 16).  Both
// operands have one type: bf16, or -- when the activations are runtime-private ones kept in fp16, see
// passes.promote_temps -- fp16, with the packed weight copy converted to fp16 by the host library.
__device__ __forceinline__ uint32_t tc_idesc_n(bool fp16, uint32_t n) {
    const uint32_t fmt = fp16 ? 0u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ uint32_t tc_idesc(bool fp16) { return tc_idesc_n(fp16, 128); }

// shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: start address,
// leading byte offset 16 (unused by swizzled K-major layouts), 1024 bytes between 8-row groups,
// descriptor version 1, layout type 2 (128-byte swizzle).  Advancing 16 K-elements inside the
// swizzle atom adds 32 bytes to the start address.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the mbarrier once every tcgen05.mma this thread has issued so far has completed
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 consecutive fp32 columns of this thread's lane (warp-wide, lanes 32 (warp & 3) .. +31)
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"          // in the same statement: no use of the registers can move above it
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}

// the same columns of two accumulators, `second` columns apart, added (second == 0: one accumulator)
__device__ __forceinline__ void tc_ld32_sum(uint32_t taddr, uint32_t second, float* v) {
    tc_ld32(taddr, v);
    if (second) {
        float w[32];
        tc_ld32(taddr + second, w);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += w[j];
    }
}

// State the next tile GEMM instruction of this CTA starts from, written by one thread behind the barrier that
// ends the epilogue: the accumulator barrier's use count, the parities of the activation stages (stage s was
// used once more per full round through the stages, and once more if s < nk mod stages) and the position in
// the weight slots (of the kind the instruction used).
__device__ __forceinline__ void tc_finish_state(Ctrl* c, uint32_t uses, uint32_t xpar0, uint32_t ws0, uint32_t wph0, int nk,
                                                uint32_t xstages, bool wide) {
    c->acc_uses = uses + 1;
    const uint32_t full = (uint32_t)nk / xstages, rem = (uint32_t)nk - full * xstages;
    c->x_par = xpar0 ^ ((full & 1u) ? (1u << xstages) - 1u : 0u) ^ ((1u << rem) - 1u);
    const uint32_t pos = ws0 + (uint32_t)nk;               // one weight slot per k-tile
    if (wide) {
        c->ww_slot = (uint8_t)(pos % kTcWideSlots);
        c->ww_phase = (uint8_t)((wph0 ^ (pos / kTcWideSlots)) & 1u);
    } else {
        c->w_slot = (uint8_t)(pos % kTcWSlots);
        c->w_phase = (uint8_t)((wph0 ^ (pos / kTcWSlots)) & 1u);
    }
}

// Epilogue, second half.  The accumulator tile has been copied to shared memory (fp32, row pitch
// kTcStagePitch words); here a warp instruction covers one output row (or two half rows), four
// consecutive columns per lane, so every global access of the epilogue -- bias, residual, store or
// reduce-add -- is a contiguous 256 or 512 bytes.  Straight from tensor memory a lane holds a row,
// and a warp store touched 32 rows: measured on the lm_head tiles of batch-64 decode (rows 256 KB
// apart, lines not in L2) the stores of one tile took 9.5 us to issue.
constexpr int kTcStagePitch = 132;                          // words: conflict-free 16-byte writes by row, reads by column
static_assert(kTcXOff + 128 * kTcStagePitch * 4 <= kWorkBytes, "epilogue staging tile");
static __device__ __noinline__ void tc_write_rows(const mk_op_desc* op, const float* stage, int m0, int rows, int ncols, int col0,
                                              int n_out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int act = op->i[3], odt = op->i[5], accum = op->i[6], rdt = op->i[7];
    const bool plain = !accum && !op->i[8];
    uint8_t* O = reinterpret_cast<uint8_t*>(op->ptr[2]);
    const uint8_t* bias = reinterpret_cast<const uint8_t*>(op->ptr[3]);
    const uint8_t* R = reinterpret_cast<const uint8_t*>(op->ptr[4]);
    const int lpr = ncols >> 2;                                // lanes per row: 32, or 16 (swiglu: two rows per pass)
    const int sub = lane / lpr, c4 = (lane % lpr) * 4, col = col0 + c4;
    if (col >= n_out) return;
    float b4[4] = {0.f, 0.f, 0.f, 0.f};
    if (plain && bias) {
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(bias + (long long)col * 2));
        b4[0] = bf16_lo(w.x); b4[1] = bf16_hi(w.x); b4[2] = bf16_lo(w.y); b4[3] = bf16_hi(w.y);
    }
    const int step = kComputeWarps * (32 / lpr);
#pragma unroll 2
    for (int row = warp * (32 / lpr) + sub; row < rows; row += step) {
        const float4 q = *reinterpret_cast<const float4*>(stage + row * kTcStagePitch + c4);
        float f[4] = {q.x, q.y, q.z, q.w};
        const long long eo = (long long)(m0 + row) * op->ld[2] + col;
        if (accum) {
            if (odt == 1) red_add_f32x4(reinterpret_cast<float*>(O) + eo, f[0], f[1], f[2], f[3]);
            else red_add_bf16x4(O + eo * 2, f);
            continue;
        }
        if (plain) {
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] = apply_act(act, f[j] + b4[j]);
            if (R) {
                const long long er = (long long)(m0 + row) * op->ld[4] + col;
                if (rdt == DT_F32) {
                    const float4 x = __ldcg(reinterpret_cast<const float4*>(R + er * 4));
                    f[0] += x.x; f[1] += x.y; f[2] += x.z; f[3] += x.w;
                } else {
                    const uint2 w = __ldcg(reinterpret_cast<const uint2*>(R + er * 2));
                    if (rdt == DT_F16) {
                        const float2 lo = unpack2h(w.x), hi = unpack2h(w.y);
                        f[0] += lo.x; f[1] += lo.y; f[2] += hi.x; f[3] += hi.y;
                    } else {
                        f[0] += bf16_lo(w.x); f[1] += bf16_hi(w.x); f[2] += bf16_lo(w.y); f[3] += bf16_hi(w.y);
                    }
                }
            }
        }
        if (odt == DT_F32) *reinterpret_cast<float4*>(O + eo * 4) = make_float4(f[0], f[1], f[2], f[3]);
        else *reinterpret_cast<uint2*>(O + eo * 2) = make_uint2(pack2t(odt, f[0], f[1]), pack2t(odt, f[2], f[3]));
    }
}

// Epilogue, second half, plain tiles (not a split-K partial, not swiglu): out = act(acc + bias) + residual, 128 columns.
// Specialised at compile time on output type, residual kind and whether there is an activation: with those as
// run-time switches inside the row loop the writer was instruction-bound (4.2 us per 128 x 128 tile against 1.3 us
// for the same stores from a specialised loop, measured stand-alone).  All residual rows of a warp (16) are
// requested before the first is used: two loads in flight per warp made a residual tile take 8.7 us, sixteen 2.3 us.
template <int ODT, int RKIND, bool ACT>              // RKIND 0: no residual, 1: 16-bit (bf16 / fp16 by rdt), 2: fp32
static __device__ __noinline__ void tc_store_rows_t(const mk_op_desc* op, const float* stage, int m0, int rows, int col0, int n_out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int act = op->i[3], rdt = op->i[7];
    const int c4 = lane * 4, col = col0 + c4;
    if (col >= n_out) return;
    float b4[4] = {0.f, 0.f, 0.f, 0.f};
    if (const uint8_t* bias = reinterpret_cast<const uint8_t*>(op->ptr[3])) {
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(bias + (long long)col * 2));
        b4[0] = bf16_lo(w.x); b4[1] = bf16_hi(w.x); b4[2] = bf16_lo(w.y); b4[3] = bf16_hi(w.y);
    }
    constexpr int kRows = 128 / kComputeWarps;          // rows of the tile per warp
    const long long ldo = op->ld[2], ldr = op->ld[4];
    uint8_t* O = reinterpret_cast<uint8_t*>(op->ptr[2]) + ((long long)m0 * ldo + col) * (ODT == DT_F32 ? 4 : 2);
    const uint8_t* R = reinterpret_cast<const uint8_t*>(op->ptr[4]) + ((long long)m0 * ldr + col) * (RKIND == 2 ? 4 : 2);
    uint2 r16[RKIND == 1 ? kRows : 1];
    float4 r32[RKIND == 2 ? kRows : 1];
    if (RKIND == 1) {
#pragma unroll
        for (int j = 0; j < kRows; ++j) {
            const int row = warp + j * kComputeWarps;
            r16[j] = row < rows ? __ldcg(reinterpret_cast<const uint2*>(R + row * ldr * 2)) : make_uint2(0u, 0u);
        }
    }
    if (RKIND == 2) {
#pragma unroll
        for (int j = 0; j < kRows; ++j) {
            const int row = warp + j * kComputeWarps;
            r32[j] = row < rows ? __ldcg(reinterpret_cast<const float4*>(R + row * ldr * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
        const int row = warp + j * kComputeWarps;
        if (row >= rows) break;
        const float4 q = *reinterpret_cast<const float4*>(stage + row * kTcStagePitch + c4);
        float f[4] = {q.x + b4[0], q.y + b4[1], q.z + b4[2], q.w + b4[3]};
        if (ACT) {
#pragma unroll
            for (int e = 0; e < 4; ++e) f[e] = apply_act(act, f[e]);
        }
        if (RKIND == 1) {
            if (rdt == DT_F16) {
                const float2 lo = unpack2h(r16[j].x), hi = unpack2h(r16[j].y);
                f[0] += lo.x; f[1] += lo.y; f[2] += hi.x; f[3] += hi.y;
            } else {
                f[0] += bf16_lo(r16[j].x); f[1] += bf16_hi(r16[j].x); f[2] += bf16_lo(r16[j].y); f[3] += bf16_hi(r16[j].y);
            }
        }
        if (RKIND == 2) { f[0] += r32[j].x; f[1] += r32[j].y; f[2] += r32[j].z; f[3] += r32[j].w; }
        if (ODT == DT_F32) *reinterpret_cast<float4*>(O + row * ldo * 4) = make_float4(f[0], f[1], f[2], f[3]);
        else if (ODT == DT_F16) *reinterpret_cast<uint2*>(O + row * ldo * 2) = make_uint2(pack2h(f[0], f[1]), pack2h(f[2], f[3]));
        else *reinterpret_cast<uint2*>(O + row * ldo * 2) = make_uint2(pack2(f[0], f[1]), pack2(f[2], f[3]));
    }
}
template <int ODT>
__device__ __forceinline__ void tc_store_rows_o(const mk_op_desc* op, const float* stage, int m0, int rows, int col0, int n_out) {
    const int rk = !op->ptr[4] ? 0 : op->i[7] == DT_F32 ? 2 : 1;
    if (op->i[3] != ACT_NONE) {                       // activations are rare in front of a residual: one instance takes every residual kind
        if (rk == 0) tc_store_rows_t<ODT, 0, true>(op, stage, m0, rows, col0, n_out);
        else if (rk == 1) tc_store_rows_t<ODT, 1, true>(op, stage, m0, rows, col0, n_out);
        else tc_store_rows_t<ODT, 2, true>(op, stage, m0, rows, col0, n_out);
    } else if (rk == 0) tc_store_rows_t<ODT, 0, false>(op, stage, m0, rows, col0, n_out);
    else if (rk == 1) tc_store_rows_t<ODT, 1, false>(op, stage, m0, rows, col0, n_out);
    else tc_store_rows_t<ODT, 2, false>(op, stage, m0, rows, col0, n_out);
}
__device__ __forceinline__ void tc_store_rows(const mk_op_desc* op, const float* stage, int m0, int rows, int col0, int n_out) {
    const int odt = op->i[5];
    if (odt == DT_F32) tc_store_rows_o<DT_F32>(op, stage, m0, rows, col0, n_out);
    else if (odt == DT_F16) tc_store_rows_o<DT_F16>(op, stage, m0, rows, col0, n_out);
    else tc_store_rows_o<DT_BF16>(op, stage, m0, rows, col0, n_out);
}

// All compute threads call this after the instruction's dependencies are met.  Returns 0, or -1
// when the CTA is aborting.
__device__ __forceinline__ int op_gemm_tc(const Params& p, Ctrl* c, uint8_t* ring, uint8_t* work, const mk_op_desc* op, int a0,
                                          int a1, int a2, int seq) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int M = op->i[0], N = op->i[1], K = op->i[2], splits = op->i[4];
    const int swi = op->i[8];
    const int m0 = a0 * 128, n0 = a1 * 128;
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
    const uint32_t xpar0 = c->x_par;            // parities at the instruction's start (written behind the previous one's last barrier)
    const uint32_t ws0 = c->w_slot, wph0 = c->w_phase;
    if (warp == 2 && lane < 2) {
        // ---- activation tiles: {64 K-elements, 128 rows} at (kbeg + 64 kt, m0) ----
        // earlier instructions wrote the work area through the generic proxy (all of that is behind
        // the barrier that ended the dependency wait); the bulk copies below write it through the
        // asynchronous one, and read activations other SMs stored with plain stores
        asm volatile("fence.proxy.async;" ::: "memory");
        unsigned long long keep;
        asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(keep));
        // k-tile kt goes to stage kt mod the number of stages, each instruction starting at stage 0; the
        // parity of a stage's barriers is the one it had at the instruction's start, flipped once per
        // round through the stages (ops with 6 and with 10 stages may alternate: bit s follows barrier s)
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
        // ---- MMAs: accumulator[128 activation rows][128 weight rows] += x tile . w tile^T ----
        // Two issuing threads, each with an accumulator of its own (columns 128 i ..): this one takes the
        // k-tiles kt = i, i + 2, ...; the epilogue adds the two.  What a thread executes between two
        // tcgen05.mma leaves the tensor pipe idle -- the instruction does not return before the previous
        // MMA is nearly done, so nothing is queued behind it.  Measured with a stand-alone loop: the four
        // MMAs of a k-tile take 0.19 us, the loop around them (two waits, two commits, counters) as much
        // again; a second thread's MMAs fill those gaps (0.43 -> 0.26 us per k-tile).  For the same reason
        // the loop has counters that step and wrap instead of divisions, descriptors by addition, and
        // waits that first ask with test_wait (a try_wait costs ~95 ns even on a completed phase).
        const uint32_t i = warp == 3 ? 0u : 1u;
        const uint32_t idesc = tc_idesc(op->i[9] == DT_F16);
        const uint64_t ad0 = tc_smem_desc(smem_u32(xs)), bd0 = tc_smem_desc(smem_u32(ring));
        const uint32_t xunits = (uint32_t)xbytes >> 4;                        // descriptor addresses count 16 bytes
        const uint32_t acc_at = tmem + 128 * i;
        uint32_t acc = 0, s = i, round = 0;
        uint32_t ws = ws0 + i, wph = wph0;
        if (ws >= kTcWSlots) { ws -= kTcWSlots; wph ^= 1u; }
        for (int kt = (int)i; kt < nk; kt += kTcIssuers) {
            if (!wait_barrier(p, c, &c->w_full[ws], wph, seq, WHERE_RING_FULL) ||
                !wait_barrier(p, c, &c->x_full[s], ((xpar0 >> s) & 1u) ^ round, seq, WHERE_RING_FULL))
                break;
            tc_fence_after();
            const uint64_t ad = ad0 + s * xunits, bd = bd0 + ws * (kTcTileBytes >> 4);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
                tc_mma(acc_at, ad + 2 * k16, bd + 2 * k16, idesc, acc);
                acc = 1;
            }
            if (!check_phase(p, c, &c->x_empty[s], ((xpar0 >> s) & 1u) ^ round, seq, WHERE_CHECK_RELEASE) ||
                !check_phase(p, c, &c->w_empty[ws], wph, seq, WHERE_CHECK_RELEASE))
                break;
            tc_commit(&c->x_empty[s]);
            tc_commit(&c->w_empty[ws]);
            s += kTcIssuers;
            if (s >= xstages) { s -= xstages; round ^= 1u; }
            ws += kTcIssuers;
            if (ws >= kTcWSlots) { ws -= kTcWSlots; wph ^= 1u; }
        }
        tc_commit(&c->acc_full);                                            // (arrives at once when this thread had no k-tile)
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
    // first half: tensor memory -> shared memory.  Warp w reads lanes 32 (w & 3) .. +31 (activation
    // rows) and column half w >> 2; the activation stages are free now (every MMA has completed).
    const int qd = warp & 3, h = warp >> 2;
    float* stage = reinterpret_cast<float*>(work + kTcXOff);
    const int rows = min(128, M - m0);
    const uint32_t two = nk > 1 ? 128u : 0u;                               // columns to the second issuing thread's accumulator, if it has a part
    if (ok && qd * 32 < rows) {
        const uint32_t tl = tmem + ((uint32_t)(qd * 32) << 16);
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
                if (n0 + tcol >= N) break;
                tc_ld32_sum(tl + tcol, two, v);
#pragma unroll
                for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(srow + tcol + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        }
    }
    tc_fence_before();
    compute_sync();
    if (ok) {
        if (swi) tc_write_rows(op, stage, m0, rows, 64, a1 * 64, N / 2);
        else if (op->i[6]) tc_write_rows(op, stage, m0, rows, 128, n0, N);              // split-K partial: reduce-add
        else tc_store_rows(op, stage, m0, rows, n0, N);
    }
    tc_fence_before();
    const bool aborting = compute_sync_or(!ok || *(volatile int*)&c->abort);
    if (t == 0) tc_finish_state(c, uses, xpar0, ws0, wph0, nk, xstages, false);
    if (aborting) return -1;
    return 0;
}

}  // namespace mk
