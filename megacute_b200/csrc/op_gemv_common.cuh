// MK_OP_GEMV: linear with <= 8 activation rows, out = act(norm(x) @ w^T + bias) + residual.
//
// Pure weight streaming.  The producer warp copies weight rows into a ring of two 64 KB stages with
// 1-D bulk copies (one 4 KB copy per row segment, completion counted on the stage's mbarrier) and
// runs ahead of the compute warps across instruction boundaries, because weights never depend on
// anything in the launch.  On the tensor-core path (GEMV_F_UNITS, below) a stage holds 16 weight
// rows x one 2048-element K segment; on the general CUDA-core path (op_gemv.cuh: K not a multiple of
// 16) it holds 8 row slots x 2048 K-elements, compute thread t owns K-elements [8t, 8t+8) of every
// slot, and partial dot products are reduced across the CTA once per group of 8 rows.
//
// descriptor: ptr 0 x, 1 w, 2 out, 3 bias, 4 residual, 5 norm gain
//             i 0 M, 1 N_out, 2 K, 3 act, 4 x dtype, 5 out dtype, 6 residual dtype
//             f 0 rms eps; flags bit0 swiglu (w rows interleaved in 64-row gate/up blocks,
//             slots 0-3 = gate rows and 4-7 = up rows of 4 outputs), bit1 rms-normalise x first
// instruction args: 0 o0, 1 o1 -- the output columns [o0, o1) this instruction produces.
#pragma once
#include "mk_device.cuh"

namespace mk {

constexpr int GEMV_F_SWIGLU = 1, GEMV_F_RMS = 2;
// GEMV_F_UNITS (set by the host when K is a multiple of 16): the tensor-core streaming path.
// A stage is 16 weight rows x one 2048-element K segment.  Each compute warp multiplies a 256-wide
// K slice of the 16 rows with warp-level MMAs (weights are the A operand straight from the stage via
// ldmatrix; the <= 8 activation rows are the B operand, split into bf16 high and low parts so the
// product keeps ~16 mantissa bits of the activation), accumulates over the segments of the row
// group, and the 8 warps combine through shared memory: the last to arrive writes the 16 outputs.
// About 12 instructions per 512 bytes of weights, so the warps mostly wait for HBM.
constexpr int GEMV_F_UNITS = 4;

struct RingPos {
    int stage = 0;
    uint32_t phase = 0;
    uint32_t comb = 0;           // compute side only: parities of slot_free[0..3] (bits 0..3) and epi_done (bit 4)
    __device__ __forceinline__ void advance() {
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
    }
};

__device__ __forceinline__ int gemv_weight_row(bool swi, int o0, int group, int slot, int* out_col) {
    if (!swi) {
        int o = o0 + group * 8 + slot;
        *out_col = o;
        return o;
    }
    int o = o0 + group * 4 + (slot & 3);
    *out_col = o;
    return 128 * (o >> 6) + (o & 63) + ((slot >> 2) << 6);
}

// ---- producer side -------------------------------------------------------------------------------
// The producer warp sees this CTA's streaming linears as one long sequence of ring stages.  A
// StageCursor names one stage of that sequence (instruction, row group, K segment) and yields,
// per lane, the weight-row segment that lane copies.  Two cursors walk the sequence: one feeds the
// shared-memory ring with bulk copies, the other runs up to Params::pf_stages stages further
// ahead and only asks L2 to fetch the same bytes (cp.async.bulk.prefetch.L2), so HBM keeps
// streaming while the ring is full and the compute warps sit in a dependency hop.
struct StageCursor {
    int idx;                 // global instruction index (this CTA's: idx = cta + k * grid); >= n_insts: end
    int seq, g, seg;         // instruction sequence number, row group and K segment inside it
    int ngroups, nseg;       // of the current instruction
    int o0, o1, K, flags;
    const __nv_bfloat16* w;
    long long ldw;
    // tile GEMM on the tcgen05 path (op_gemm_tc.cuh): the weight k-tiles [kt, nk) of the instruction
    // are still to be copied, through the tensor map `wmap`, from coordinates (kbeg + 64 kt, n0)
    bool gemm;
    int kt, nk, kbeg, n0, wide;
    bool reread;                 // the weight tiles are read again and again, by the instructions of many row tiles (more than two)
    const void* wmap;
    // ... or, when the host library has packed the weights into tile images (ptr 10), the 16 KB
    // block `wtile0 + kt * wstride` of that array (k-tile-major: wstride = number of n tiles)
    const uint8_t* wpack;
    long long wtile0;
    int wstride;
    // many-sequence decode attention (op_decode_bulk.cuh): the K and V tiles [kv_t, kv_nt) of the
    // instruction's KV split are still to be copied; kv_which alternates K (0) and V (1)
    bool kv;
    int kv_t, kv_nt, kv_which, kv_rb;
    bool kv_gated;           // unfused form: the first copy waits for kv_go
    const uint8_t* kv_src[2];
    long long kv_pitch[2];   // bytes between cache rows

    // position on the next streaming-linear instruction at or after `idx`
    __device__ __forceinline__ void seek(const Params& p) {
        for (; idx < p.n_insts; idx += gridDim.x) {
            const Inst in = fetch_inst(p, idx);
            const int opi = in.opi - 1;
            if (opi < 0 || opi >= p.n_ops) { idx = p.n_insts; return; }
            const mk_op_desc* op = p.ops + opi;
            if (op->kind == MK_OP_DECODE_ATTN && op->i[11]) {
                const int KVH = op->i[2], L = op->i[4], S = op->i[5];
                const bool fused = op->i[6] != 0;
                // pos is rewritten only by the launch's last instruction, behind every reader's arrival
                const int posv = reinterpret_cast<const volatile int*>(op->ptr[3])[(long long)in.a0 * op->i[12]];
                int k_begin, k_end;
                kv_split_range(fused ? posv : posv + 1, S, in.a2, k_begin, k_end);
                gemm = false; kv = true; seq = in.seq;
                kv_t = 0; kv_nt = (k_end - k_begin + kKvTileRows - 1) / kKvTileRows; kv_which = 0;
                kv_rb = KVH * 64 * 2;
                kv_gated = !fused;
                for (int w = 0; w < 2; ++w) {
                    kv_pitch[w] = (long long)op->ld[1 + w] * 2;
                    kv_src[w] = reinterpret_cast<const uint8_t*>(op->ptr[1 + w]) + ((long long)in.a0 * L + k_begin) * kv_pitch[w];
                }
                if (kv_nt > 0 || kv_gated) return;     // (a gated instruction without tiles still consumes its kv_go)
                continue;
            }
            if (op->kind == MK_OP_GEMM && op->ptr[11]) {
                // a 256-wide output tile (i 10) takes two 128-row weight tiles per k-tile, one after the
                // other through the same single-tile slots: `kt` counts weight tiles, `wide` of them per k-tile
                const int kc = op->i[2] / op->i[4];
                wide = op->i[10] == 256 ? 2 : 1;
                reread = op->i[0] > 256;      // (two row tiles run side by side and share the line in flight: measured, evict-first is then the faster)
                gemm = true; kv = false; seq = in.seq; kt = 0; nk = kc / 64 * wide; kbeg = in.a2 * kc; n0 = in.a1 * 128 * wide;
                wmap = reinterpret_cast<const uint8_t*>(op->ptr[11]) + 128;
                wpack = reinterpret_cast<const uint8_t*>(op->ptr[10]);
                wstride = (op->i[1] + 127) / 128;
                wtile0 = (long long)(kbeg / 64) * wstride + in.a1 * wide;
                if (nk > 0) return;
                continue;
            }
            if (op->kind != MK_OP_GEMV) continue;
            gemm = false; kv = false;
            seq = in.seq; o0 = in.a0; o1 = in.a1; K = op->i[2]; flags = op->flags;
            w = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]);
            ldw = op->ld[1];
            const int n = o1 - o0;
            const bool swi = flags & GEMV_F_SWIGLU;
            if (flags & GEMV_F_UNITS) {
                ngroups = (swi ? 2 : 1) * ((n + 15) / 16);
                nseg = (K + kSegElems - 1) / kSegElems;
            } else {
                const int per = swi ? 4 : 8;
                ngroups = (n + per - 1) / per;
                nseg = (K + kGemvKChunk - 1) / kGemvKChunk;
            }
            g = 0; seg = 0;
            if (ngroups > 0) return;
        }
    }
    __device__ __forceinline__ bool valid(const Params& p) const { return idx < p.n_insts; }
    __device__ __forceinline__ void advance(const Params& p) {
        if (gemm || kv) {                             // (the L2 prefetch cursor: whole instruction at once)
            idx += gridDim.x;
            seek(p);
            return;
        }
        if (++seg < nseg) return;
        seg = 0;
        if (++g < ngroups) return;
        idx += gridDim.x;
        seek(p);
    }
    // this lane's piece of the stage: source, bytes (0 = none) and offset inside the ring stage
    __device__ __forceinline__ void piece(int lane, const __nv_bfloat16*& src, int& bytes, int& dst_off) const {
        const bool swi = flags & GEMV_F_SWIGLU;
        src = w; bytes = 0; dst_off = 0;
        if (gemm || kv) return;
        if (flags & GEMV_F_UNITS) {
            const int r = lane & 15;
            const int o = o0 + (swi ? g >> 1 : g) * 16 + r;
            const int row = swi ? 128 * (o >> 6) + (o & 63) + ((g & 1) << 6) : o;
            const int k0 = seg * kSegElems;
            if (lane < 16 && o < o1) { src = w + row * ldw + k0; bytes = min(kSegElems, K - k0) * 2; dst_off = r * kSegStride; }
        } else {
            int col;
            const int row = gemv_weight_row(swi, o0, g, lane & 7, &col);
            const int k0 = seg * kGemvKChunk;
            if (lane < 8 && col < o1) { src = w + row * ldw + k0; bytes = min(kGemvKChunk, K - k0) * 2; dst_off = (lane & 7) * (kGemvKChunk * 2); }
        }
    }
};

// Producer warp main loop.  TRACE: role-0 records (seq, first stage issued, -, last stage issued).
template <bool TRACE>
__device__ __forceinline__ void producer_loop(const Params& p, Ctrl* c, uint8_t* ring) {
    const int lane = threadIdx.x & 31;
    RingPos pos;
    StageCursor rc, pc;
    rc.idx = blockIdx.x;
    rc.seek(p);
    pc = rc;
    int ahead = 0;                                   // stages the prefetch cursor is ahead of the ring cursor
    long long t_first = 0;
    int slot_first = 0;
    const unsigned long long stream_policy = l2_policy_evict_first();
    // weights of a tile GEMM with several row tiles are read once per row tile: those stay in L2 with normal priority
    unsigned long long keep_policy;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(keep_policy));
    // tile GEMM weight slots and decode attention KV slots: positions, and which kind of slot the
    // ring's memory currently serves
    int wslot = 0;
    uint32_t wphase = 0;
    int kvslot = 0;
    uint32_t kvphase = 0, kvgo = 0;
    enum { MODE_STAGES = 0, MODE_WTILES = 1, MODE_KVTILES = 2, MODE_WWIDE = 3 };
    int wwslot = 0;
    uint32_t wwphase = 0;
    int mode = MODE_STAGES;
    // Wait until the compute side has released every slot of the kind used so far (slot s was last
    // filled in the current round if s < position, else in the previous one).
    auto drain = [&](int kind) -> bool {
        int ok = 1;
        if (lane == 0) {
            if (kind == MODE_WTILES) {
                for (int s = 0; s < kTcWSlots && ok; ++s)
                    ok = wait_barrier(p, c, &c->w_empty[s], (wphase ^ (s < wslot ? 1u : 0u)) ^ 1u, rc.seq, WHERE_RING_EMPTY) ? 1 : 0;
            } else if (kind == MODE_WWIDE) {
                for (int s = 0; s < kTcWideSlots && ok; ++s)
                    ok = wait_barrier(p, c, &c->ww_empty[s], (wwphase ^ (s < wwslot ? 1u : 0u)) ^ 1u, rc.seq, WHERE_RING_EMPTY) ? 1 : 0;
            } else if (kind == MODE_KVTILES) {
                for (int s = 0; s < kKvSlots && ok; ++s)
                    ok = wait_barrier(p, c, &c->kv_empty[s], (kvphase ^ (s < kvslot ? 1u : 0u)) ^ 1u, rc.seq, WHERE_RING_EMPTY) ? 1 : 0;
            } else {
                for (int s = 0; s < kStages && ok; ++s)
                    ok = wait_barrier(p, c, &c->empty[s], (pos.phase ^ (s < pos.stage ? 1u : 0u)) ^ 1u, rc.seq, WHERE_RING_EMPTY) ? 1 : 0;
            }
        }
        return __shfl_sync(0xffffffffu, ok, 0) != 0;
    };
    auto enter = [&](int kind) -> bool {              // make the ring's memory serve `kind`
        if (mode == kind) return true;
        if (!drain(mode)) return false;
        mode = kind;
        return true;
    };
    while (rc.valid(p)) {
        if (rc.kv) {
            // decode attention, many-sequence form: one tile of 16 whole cache rows per slot, as four
            // copies of four rows issued by four lanes at once; K and V tiles alternate.  The whole
            // instruction is streamed from this tight loop: measured, a single lane that issued every
            // copy and walked the outer loop per slot spent ~950 cycles per 16 KB slot (32 GB/s).
            if (!enter(MODE_KVTILES)) return;
            if (rc.kv_gated) {                        // unfused form: the appended row is readable once the dependencies are met
                int go = 1;
                if (lane == 0) go = wait_barrier(p, c, &c->kv_go, kvgo, rc.seq, WHERE_DEP) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, go, 0)) return;
                kvgo ^= 1u;
            }
            const int g = lane & 3;
            const uint32_t group_bytes = (uint32_t)(kKvGroupRows * rc.kv_rb), tile_bytes = (uint32_t)(kKvTileRows * rc.kv_rb);
            const uint8_t* src[2] = {rc.kv_src[0] + (long long)g * kKvGroupRows * rc.kv_pitch[0],
                                     rc.kv_src[1] + (long long)g * kKvGroupRows * rc.kv_pitch[1]};
            const long long step[2] = {(long long)kKvTileRows * rc.kv_pitch[0], (long long)kKvTileRows * rc.kv_pitch[1]};
            uint8_t* dst = ring + g * (group_bytes + kKvGroupSkew);
#pragma unroll 1
            for (int t = 0; t < rc.kv_nt; ++t) {
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    int ok = 1;
                    if (lane == 0) {
                        ok = wait_barrier(p, c, &c->kv_empty[kvslot], kvphase ^ 1u, rc.seq, WHERE_RING_EMPTY) ? 1 : 0;
                        if (ok) mbar_arrive_expect_tx(&c->kv_full[kvslot], tile_bytes);
                    }
                    if (!__shfl_sync(0xffffffffu, ok, 0)) return;      // (also: the expected bytes are registered before any copy is issued)
                    if (lane < kKvTileRows / kKvGroupRows)
                        bulk_g2s_hint(dst + kvslot * kKvSlotBytes, src[w], group_bytes, &c->kv_full[kvslot], stream_policy);
                    src[w] += step[w];
                    if (++kvslot == kKvSlots) { kvslot = 0; kvphase ^= 1u; }
                }
            }
            rc.idx += gridDim.x;
            rc.seek(p);
            continue;
        }
        if (rc.gemm && rc.wide == 2) {
            // 128 x 256 tile GEMM: the two weight tiles of a k-tile (256 rows x 64 K-elements, adjacent in the packed
            // array) fill one 32 KB slot and complete one barrier, so that the issuing thread pays one wait, four
            // N = 256 MMAs and one commit per k-tile and operand (measured stand-alone with two issuing threads:
            // 0.28 us per k-tile against 0.40 with a barrier pair per 16 KB tile).
            if (!enter(MODE_WWIDE)) return;
            const int nkt = rc.nk >> 1;
            // Two lanes, every other k-tile each.  Lanes run in lockstep, so a step waits for the slower lane's slot: with
            // as many lanes as slots the four copies left in bursts, once the last slot of the previous burst had been
            // consumed, and the consumer starved for a copy's latency per burst (0.57 us per k-tile; 0.48 before).
            constexpr int kLanes = 2;
            const unsigned long long wpol = rc.reread ? keep_policy : stream_policy;
            bool mine = true;
            if (lane < kLanes) {
                const uint8_t* src = rc.wpack ? rc.wpack + rc.wtile0 * (long long)kTcTileBytes : nullptr;
                const long long kstep = (long long)rc.wstride * kTcTileBytes;
                uint32_t sl = (uint32_t)wwslot + lane, ph = wwphase;
                if (sl >= kTcWideSlots) { sl -= kTcWideSlots; ph ^= 1u; }
#pragma unroll 1
                for (int kt = lane; kt < nkt; kt += kLanes) {
                    if (!wait_barrier(p, c, &c->ww_empty[sl], ph ^ 1u, rc.seq, WHERE_RING_EMPTY)) { mine = false; break; }
                    if (!check_phase(p, c, &c->ww_full[sl], ph, rc.seq, WHERE_CHECK_ARM)) { mine = false; break; }
                    uint8_t* dst = ring + sl * (2 * kTcTileBytes);
                    mbar_arrive_expect_tx(&c->ww_full[sl], 2u * kTcTileBytes);
                    if (src) {
                        bulk_g2s_hint(dst, src + kt * kstep, 2u * kTcTileBytes, &c->ww_full[sl], wpol);
                    } else {
                        tma_load_2d(dst, rc.wmap, rc.kbeg + kt * 64, rc.n0, &c->ww_full[sl], wpol);
                        tma_load_2d(dst + kTcTileBytes, rc.wmap, rc.kbeg + kt * 64, rc.n0 + 128, &c->ww_full[sl], wpol);
                    }
                    sl += kLanes;
                    if (sl >= kTcWideSlots) { sl -= kTcWideSlots; ph ^= 1u; }
                }
            }
            const bool ok = __all_sync(0xffffffffu, mine);
            const uint32_t wpos = (uint32_t)wwslot + (uint32_t)nkt;
            wwslot = (int)(wpos % kTcWideSlots);
            wwphase ^= (wpos / kTcWideSlots) & 1u;
            if (!ok) return;
            rc.idx += gridDim.x;
            rc.seek(p);
            continue;
        }
        if (rc.gemm) {
            // tile GEMM: one weight k-tile (128 rows x 64 K-elements, 16 KB) per slot -- one plain bulk
            // copy when the weights are packed, one bulk tensor copy otherwise.  Eight single-tile
            // slots rather than two large ones: a slot is refilled the moment its tile has been
            // consumed, so ~100 KB stay in flight.  The instruction's tiles are issued from this tight
            // loop by four lanes at once, lane l taking tiles l, l + 4, ...: one lane's wait / expect /
            // copy sequence takes ~0.2 us (measured: 16 KB copies from one thread top out at 68 GB/s
            // however many are in flight), more than the MMAs of a tile; walking the outer loop (cursor,
            // warp votes) once per tile cost ~950 cycles.
            if (!enter(MODE_WTILES)) return;
            constexpr int kLanes = 4;
            const unsigned long long wpol = rc.reread ? keep_policy : stream_policy;
            bool mine = true;
            if (lane < kLanes) {
                const uint8_t* src = rc.wpack ? rc.wpack + rc.wtile0 * (long long)kTcTileBytes : nullptr;
                const long long kstep = (long long)rc.wstride * kTcTileBytes;
                uint32_t sl = (uint32_t)wslot + lane, ph = wphase;
                if (sl >= kTcWSlots) { sl -= kTcWSlots; ph ^= 1u; }
#pragma unroll 1
                for (int kt = lane; kt < rc.nk; kt += kLanes) {
                    if (!wait_barrier(p, c, &c->w_empty[sl], ph ^ 1u, rc.seq, WHERE_RING_EMPTY)) { mine = false; break; }
                    uint8_t* dst = ring + tc_wslot_off(sl);
                    if (!check_phase(p, c, &c->w_full[sl], ph, rc.seq, WHERE_CHECK_ARM)) { mine = false; break; }
                    mbar_arrive_expect_tx(&c->w_full[sl], (uint32_t)kTcTileBytes);
                    const int ktile = rc.wide == 2 ? kt >> 1 : kt, half = rc.wide == 2 ? kt & 1 : 0;
                    if (src) bulk_g2s_hint(dst, src + ktile * kstep + half * kTcTileBytes, (uint32_t)kTcTileBytes, &c->w_full[sl], wpol);
                    else tma_load_2d(dst, rc.wmap, rc.kbeg + ktile * 64, rc.n0 + half * 128, &c->w_full[sl], wpol);
                    sl += kLanes;
                    if (sl >= kTcWSlots) { sl -= kTcWSlots; ph ^= 1u; }
                }
            }
            const bool ok = __all_sync(0xffffffffu, mine);
            const uint32_t wpos = (uint32_t)wslot + (uint32_t)rc.nk;
            wslot = (int)(wpos % kTcWSlots);
            wphase ^= (wpos / kTcWSlots) & 1u;
            if (!ok) return;
            rc.idx += gridDim.x;
            rc.seek(p);
            continue;
        }
        if (!enter(MODE_STAGES)) return;
        // one lane looks whether the ring has a free stage (non-blocking)
        int free_now = 0;
        if (lane == 0) free_now = mbar_try_wait(&c->empty[pos.stage], pos.phase ^ 1u) ? 1 : 0;
        free_now = __shfl_sync(0xffffffffu, free_now, 0);
        if (!free_now && ahead < p.pf_stages && pc.valid(p)) {
            // ring full: let L2 fetch a stage further down the stream
            if (ahead == 0) { pc = rc; }
            const __nv_bfloat16* src; int bytes, off;
            pc.piece(lane, src, bytes, off);
            if (bytes) bulk_prefetch_l2(src, (uint32_t)bytes);
            pc.advance(p);
            ++ahead;
            continue;
        }
        if (!free_now) {
            int ok = 1;
            if (lane == 0) ok = wait_barrier(p, c, &c->empty[pos.stage], pos.phase ^ 1u, rc.seq, WHERE_RING_EMPTY) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, ok, 0)) return;
        }
        const __nv_bfloat16* src; int bytes, off;
        rc.piece(lane, src, bytes, off);
        const int total = __reduce_add_sync(0xffffffffu, bytes);
        if (lane == 0) mbar_arrive_expect_tx(&c->full[pos.stage], (uint32_t)total);
        __syncwarp();
        if (bytes) bulk_g2s_hint(ring + pos.stage * kStageBytes + off, src, (uint32_t)bytes, &c->full[pos.stage], stream_policy);
        if (TRACE && rc.g == 0 && rc.seg == 0) { t_first = (long long)globaltimer(); slot_first = (rc.idx - blockIdx.x) / gridDim.x; }
        const bool last = rc.g == rc.ngroups - 1 && rc.seg == rc.nseg - 1;
        if (TRACE && last && lane == 0) trace_rec<TRACE>(p, 0, slot_first, rc.seq, t_first, t_first, (long long)globaltimer());
        pos.advance();
        rc.advance(p);
        if (ahead > 0) --ahead;
    }
}

}  // namespace mk
