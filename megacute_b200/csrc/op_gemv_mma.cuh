// Compute-warp side of the tensor-core streaming linear (MK_OP_GEMV with GEMV_F_UNITS):
//   out[m][o] = act(rstd[m] * sum_k w[o][k] * (x[m][k] * gain[k]) + bias[o]) + residual[m][o],  m < M <= 8
// Stage layout, flag and producer side: op_gemv_common.cuh.
//
// The code is deliberately compact (rolled outer loops, one code path for every K): a decode step
// runs each op body once per instruction, so the bodies execute cold and a large unrolled body is
// paid for in instruction-cache misses (measured: "no instruction" was the top stall reason).
//
// Shared memory (work region):
//   xf       [M][K/16][4 lanes][4 words]: x * gain split into bf16 high and low parts, stored in
//            MMA B-fragment order: for k-step s and lane quad position j the 16 bytes are
//            {hi k=2j,2j+1 | hi k=2j+8,2j+9 | lo k=2j,2j+1 | lo k=2j+8,2j+9} of the 16 k of step s,
//            so a lane fetches its whole B operand of a k-step with one 128-bit load.  Rows are
//            padded by 64 bytes so the 8 activation rows of a quarter-warp hit different banks.
//   red      [4 slots][8 warps][32 lanes] float4: per-warp partial 16 x 8 tiles of a row group
//   rowstat  [8 warps][8 rows] partial sums of x^2
//
// The eight compute warps only stream: each deposits its partial tile of a row group in a slot and
// moves on to the next stage.  A ninth warp, the finisher (gemv_finisher below), adds the eight
// partials and runs the epilogue (rstd, bias, activation, swiglu, residual, store).  With the
// epilogue on a compute warp that warp is late for the next group by the epilogue's length, and
// since every group needs every warp's K slice each group costs MMA + combine + epilogue; the ring
// has only two stages, so a stage's period is (that + the refill latency) / 2.
// Hand-over per slot: Ctrl::slot_full (8 arrivals, one per compute warp) and Ctrl::slot_free (the
// finisher); Ctrl::epi_done tells the compute warps that the instruction's last store has left.
#pragma once
#include "mma.cuh"
#include "op_gemv_common.cuh"

namespace mk {

constexpr int kMmaRedOff = 66 * 1024;                      // xf takes at most 64 KB + 512 B
constexpr int kMmaStatOff = kMmaRedOff + 4 * 8 * 32 * 16;  // + 16 KB

__device__ __forceinline__ float4 lds_volatile4(const float4* p) {
    float4 v;
    asm volatile("ld.volatile.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ void sts_volatile4(float4* p, float4 v) {
    asm volatile("st.volatile.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(smem_u32(p)), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// The op waits for its own dependencies so that loads which depend on nothing in the launch (the
// norm gain) are already in flight when the wait ends.
__device__ __forceinline__ void gemv_mma(const Params& p, Ctrl* c, uint8_t* ring, uint8_t* work, const mk_op_desc* op,
                                         int o0, int o1, int seq, RingPos& pos, int nwait, int wait_off) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int M = op->i[0], K = op->i[2];
    const bool swi = op->flags & GEMV_F_SWIGLU, rms = op->flags & GEMV_F_RMS;
    const int S = (K + kSegElems - 1) / kSegElems;
    const int xrow = K * 4 + 64;                                              // bytes per activation row of xf
    uint8_t* xf = work;
    float4* red = reinterpret_cast<float4*>(work + kMmaRedOff);
    float* rowstat = reinterpret_cast<float*>(work + kMmaStatOff);

    // ---- before the dependency wait: the norm gain of this thread's first vectors ----
    const int nv = K >> 3;
    const uint4* gain = (rms && op->ptr[5]) ? reinterpret_cast<const uint4*>(op->ptr[5]) : nullptr;
    const uint4 ones = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    uint4 g0[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int v = t + i * kComputeThreads;
        g0[i] = (gain && v < nv) ? __ldg(gain + v) : ones;
    }
    // everything below that does not depend on the activations is also set up before the wait:
    // the op runs once per instruction, cold, and this code would otherwise sit between the
    // arrival of x and the first MMA
    const int n = o1 - o0;
    const int ngroups = (swi ? 2 : 1) * ((n + 15) / 16);
    constexpr int kSlice = kSegElems / kComputeWarps;                         // 256: a warp's K slice of a segment
    const int kw = warp * kSlice;
    // B operand (16 k x 8 columns).  Up to 4 activation rows: columns 0..3 carry the high parts of
    // rows 0..3 and columns 4..7 their low parts, so ONE MMA per k-step yields both products (they
    // are added in the epilogue).  5 to 8 rows: a column per row, high and low parts in two MMAs.
    const bool packed = M <= 4;
    const int bn = lane >> 2;                                                 // this lane's B column
    const int bm = packed ? (bn & 3) : bn;                                    // the activation row behind it
    const uint32_t a_lane = (uint32_t)((lane & 15) * kSegStride + ((lane >> 4) * 8) * 2 + kw * 2);
    const uint32_t b_lane = smem_u32(xf) + (bm < M ? bm : 0) * xrow + (kw >> 4) * 64 + (lane & 3) * 16 +
                            (packed ? (bn >> 2) * 8 : 0);
    const int xdt = op->i[4];
    const void* x = reinterpret_cast<const void*>(op->ptr[0]);
    const long long ldx = op->ld[0];
    if (wait_deps(p, c, nwait, wait_off, seq)) return;
    if (t == 0) {
        mbar_arrive(&c->deps_met);          // the finisher may now read the residual of the first row group
        if (p.trace_cap > 0) c->t_dep = (long long)globaltimer();
    }

    // ---- stage x * gain (high + low bf16 parts, fragment order); accumulate sum(x^2) per row ----
    {
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
            float ss = 0.f;
#pragma unroll 1
            for (int vb = 0; vb < nv; vb += 4 * kComputeThreads) {            // batches of 4 vectors per thread
                float f[4][8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {                                 // all loads of the batch first
                    const int v = vb + t + i * kComputeThreads;
                    if (v < nv) load8(x, m * ldx + v * 8, xdt, f[i]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int v = vb + t + i * kComputeThreads;
                    if (v < nv) {
                        float gq[8];
                        unpack8(vb == 0 ? g0[i] : (gain ? __ldg(gain + v) : ones), gq);
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float y0 = f[i][2 * j] * gq[2 * j], y1 = f[i][2 * j + 1] * gq[2 * j + 1];
                            ss += f[i][2 * j] * f[i][2 * j] + f[i][2 * j + 1] * f[i][2 * j + 1];
                            const float h0 = round_bf16(y0), h1 = round_bf16(y1);
                            hi[j] = pack2(h0, h1);
                            lo[j] = pack2(y0 - h0, y1 - h1);
                        }
                        uint32_t* d = reinterpret_cast<uint32_t*>(xf + m * xrow + (v >> 1) * 64 + (v & 1) * 4);
#pragma unroll
                        for (int j = 0; j < 4; ++j) { d[j * 4] = hi[j]; d[j * 4 + 2] = lo[j]; }
                    }
                }
            }
            if (rms) {
                ss = warp_sum(ss);
                if (lane == 0) rowstat[warp * 8 + m] = ss;
            }
        }
        compute_sync();
    }
    phase_mark(p, c, 0);
#pragma unroll 1
    for (int g = 0; g < ngroups; ++g) {
        // four independent accumulator tiles (even / odd k-step x high / low part of x) keep the
        // chain of dependent MMAs short; they are summed once per row group
        float accs[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) accs[q][e] = 0.f;
        bool ok = true;
#pragma unroll 1
        for (int seg = 0; seg < S; ++seg) {
            ok = wait_barrier(p, c, &c->full[pos.stage], pos.phase, seq, WHERE_RING_FULL) && ok;
            if (g == 0 && seg == 0) phase_mark(p, c, 1);
            int left = min(kSegElems, K - seg * kSegElems) - kw;              // K elements of this warp's slice
            if (ok) {
                uint32_t a_base = smem_u32(ring + pos.stage * kStageBytes) + a_lane;
                uint32_t b_base = b_lane + seg * (kSegElems / 16) * 64;
#pragma unroll 1
                for (int half = 0; half < kSlice / 128 && left > 0; ++half) {     // batches of 8 k-steps
                    uint32_t a[8][4];
                    // lanes of absent activation rows feed zeros and stay out of the load: with one
                    // row only a quarter of the warp touches shared memory
                    if (packed) {
                        uint2 b[8];
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            if (ks * 16 < left) {
                                ldmatrix_x4(a_base + ks * 32, a[ks][0], a[ks][1], a[ks][2], a[ks][3]);
                                b[ks] = bm < M ? lds64(b_base + ks * 64) : make_uint2(0u, 0u);
                            }
                        }
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            if (ks * 16 < left) mma_bf16(accs[ks & 3], a[ks], b[ks].x, b[ks].y);
                    } else {
                        uint4 b[8];
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            if (ks * 16 < left) {
                                ldmatrix_x4(a_base + ks * 32, a[ks][0], a[ks][1], a[ks][2], a[ks][3]);
                                b[ks] = bm < M ? lds128(b_base + ks * 64) : make_uint4(0u, 0u, 0u, 0u);
                            }
                        }
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            if (ks * 16 < left) {
                                mma_bf16(accs[(ks & 1) * 2], a[ks], b[ks].x, b[ks].y);
                                mma_bf16(accs[(ks & 1) * 2 + 1], a[ks], b[ks].z, b[ks].w);
                            }
                        }
                    }
                    a_base += 8 * 32;
                    b_base += 8 * 64;
                    left -= 128;
                }
            }
            // the stage goes back to the producer as soon as this warp has read its slice
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->empty[pos.stage]);
            pos.advance();
        }
        // ---- hand the partial tile to the finisher.  Four slots round-robin; a slot is reused
        // four groups later, once the finisher has freed it (it almost always has). ----
        const int sl = g & 3;
        ok = wait_barrier(p, c, &c->slot_free[sl], ((pos.comb >> sl) & 1u) ^ 1u, seq, WHERE_COMBINE) && ok;
        pos.comb ^= 1u << sl;
        sts_volatile4(&red[sl * (8 * 32) + warp * 32 + lane],
                      make_float4((accs[0][0] + accs[1][0]) + (accs[2][0] + accs[3][0]), (accs[0][1] + accs[1][1]) + (accs[2][1] + accs[3][1]),
                                  (accs[0][2] + accs[1][2]) + (accs[2][2] + accs[3][2]), (accs[0][3] + accs[1][3]) + (accs[2][3] + accs[3][3])));
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->slot_full[sl]);                        // release: the warp's deposit
    }
    // the instruction's results are in memory when the finisher says so
    wait_barrier(p, c, &c->epi_done, (pos.comb >> 4) & 1u, seq, WHERE_COMBINE);
    pos.comb ^= 16u;
    phase_mark(p, c, 2);
}

// The finisher warp: walks the CTA's instructions like the producer does and, for every streaming
// linear of the tensor-core path, turns the deposited partial tiles into outputs.
// Lane l holds rows ob = o0 + 16 * group + (l >> 2) and ob + 8, activation rows m0 = 2 * (l & 3), m0 + 1
// (the MMA result layout); with packed activations (M <= 4) lanes l & 3 >= 2 hold low-part products.
__device__ __forceinline__ void gemv_finisher(const Params& p, Ctrl* c, uint8_t* work) {
    const int lane = threadIdx.x & 31;
    const float4* red = reinterpret_cast<const float4*>(work + kMmaRedOff);
    const float* rowstat = reinterpret_cast<const float*>(work + kMmaStatOff);
    uint32_t fullpar = 0;                                                     // parities of slot_full[0..3], bit 4: deps_met
    for (int idx = blockIdx.x; idx < p.n_insts; idx += gridDim.x) {
        const Inst in = fetch_inst(p, idx);
        const int opi = in.opi - 1;
        if (opi < 0 || opi >= p.n_ops) return;
        const mk_op_desc* op = p.ops + opi;
        if (op->kind != MK_OP_GEMV || !(op->flags & GEMV_F_UNITS)) continue;
        const int M = op->i[0], K = op->i[2], act = op->i[3], odt = op->i[5], rdt = op->i[6];
        const bool swi = op->flags & GEMV_F_SWIGLU, rms = op->flags & GEMV_F_RMS;
        const int o0 = in.a0, o1 = in.a1, seq = in.seq;
        const int ngroups = (swi ? 2 : 1) * ((o1 - o0 + 15) / 16);
        const void* biasp = reinterpret_cast<const void*>(op->ptr[3]);
        const void* resp = reinterpret_cast<const void*>(op->ptr[4]);
        void* outp = reinterpret_cast<void*>(op->ptr[2]);
        const long long ldo = op->ld[2], ldr = op->ld[4];
        const float eps = op->f[0];
        const bool packed = M <= 4;
        const int m0 = 2 * (lane & 3);
        const bool storer = !(packed && (lane & 3) >= 2);
        float rs[2] = {1.f, 1.f};
        float gate[4] = {0.f, 0.f, 0.f, 0.f};
        // this lane's arrival target, read now so that it is in a register when the last store has left
        const int arrive_to = lane < in.narrive ? __ldg(p.arrives + in.arrive_off + lane) : -1;
        // Operands of the epilogue may be results of earlier instructions: nothing is read before
        // the compute warps have seen the instruction's dependencies met.
        bool ok = wait_barrier(p, c, &c->deps_met, (fullpar >> 4) & 1u, seq, WHERE_COMBINE, 2);
        fullpar ^= 16u;
        if (!ok) return;
#pragma unroll 1
        for (int g = 0; g < ngroups; ++g) {
            const int sl = g & 3;
            const int ob = o0 + (swi ? g >> 1 : g) * 16 + (lane >> 2);
            // epilogue operands are requested before the hand-over wait so their latency is hidden
            float bias_v[2] = {0.f, 0.f}, res_v[4] = {0.f, 0.f, 0.f, 0.f};
            auto fetch_operands = [&]() {
                if (swi || !storer) return;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int o = ob + h * 8;
                    if (o < o1) {
                        if (biasp) bias_v[h] = load1(biasp, o, 0);
                        if (resp) {
                            if (m0 < M) res_v[h * 2] = load1(resp, (long long)m0 * ldr + o, rdt);
                            if (m0 + 1 < M) res_v[h * 2 + 1] = load1(resp, (long long)(m0 + 1) * ldr + o, rdt);
                        }
                    }
                }
            };
            fetch_operands();
            ok = wait_barrier(p, c, &c->slot_full[sl], (fullpar >> sl) & 1u, seq, WHERE_COMBINE) && ok;
            fullpar ^= 1u << sl;
            if (!ok) return;                                                  // the launch is failing
            if (g == 0) {
                if (rms && storer) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        if (m0 + j < M) {
                            float sq = 0.f;
#pragma unroll
                            for (int w8 = 0; w8 < kComputeWarps; ++w8) sq += rowstat[w8 * 8 + m0 + j];
                            rs[j] = rsqrt_approx(sq / (float)K + eps);
                        }
                    }
                }
            }
            float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w8 = 0; w8 < kComputeWarps; ++w8) {
                const float4 q = lds_volatile4(&red[sl * (8 * 32) + w8 * 32 + lane]);
                v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->slot_free[sl]);                    // the slot has been read
            if (packed) {
                // columns 4..7 hold the low-part products of rows 0..3: add them to columns 0..3,
                // which sit two lanes further down in the quad
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] += __shfl_xor_sync(0xffffffffu, v[e], 2);
            }
            if (storer) {
                // v[0], v[1]: row ob, activation rows m0, m0 + 1;  v[2], v[3]: row ob + 8
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int o = ob + (e >> 1) * 8, m = m0 + (e & 1);
                    const float y = v[e] * rs[e & 1];
                    if (swi && !(g & 1)) {
                        gate[e] = y;
                    } else if (o < o1 && m < M) {
                        store1(outp, (long long)m * ldo + o, odt,
                               swi ? gate[e] * sigmoidf_(gate[e]) * y : apply_act(act, y + bias_v[e >> 1]) + res_v[e]);
                    }
                }
            }
        }
        // The instruction's arrivals leave from here, right behind its last store: __syncwarp orders
        // every lane's stores before the arriving lanes' red.release.gpu, whose release is cumulative
        // over them.  (More than 32 targets: the compute warps send the rest, see the wrapper.)
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->epi_done);                             // shared memory is free: the compute warps move on
        if (arrive_to >= 0) red_release_add(p.counters + arrive_to, 1);
    }
}

}  // namespace mk
