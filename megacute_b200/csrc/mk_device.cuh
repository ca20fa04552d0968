// Device-side building blocks of the persistent megakernel: PTX wrappers, bounded waits,
// dependency counters, trace records.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/megacute_b200.h"

namespace mk {

// ---- CTA shape (mirrors megacute_b200/config.py) --------------------------------------------
constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kThreads = kComputeThreads + 96;           // + one producer warp + one finisher warp + one feeder warp
constexpr int kProducerWarp = kComputeWarps;
constexpr int kFinisherWarp = kComputeWarps + 1;
constexpr int kFeederWarp = kComputeWarps + 2;           // tile requests and MMA issue of the tcgen05 prefill attention

// ---- shared memory map -----------------------------------------------------------------------
constexpr int kGemvRows = 8;                              // weight rows per ring stage
constexpr int kGemvKChunk = 2048;                         // elements of a row per stage (8 per thread)
// A ring stage holds 16 weight-row segments of 2048 elements, each padded by 16 bytes so that the
// 8 rows an ldmatrix touches fall in different banks (tensor-core path), or 8 rows x 2048 elements
// (general path).  Two large stages rather than several small ones: measured with a consumer that
// only waits and releases, a ring of 4 x (16 x 2 KB bulk copies) tops out at 4.7 TB/s, 2 x (16 x
// 4 KB) reaches 6.8 TB/s in the same shared memory: copies of 4 KB and up and fewer stage
// hand-overs per byte are what the copy engine needs.
constexpr int kSegElems = 2048;
constexpr int kSegStride = kSegElems * 2 + 16;            // bytes between row segments of a stage
constexpr int kStageBytes = 16 * kSegStride;              // 65 792 B
constexpr int kStages = 2;
constexpr int kRingBytes = kStages * kStageBytes;         // 128.5 KB, written only by bulk copies
constexpr int kWorkBytes = 96 * 1024 + 512;               // scratch of the instruction being executed (with the 512 bytes in front of
                                                          // its first 1024-byte boundary: six whole 16 KB operand tiles)
constexpr int kXbufBytes = 64 * 1024;                     // GEMV: fp32 activation rows (front of work)
constexpr int kCtrlBytes = 2048;                          // mbarriers, flags, staged instruction metadata
constexpr int kSmemBytes = kRingBytes + kWorkBytes + kCtrlBytes;
// tcgen05 tile GEMM (op_gemm_tc.cuh): operand tiles are 128 rows x 64 bf16 with the 128-byte swizzle
// and must start on 1024-byte boundaries.  Weight tiles travel through the ring's memory as eight
// single-tile slots with barriers of their own (the producer drains one kind of slot -- these, or
// the streaming linear's two stages -- before it fills the other kind); activation tiles use the
// work area.
constexpr int kTcTileBytes = 128 * 128;
constexpr int kTcXStages = 6;                             // activation stages of 128 rows ...
constexpr int kTcXHalfStages = 10;                        // ... or of 64 rows (ops with at most 64): the MMA still reads 128 rows from a
                                                          // stage's start, so half a tile of the work area must follow the last one
constexpr int kTcXOff = 512;                              // first 1024-aligned byte of the work area
constexpr int kTcCols = 512;                              // tensor-memory columns held by the CTA: a 128 x 256 accumulator (tile GEMM),
                                                          // or two S tiles and O (prefill attention)
constexpr uint32_t kTcNoTmem = 0xffffffffu;               // Ctrl::tmem_base before the CTA's first allocation
static_assert((kRingBytes + kTcXOff) % 1024 == 0 && kTcXOff + kTcXStages * kTcTileBytes <= kWorkBytes &&
                  kTcXOff + (kTcXHalfStages + 1) * (kTcTileBytes / 2) <= kWorkBytes && kTcXHalfStages <= 2 * kTcXStages,
              "activation tiles");
// many-sequence decode attention (op_decode_bulk.cuh): the ring's memory as seven slots, each one tile of
// 16 whole cache rows (at most 1 KB each) stored as four 4-row groups 32 bytes apart beyond their size.
// A third kind of slot beside the streaming linear's stages and the tile GEMM's weight slots: the
// producer warp drains one kind before it fills another.
constexpr int kKvSlots = 7;
constexpr int kKvSlotBytes = 4 * (4 * 1024 + 32);
static_assert(kKvSlots * kKvSlotBytes <= kRingBytes, "KV slots exceed the ring");
constexpr int kKvTileRows = 16;
constexpr int kKvGroupRows = 4;
constexpr int kKvGroupSkew = 32;                          // bytes between groups beyond their size
// rows [k_begin, k_end) of a sequence's n cached keys that split s of S attends; multiples of 16 so that
// tiles never straddle the end of a sequence's cache rows (max_seq is a multiple of 128)
__host__ __device__ inline void kv_split_range(int n, int S, int s, int& k_begin, int& k_end) {
    const int per = (((n + S - 1) / S) + kKvTileRows - 1) / kKvTileRows * kKvTileRows;
    k_begin = s * per < n ? s * per : n;
    k_end = k_begin + per < n ? k_begin + per : n;
}
constexpr int kTcWSlots = 8;
constexpr int kTcWideSlots = 4;                           // ... of a 128 x 256 tile: the same memory as pairs of slots (256 rows x 64 K-elements, 32 KB)
constexpr int kTcIssuers = 2;                             // threads that issue tcgen05.mma, each into an accumulator of its own
// k-tiles alternate between the issuing threads, and a thread waits for a stage or slot by the parity of its barrier's
// phase: that is only sound if the same thread consumed the stage's previous round (a thread waiting one round early
// would find the parity of the round before that complete and read a tile still in flight -- with five activation
// stages this happened, rarely, as a hang or a launch failure).  So every stage count is a multiple of the issuers.
static_assert(kTcXStages % kTcIssuers == 0 && kTcXHalfStages % kTcIssuers == 0 && kTcWSlots % kTcIssuers == 0 && kTcWideSlots % kTcIssuers == 0, "stage counts vs issuing threads");
__host__ __device__ constexpr int tc_wslot_off(int slot) { return slot * kTcTileBytes; }
static_assert(kTcWSlots * kTcTileBytes <= kRingBytes, "weight slots");

struct Params {
    const int4* insts;            // [n_insts][4]
    int n_insts;
    const int2* waits;            // (counter, target)
    const int* arrives;
    int* counters;
    const mk_op_desc* ops;
    int n_ops;
    long long* trace;             // [grid][kTraceRoles][cap][4] or null
    int trace_cap;
    int* status;                  // MK_ST_WORDS words; word 0 != 0 aborts every waiter
    int epoch;
    unsigned long long timeout_ns;
    int pf_stages;                // how many ring stages ahead of the ring the producer prefetches into L2
};

// Instruction metadata staged in shared memory one instruction ahead of its use.  Everything an
// instruction needs before its first useful load (its words, its op descriptor, its wait and
// arrival lists) would otherwise be a chain of dependent global loads, each a round trip to L2 or
// DRAM on the critical path between two dependent instructions.
constexpr int kMetaWaits = 16;    // longer lists are read from global memory
constexpr int kMetaArrives = 8;
struct Meta {
    mk_op_desc desc[2];           // current / next instruction's op
    int4 inst[3][4];              // rows of the current and the next two instructions
    int2 waits[2][kMetaWaits];
    int arrives[2][kMetaArrives];
};

struct AttnBars {                 // tcgen05 prefill attention (op_attention_tc.cuh): re-initialised by every instruction
    unsigned long long q_full, k_full[2], k_empty[2], v_full, v_empty, s_full[2], s_empty[2], p_full, pv_done;
};

struct Ctrl {                     // lives in the last kCtrlBytes of shared memory
    Meta meta;
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long slot_full[4];  // streaming linear: the 8 compute warps have deposited a row group's partial tiles
    unsigned long long slot_free[4];  // ... the finisher warp has read them
    unsigned long long epi_done;      // ... the finisher has issued the instruction's last stores (its arrivals follow)
    unsigned long long deps_met;      // ... the compute warps have seen the instruction's dependencies met
    unsigned long long x_full[2 * kTcXStages];   // tcgen05 tile GEMM: an activation k-tile has landed in the work area
    unsigned long long x_empty[2 * kTcXStages];  // ... the MMAs that read it have completed
    unsigned long long w_full[kTcWSlots];    // ... a weight k-tile has landed in its slot of the ring
    unsigned long long w_empty[kTcWSlots];   // ... the MMAs that read it have completed
    unsigned long long ww_full[kTcWideSlots];    // ... the same for the 32 KB slots of 128 x 256 tiles (barriers and positions of their
    unsigned long long ww_empty[kTcWideSlots];   //     own: the producer drains one kind before it fills the other)
    unsigned long long acc_full;      // ... every MMA of the instruction has completed (one arrival per issuing thread)
    unsigned long long kv_full[kKvSlots];    // many-sequence decode attention: a K or V tile has landed in its slot
    unsigned long long kv_empty[kKvSlots];   // ... every compute warp has read it
    unsigned long long kv_go;                // ... (unfused form) the instruction's dependencies are met: the row appended in this launch may be read
    uint32_t kv_cons;                        // ... the compute warps' position in the slots (slot | phase << 8)
    AttnBars attn;
    unsigned long long attn_go;              // tcgen05 prefill attention: the compute warps are at the instruction (dependencies met,
                                             // barriers initialised); the feeding thread of the producer warp may start
    uint32_t tmem_base;               // ... tensor-memory address of the accumulator (written by tcgen05.alloc)
    uint32_t tmem_ready;              // ... 1 once it is allocated; written behind the barrier that follows the allocation, so all
                                      //     threads of an instruction read the same value (tmem_base changes while they arrive)
    uint32_t x_par;                       // ... bit s: parity of the next completion of x_full[s] and of x_empty[s] (between
                                          //     instructions both have completed equally often); set at an instruction's end
    uint8_t w_slot, w_phase;              // ... the MMA thread's position in the weight slots
    uint8_t ww_slot, ww_phase;            // ... and in the 32 KB slots
    uint32_t acc_uses;                // ... instructions that have used acc_full (its parity)
    int abort;                    // set once a wait of this CTA gave up or saw the global abort
    int flag;                     // scratch broadcast word (split-KV last arriver)
    long long t_dep;              // tracing: when the dependencies of the current instruction were met
    long long t_fetch;            // tracing: when a body that keeps the walk (walk.cuh) turned to the current instruction
    int run_idx;                  // index of the instruction such a body is executing
    long long t_pub;              // tracing: when its arrivals were published (0: the op left no mark)
    long long t_phase[3];         // tracing: op-internal phase marks (role 2 records)
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "Ctrl outgrew its shared-memory slot");
constexpr int kTraceRoles = 3;    // 0 producer, 1 compute, 2 op-internal phases
__device__ __forceinline__ void phase_mark(const Params& p, Ctrl* c, int k);

// ---- small PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking form.  Measured on B200 in a stand-alone loop: a try_wait costs its thread ~95 ns even when
// the phase is already complete (it may suspend the thread), a test_wait ~1 ns; whatever the thread that
// issues tcgen05.mma or bulk copies executes between two of them leaves the pipe it feeds idle, so every
// wait below first asks with test_wait.
__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier (no multicast).
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Same with an L2 eviction policy (createpolicy).  Streamed weights are read once per launch and
// are many times the size of L2; marking them evict-first keeps them from pushing out what is
// read again soon: instruction tables, op descriptors, activations and the KV cache.
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, unsigned long long* bar,
                                              unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// 2-D tiled bulk tensor copy global -> shared through a tensor map (no multicast), with an L2
// eviction policy.  x is the innermost coordinate in elements; x times the element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int x, int y, unsigned long long* bar,
                                            unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    int sz = valid ? 16 : 0;      // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_small(void* dst, const void* src, int bytes) {      // 4 or 8 bytes
    if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// named barrier over the compute warps only (the producer warp never joins it)
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float sigmoidf_(float x) { return rcp(1.0f + ex2(-x * kLog2e)); }

// activation codes (config.py ACT_CODE)
enum { ACT_NONE = 0, ACT_RELU, ACT_SILU, ACT_GELU, ACT_EXP, ACT_NEG, ACT_SIGMOID, ACT_SQUARE, ACT_SWIGLU };
__device__ __forceinline__ float apply_act(int act, float x) {
    switch (act) {
        case ACT_RELU: return fmaxf(x, 0.0f);
        case ACT_SILU: return x * sigmoidf_(x);
        case ACT_GELU: return 0.5f * x * (1.0f + tanh_approx(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        case ACT_EXP: return ex2(x * kLog2e);
        case ACT_NEG: return -x;
        case ACT_SIGMOID: return sigmoidf_(x);
        case ACT_SQUARE: return x * x;
        default: return x;
    }
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float round_f16(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Element types of activations (descriptor dtype codes; graph.py DTYPE_CODE): 0 bf16, 1 fp32, 2 fp16.
// fp16 is what runtime-private activations that feed a tile GEMM are kept in: the tensor core takes it
// as it takes bf16, with 11 instead of 8 significant bits; conversions saturate at +-65504.
enum { DT_BF16 = 0, DT_F32 = 1, DT_F16 = 2 };
__device__ __forceinline__ uint32_t pack2h(float a, float b) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}
__device__ __forceinline__ float2 unpack2h(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
// two consecutive values in the 16-bit type `dtype` (DT_BF16 or DT_F16)
__device__ __forceinline__ uint32_t pack2t(int dtype, float a, float b) { return dtype == DT_F16 ? pack2h(a, b) : pack2(a, b); }
// load 8 consecutive elements as fp32 from a bf16, fp32 or fp16 row; 16-byte aligned.
// Loads go to L2 (ld.global.cg): activations are rewritten by other SMs inside one launch and L1
// is not coherent, so a line cached by an earlier instruction of this SM could be stale.
__device__ __forceinline__ void load8(const void* base, long long elem, int dtype, float* f) {
    if (dtype == DT_BF16) {
        uint4 v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem));
        unpack8(v, f);
    } else if (dtype == DT_F16) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(base) + elem));
        const float2 a = unpack2h(v.x), b = unpack2h(v.y), c = unpack2h(v.z), d = unpack2h(v.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem);
        float4 a = __ldcg(p), b = __ldcg(p + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}
// The same in two steps, so that a loop can request several vectors before it uses the first: the raw 16 or 32
// bytes (one or two 16-byte loads in flight per call), converted later.  A pointwise instruction is a handful of
// vectors per thread; requested one by one, each waits for its own L2 round trip (measured: a 32 x 512 modulate
// tile, 8 vectors per thread, took 8.6 us).
struct Raw8 { uint4 lo, hi; };
__device__ __forceinline__ Raw8 load8_raw(const void* base, long long elem, int dtype) {
    Raw8 r;
    if (dtype == DT_F32) {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + elem);
        r.lo = __ldcg(p); r.hi = __ldcg(p + 1);
    } else {
        r.lo = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + elem));
        r.hi = r.lo;
    }
    return r;
}
__device__ __forceinline__ void unpack8_raw(const Raw8& r, int dtype, float* f) {
    if (dtype == DT_BF16) {
        unpack8(r.lo, f);
    } else if (dtype == DT_F16) {
        const float2 a = unpack2h(r.lo.x), b = unpack2h(r.lo.y), c = unpack2h(r.lo.z), d = unpack2h(r.lo.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    } else {
        f[0] = __uint_as_float(r.lo.x); f[1] = __uint_as_float(r.lo.y); f[2] = __uint_as_float(r.lo.z); f[3] = __uint_as_float(r.lo.w);
        f[4] = __uint_as_float(r.hi.x); f[5] = __uint_as_float(r.hi.y); f[6] = __uint_as_float(r.hi.z); f[7] = __uint_as_float(r.hi.w);
    }
}
__device__ __forceinline__ void store8(void* base, long long elem, int dtype, const float* f) {
    if (dtype == DT_BF16) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + elem) = pack8(f);
    } else if (dtype == DT_F16) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(base) + elem) =
            make_uint4(pack2h(f[0], f[1]), pack2h(f[2], f[3]), pack2h(f[4], f[5]), pack2h(f[6], f[7]));
    } else {
        float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + elem);
        p[0] = make_float4(f[0], f[1], f[2], f[3]);
        p[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}
__device__ __forceinline__ float load1(const void* base, long long elem, int dtype) {
    if (dtype == DT_F32) return __ldcg(reinterpret_cast<const float*>(base) + elem);
    const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(base) + elem);
    if (dtype == DT_F16) return __half2float(__ushort_as_half(u));
    return __uint_as_float((uint32_t)u << 16);
}
__device__ __forceinline__ void store1(void* base, long long elem, int dtype, float v) {
    if (dtype == DT_BF16) reinterpret_cast<__nv_bfloat16*>(base)[elem] = __float2bfloat16_rn(v);
    else if (dtype == DT_F16) reinterpret_cast<unsigned short*>(base)[elem] = (unsigned short)(pack2h(v, 0.f) & 0xffffu);
    else reinterpret_cast<float*>(base)[elem] = v;
}

// ---- error reporting and bounded waits ---------------------------------------------------------
// Every spin in the kernel goes through one of the two waits below.  A wait gives up when the
// global abort word is set or when it has spun longer than Params::timeout_ns; it then records
// who gave up (first writer wins), raises the global abort word so every other waiter leaves too,
// and returns false.  Callers keep going through their barriers and leave at the next uniform
// check of Ctrl::abort, so a failed launch always terminates and the context stays usable.
__device__ __forceinline__ void report(const Params& p, Ctrl* c, int code, int seq, int where, int a, int b, int cc) {
    c->abort = 1;
    if (atomicCAS(&p.status[MK_ST_CODE], 0, code) == 0) {
        p.status[MK_ST_CTA] = blockIdx.x;
        p.status[MK_ST_WARP] = threadIdx.x >> 5;
        p.status[MK_ST_SEQ] = seq;
        p.status[MK_ST_WHERE] = where;
        p.status[MK_ST_A] = a;
        p.status[MK_ST_B] = b;
        p.status[MK_ST_C] = cc;
        __threadfence();
    }
}

enum { WHERE_RING_FULL = 1, WHERE_RING_EMPTY = 2, WHERE_DEP = 3, WHERE_DRAIN = 4, WHERE_COMBINE = 5, WHERE_CHECK_ARM = 6, WHERE_CHECK_RELEASE = 7 };

// `patience`: multiple of the time limit this wait allows.  A role that by design waits through everything the CTA does
// before (the finisher warp, for the dependencies of a streaming linear far down the program) gives twice the limit, so
// that when something earlier is stuck, the wait that is stuck reports first.
__device__ __forceinline__ bool wait_barrier(const Params& p, Ctrl* c, unsigned long long* bar, uint32_t parity,
                                             int seq, int where, unsigned patience = 1) {
    if (mbar_test_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0) {
            if (*(volatile int*)&c->abort) return false;
            if (ld_volatile(&p.status[MK_ST_CODE]) != 0) { c->abort = 1; return false; }
            unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.timeout_ns * patience) {
                report(p, c, MK_DEV_TIMEOUT_BARRIER, seq, where, (int)(bar - c->full), (int)parity, 0);
                return false;
            }
        }
    }
}

// -DMK_CHECK builds (libmegacute_b200_check.so; the package loads it when MEGACUTE_B200_CHECK=1): before a barrier of a
// producer / consumer pair is armed (arrive.expect_tx) or released (tcgen05.commit, arrive) for the phase of parity
// `parity`, the phase before it must be complete -- else the hand-off protocol has lost count (a slot filled twice, a
// release for a fill that never came), which otherwise shows as a hang or as corrupted operands much later.  The
// check records the barrier and ends the launch; without MK_CHECK it compiles to nothing.
__device__ __forceinline__ bool check_phase(const Params& p, Ctrl* c, unsigned long long* bar, uint32_t parity, int seq, int where) {
#ifdef MK_CHECK
    if (!mbar_test_wait(bar, parity ^ 1u)) {
        report(p, c, MK_DEV_CHECK, seq, where, (int)(bar - c->full), (int)parity, 0);
        return false;
    }
#endif
    return true;
}

__device__ __forceinline__ bool wait_counter(const Params& p, Ctrl* c, int counter, int target, int seq) {
    const int* addr = p.counters + counter;
    const int want = target * p.epoch;
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        int v = ld_acquire(addr);
        if (v >= want) return true;
        if ((it & 63u) == 0) {
            if (*(volatile int*)&c->abort) return false;
            if (ld_volatile(&p.status[MK_ST_CODE]) != 0) { c->abort = 1; return false; }
            unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.timeout_ns) {
                report(p, c, MK_DEV_TIMEOUT_COUNTER, seq, WHERE_DEP, counter, v, want);
                return false;
            }
        }
    }
}

// One decoded instruction, held in registers (never address-taken, so it is never demoted to
// local memory: with 227 KB of the SM given to shared memory the L1 left for local traffic is tiny).
struct Inst {
    int opi;                      // 1 + op index
    int a0, a1, a2, a3;           // op-specific arguments
    int nwait, wait_off, narrive, arrive_off, seq;
};
__device__ __forceinline__ Inst decode_inst(const int4* row) {      // row in shared memory
    const int4 w0 = row[0], w1 = row[1], w2 = row[2], w3 = row[3];
    Inst i;
    i.opi = w0.x; i.a0 = w0.y; i.a1 = w0.z; i.a2 = w0.w; i.a3 = w1.x;
    i.nwait = w2.x; i.wait_off = w2.y; i.narrive = w2.z; i.arrive_off = w2.w; i.seq = w3.x;
    return i;
}
__device__ __forceinline__ Inst fetch_inst(const Params& p, int idx) {
    const int4* src = p.insts + (long long)idx * 4;
    const int4 w0 = __ldg(src), w1 = __ldg(src + 1), w2 = __ldg(src + 2), w3 = __ldg(src + 3);
    Inst i;
    i.opi = w0.x; i.a0 = w0.y; i.a1 = w0.z; i.a2 = w0.w; i.a3 = w1.x;
    i.nwait = w2.x; i.wait_off = w2.y; i.narrive = w2.z; i.arrive_off = w2.w; i.seq = w3.x;
    return i;
}

// Barrier over the compute warps that also ORs a predicate: the result is the same in every thread.
__device__ __forceinline__ bool compute_sync_or(int pred) {
    int out;
    asm volatile(
        "{ .reg .pred p, q; setp.ne.s32 p, %1, 0; bar.red.or.pred q, 1, %2, p; selp.s32 %0, 1, 0, q; }"
        : "=r"(out)
        : "r"(pred), "n"(kComputeThreads)
        : "memory");
    return out != 0;
}

// All compute threads call this.  Threads take waits round-robin.  Returns (uniformly) whether
// the CTA is aborting.  wait_off < 0 names the staged list Meta::waits[-1 - wait_off].
__device__ __forceinline__ bool wait_deps(const Params& p, Ctrl* c, int nwait, int wait_off, int seq) {
    const int2* tab = wait_off < 0 ? c->meta.waits[-1 - wait_off] : p.waits + wait_off;
    for (int k = threadIdx.x; k < nwait; k += kComputeThreads) {
        const int2 w = tab[k];
        wait_counter(p, c, w.x, w.y, seq);
    }
    return compute_sync_or(*(volatile int*)&c->abort);
}
// All compute threads call this after their global writes of the instruction.  Returns
// (uniformly) whether the CTA is aborting; arrivals are skipped in that case.
// arrive_off < 0 names the staged list Meta::arrives[-1 - arrive_off].  The barrier also ends the
// instruction for the metadata staging: copies issued for the next instruction are waited for
// before it, so every thread sees them after it.
__device__ __forceinline__ bool publish(const Params& p, Ctrl* c, int narrive, int arrive_off) {
    asm volatile("cp.async.wait_all;" ::: "memory");
    // The staged list is read before the barrier: after it, the staging for the instruction after
    // next may already be overwriting the list.
    const int* tab = arrive_off < 0 ? c->meta.arrives[-1 - arrive_off] : p.arrives + arrive_off;
    const int first = (int)threadIdx.x < narrive ? tab[threadIdx.x] : -1;
    // The barrier orders every compute thread's global writes before the arriving threads'
    // red.release.gpu, whose release is cumulative over them: no per-thread gpu-scope fence needed.
    if (compute_sync_or(*(volatile int*)&c->abort)) return true;
    if (first >= 0) red_release_add(p.counters + first, 1);
    for (int k = threadIdx.x + kComputeThreads; k < narrive; k += kComputeThreads) red_release_add(p.counters + tab[k], 1);
    // The arriving lanes rejoin their warp here: a tail "if (lane arrives) red; return" may be compiled as an early return
    // of the other lanes, and the .sync.aligned instructions of the next op body (tcgen05.alloc / ld, mma.sync) want the
    // whole warp together.
    __syncwarp();
    return false;
}

// An op body is a function of another translation unit, called through the ABI: on entry it saves the callee-saved
// registers it is going to use to local memory and on return it loads them back -- for the tile GEMM 62 registers
// of 256 threads, 63 KB each way, with almost no L1 to hold them.  Measured on batch-64 decode: 1.4 us from the end
// of the dependency wait to the body's first statement.  So the bodies with a large frame (tile GEMM; the streaming
// linear and decode attention always did) wait for the instruction's dependencies themselves, behind their entry, and
// publish its arrivals before they return: both transfers then run while the CTA would be waiting for other SMs
// anyway (batch-64 decode 1.364 -> 1.31 ms).  With the wait right behind a barrier, the warps reach the body's first
// statements with empty memory queues and a few hundred cycles apart at times: whatever a body decides there must
// be decided on words that only change behind a barrier (Ctrl::tmem_ready, not the address tcgen05.alloc writes).
struct Sync {
    int nwait, wait_off, narrive, arrive_off;
};
__device__ __forceinline__ bool begin_op(const Params& p, Ctrl* c, const Sync& s, int seq) {
    const bool aborting = wait_deps(p, c, s.nwait, s.wait_off, seq);
    if (p.trace_cap > 0 && threadIdx.x == 0) c->t_dep = (long long)globaltimer();
    return aborting;
}
__device__ __forceinline__ bool end_op(const Params& p, Ctrl* c, const Sync& s) {
    const bool aborting = publish(p, c, s.narrive, s.arrive_off);
    if (p.trace_cap > 0 && threadIdx.x == 0) c->t_pub = (long long)globaltimer();
    return aborting;
}

// Instruction metadata runs one instruction ahead in shared memory (Meta): while instruction i executes, warp 1 has
// asynchronous copies in flight for the row of i + 2 and, from the already staged row of i + 1, for that
// instruction's op descriptor, waits and arrivals.  The barrier that ends instruction i (publish) makes them visible.
__device__ __forceinline__ void stage_row(const Params& p, Meta* mt, int idx, int s3, int lane) {       // lanes 0..3 of the calling warp
    if (idx < p.n_insts && lane < 4) cp_async16(&mt->inst[s3][lane], p.insts + (long long)idx * 4 + lane, true);
}
__device__ __forceinline__ void stage_op(const Params& p, Meta* mt, int s3, int s2, int lane) {         // whole calling warp; row s3 must be visible already
    const int4 w0 = mt->inst[s3][0], w2 = mt->inst[s3][2];
    const int opi = w0.x - 1;
    if (opi >= 0 && opi < p.n_ops && lane < 16)
        cp_async16(reinterpret_cast<uint8_t*>(&mt->desc[s2]) + lane * 16, reinterpret_cast<const uint8_t*>(p.ops + opi) + lane * 16, true);
    if (w2.x <= kMetaWaits && lane < w2.x) cp_async_small(&mt->waits[s2][lane], p.waits + w2.y + lane, 8);
    if (w2.z <= kMetaArrives && lane >= 16 && lane - 16 < w2.z) cp_async_small(&mt->arrives[s2][lane - 16], p.arrives + w2.w + lane - 16, 4);
}

__device__ __forceinline__ void phase_mark(const Params& p, Ctrl* c, int k) {
    if (p.trace_cap > 0 && threadIdx.x == 0) c->t_phase[k] = (long long)globaltimer();
}

template <bool TRACE>
__device__ __forceinline__ void trace_rec(const Params& p, int role, int slot, long long seq, long long t0, long long t1,
                                          long long t2) {
    if constexpr (TRACE) {
        if (slot < p.trace_cap) {
            long long* r = p.trace + (((long long)blockIdx.x * kTraceRoles + role) * p.trace_cap + slot) * 4;
            r[0] = seq; r[1] = t0; r[2] = t1; r[3] = t2;
        }
    }
}

// the same with the tracing decided at run time (walk.cuh)
__device__ __forceinline__ void trace_rec_rt(const Params& p, int role, int slot, long long seq, long long t0, long long t1, long long t2) {
    if (slot < p.trace_cap) {
        long long* r = p.trace + (((long long)blockIdx.x * kTraceRoles + role) * p.trace_cap + slot) * 4;
        r[0] = seq; r[1] = t0; r[2] = t1; r[3] = t2;
    }
}

}  // namespace mk
