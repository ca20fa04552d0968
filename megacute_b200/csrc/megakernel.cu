// The persistent megakernel and its C ABI (include/megacute_b200.h).  sm_100a only.
//
// One launch executes a whole graph.  grid = number of SMs, one CTA per SM, 10 warps:
//   warps 0-7  compute: fetch this CTA's next instruction (global indices c, c+grid, ...), wait
//              for its dependency counters (acquire), run the op, publish its arrivals (release);
//   warp 8     producer: walks the same instruction list ahead of the compute warps and streams
//              the weight rows of every streaming linear (and the weight tiles of every tcgen05
//              tile GEMM) into shared memory with bulk copies, across instruction boundaries --
//              weights depend on nothing in the launch, so HBM keeps streaming while the compute
//              warps sit in a dependency hop;
//   warp 9     finisher: adds the compute warps' partial tiles of a streaming linear, runs its
//              epilogue and sends the instruction's arrivals.
// This replaces the reference's JIT-traced kernel (megacute/kernel.py:251-571) and its per-op
// role bodies (megacute/ops/*.py).
#include <cuda.h>          // CUtensorMap and cuTensorMapEncodeTiled's signature (resolved at run time, libcuda is not linked)

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "mk_device.cuh"
#include "mma.cuh"
#include "op_gemv_common.cuh"
#include "ops.cuh"
#include "walk.cuh"

namespace mk {

template <bool TRACE>
__global__ void __launch_bounds__(kThreads, 1) megakernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* ring = smem;
    Ctrl* c = reinterpret_cast<Ctrl*>(smem + kRingBytes + kWorkBytes);
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&c->full[s], 1);
            mbar_init(&c->empty[s], kComputeWarps);
        }
        for (int s = 0; s < 4; ++s) {
            mbar_init(&c->slot_full[s], kComputeWarps);
            mbar_init(&c->slot_free[s], 1);
        }
        mbar_init(&c->epi_done, 1);
        mbar_init(&c->deps_met, 1);
        for (int s = 0; s < 2 * kTcXStages; ++s) {
            mbar_init(&c->x_full[s], 1);
            mbar_init(&c->x_empty[s], 1);
        }
        c->x_par = 0;
        for (int s = 0; s < kTcWSlots; ++s) {
            mbar_init(&c->w_full[s], 1);
            mbar_init(&c->w_empty[s], 1);
        }
        c->w_slot = c->w_phase = 0;
        for (int s = 0; s < kTcWideSlots; ++s) {
            mbar_init(&c->ww_full[s], 1);
            mbar_init(&c->ww_empty[s], 1);
        }
        c->ww_slot = c->ww_phase = 0;
        mbar_init(&c->attn_go, 1);
        mbar_init(&c->acc_full, kTcIssuers);
        for (int s = 0; s < kKvSlots; ++s) {
            mbar_init(&c->kv_full[s], 1);
            mbar_init(&c->kv_empty[s], kComputeWarps);
        }
        mbar_init(&c->kv_go, 1);
        c->kv_cons = 0;
        c->acc_uses = 0;
        c->tmem_base = kTcNoTmem;
        c->tmem_ready = 0;
        c->abort = 0;
        c->flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kProducerWarp) {
        // ---------------- producer warp ----------------
        producer_loop<TRACE>(p, c, ring);
    } else if (warp == kFinisherWarp) {
        // ---------------- finisher warp: epilogues of the streaming linear ----------------
        mk_gemv_finisher(p);
    } else if (warp == kFeederWarp) {
        // ---------------- feeder warp: tiles and MMAs of the tcgen05 prefill attention ----------------
        // (a warp of its own rather than a branch of the producer's loop: the call in that loop cost every decode step
        // 0.5 %, whether or not the graph had such an op; here a graph without one costs a walk over the instruction list)
        mk_attention_feeder(p);
    } else {
        // ---------------- compute warps ----------------
        // Instruction metadata runs one instruction ahead in shared memory (Meta): while instruction
        // i executes, warp 1 has asynchronous copies in flight for the row of i + 2 and, from the
        // already staged row of i + 1, for that instruction's op descriptor, waits and arrivals.
        // The barrier that ends instruction i (publish) makes them visible to every thread.
        RingPos pos;
        int slot = 0;
        Meta* mt = &c->meta;
        const int lane = threadIdx.x & 31;
        if (warp == 1) {
            stage_row(p, mt, blockIdx.x, 0, lane);
            stage_row(p, mt, blockIdx.x + gridDim.x, 1, lane);
            cp_async_commit();
            cp_async_wait<0>();
            __syncwarp();
            if (blockIdx.x < p.n_insts) stage_op(p, mt, 0, 0, lane);
            cp_async_commit();
            cp_async_wait<0>();
        }
        compute_sync();
        for (int idx = blockIdx.x; idx < p.n_insts; idx += gridDim.x, ++slot) {
            const int s3 = slot % 3, s2 = slot & 1;
            const Inst in = decode_inst(mt->inst[s3]);
            if (warp == 1) {
                stage_row(p, mt, idx + 2 * gridDim.x, (slot + 2) % 3, lane);
                if (idx + gridDim.x < p.n_insts) stage_op(p, mt, (slot + 1) % 3, s2 ^ 1, lane);
                cp_async_commit();
            }
            const int opi = in.opi - 1;
            if (opi < 0 || opi >= p.n_ops) {
                if (threadIdx.x == 0) report(p, c, MK_DEV_BAD_INST, in.seq, 0, in.opi, idx, 0);
                break;
            }
            const mk_op_desc* op = &mt->desc[s2];
            const int wait_off = in.nwait <= kMetaWaits ? -1 - s2 : in.wait_off;
            const int arrive_off = in.narrive <= kMetaArrives ? -1 - s2 : in.arrive_off;
            const long long t0 = TRACE && threadIdx.x == 0 ? (long long)globaltimer() : 0;
            if (TRACE && threadIdx.x == 0) c->t_pub = 0;
            // the streaming linear, decode attention and the tile GEMM wait for the instruction's dependencies behind their
            // own entry and publish the arrivals before they return (begin_op / end_op say why); the kernel does both
            // around the bodies whose entry is cheap
                        const int ppos = pos.stage | ((int)pos.phase << 8);
            int npos = ppos;
            bool known = true, aborting = false, traced = false;
            switch (op->kind) {
                case MK_OP_GEMV:
                    if (op->flags & GEMV_F_UNITS) {
                        npos = mk_op_gemv_units(p, op, in.a0, in.a1, in.seq, ppos, in.nwait, wait_off, in.narrive, arrive_off);
                        aborting = npos < 0;
                    } else {
                        if (wait_deps(p, c, in.nwait, wait_off, in.seq)) { aborting = true; break; }
                        if (TRACE && threadIdx.x == 0) c->t_dep = (long long)globaltimer();
                        npos = mk_op_gemv_general(p, op, in.a0, in.a1, in.seq, ppos);
                        aborting = publish(p, c, in.narrive, arrive_off);
                    }
                    break;
                case MK_OP_GEMM: {
                    // (runs this instruction and the CTA's following ones for as long as they are the body's own: walk.cuh)
                    const int last = (op->i[10] == 256 && op->ptr[11]) ? mk_run_gemm_wide(p, idx) : mk_run_gemm(p, idx);
                    aborting = last < 0;
                    if (!aborting) {
                        slot += (last - idx) / (int)gridDim.x;
                        idx = last;
                    }
                    traced = true;
                    break;
                }
                case MK_OP_ATTENTION:
                    if (wait_deps(p, c, in.nwait, wait_off, in.seq)) { aborting = true; break; }
                    if (TRACE && threadIdx.x == 0) c->t_dep = (long long)globaltimer();
                    if (op->ptr[11]) aborting = mk_op_attention_tc(p, op, in.a0, in.a1, in.a2, in.seq) < 0;
                    else mk_op_attention(op, in.a0, in.a1, in.a2);
                    aborting = publish(p, c, in.narrive, arrive_off) || aborting;
                    break;
                case MK_OP_DECODE_ATTN:
                    aborting = mk_op_decode_attn(p, op, in.a0, in.a1, in.a2, in.nwait, wait_off, in.seq, in.narrive, arrive_off);
                    break;
                default:
                    if (wait_deps(p, c, in.nwait, wait_off, in.seq)) { aborting = true; break; }
                    if (TRACE && threadIdx.x == 0) c->t_dep = (long long)globaltimer();
                    known = mk_op_pointwise(op, in.a0, in.a1);
                    aborting = publish(p, c, in.narrive, arrive_off);
                    break;
            }
            if (!known && threadIdx.x == 0) report(p, c, MK_DEV_BAD_INST, in.seq, 1, op->kind, idx, 0);
            pos.stage = npos & 0xff;
            pos.phase = (uint32_t)(npos >> 8);
            if (TRACE && threadIdx.x == 0 && !traced) {
                const bool marks = op->kind == MK_OP_GEMV || op->kind == MK_OP_DECODE_ATTN || op->kind == MK_OP_GEMM || op->kind == MK_OP_ATTENTION;
                trace_rec<TRACE>(p, 1, slot, in.seq, t0, c->t_dep, c->t_pub ? c->t_pub : (long long)globaltimer());
                if (marks) trace_rec<TRACE>(p, 2, slot, in.seq, c->t_phase[0], c->t_phase[1], c->t_phase[2]);
            }
            if (aborting) break;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");      // staged metadata of instructions that never ran
    }
    __syncthreads();
    // Abort path only: bulk copies may still be landing in the ring.  Wait (bounded) for the
    // latest fill of every stage before the CTA gives its shared memory back.
    if (c->abort && threadIdx.x == kProducerWarp * 32) {
        for (int s = 0; s < kStages; ++s) {
            unsigned long long t0 = globaltimer();
            // a stage whose fill was issued has a pending phase; both parities are polled because
            // the role that knew the parity has already left its loop
            while (!(mbar_try_wait(&c->full[s], 0) || mbar_try_wait(&c->full[s], 1))) {
                if (globaltimer() - t0 > 20000000ull) break;      // 20 ms
            }
        }
        for (int s = 0; s < kTcWSlots; ++s) {
            unsigned long long t0 = globaltimer();
            while (!(mbar_try_wait(&c->w_full[s], 0) || mbar_try_wait(&c->w_full[s], 1))) {
                if (globaltimer() - t0 > 20000000ull) break;
            }
        }
        for (int s = 0; s < kTcWideSlots; ++s) {
            unsigned long long t0 = globaltimer();
            while (!(mbar_try_wait(&c->ww_full[s], 0) || mbar_try_wait(&c->ww_full[s], 1))) {
                if (globaltimer() - t0 > 20000000ull) break;
            }
        }
        for (int s = 0; s < kKvSlots; ++s) {                       // KV tiles of the many-sequence decode attention
            unsigned long long t0 = globaltimer();
            while (!(mbar_try_wait(&c->kv_full[s], 0) || mbar_try_wait(&c->kv_full[s], 1))) {
                if (globaltimer() - t0 > 20000000ull) break;
            }
        }
        unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) {}                  // let in-flight copies retire
    }
    __syncthreads();
    // tensor memory of the tile GEMM (allocated by the CTA's first such instruction) goes back here
    if (warp == 0 && c->tmem_base != kTcNoTmem) {
        __syncwarp();                       // (.sync.aligned: the whole warp, converged)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(c->tmem_base), "r"(kTcCols) : "memory");
    }
}

// Weight packing for the tcgen05 tile GEMM.  A bulk tensor copy of a 128-row x 64-column tile is 128
// row requests of 128 bytes, and the copy engine of an SM sustains only ~28 GB/s of such rows
// (measured: ~4 TB/s over the chip, whatever the depth of the pipeline), where one plain bulk copy of
// the same bytes runs at the HBM rate.  So the library keeps, per weight matrix, a copy laid out as
// the shared-memory images of its tiles: tile (n tile j, k tile t) is the 16 KB block t * ceil(N/128) + j,
// row r's 16-byte chunk c at r * 128 + ((c ^ (r & 7)) << 4) -- the 128-byte swizzle a bulk tensor
// copy would have applied.  Rows beyond N are zero.  One thread moves one 16-byte chunk.
// k-tile-major on purpose: the CTAs of an op walk K in step, each on its own n tile, so at any
// moment they read neighbouring blocks (one sequential stream over the chip) instead of addresses a
// large power of two apart.
// to_fp16: the copy holds the weights as fp16 -- for ops whose activations are fp16, because the tensor
// core wants both operands of one type.  Exact for every bf16 value of normal fp16 magnitude
// (6.1e-5 .. 65504); smaller ones land on fp16's subnormal grid (absolute error below 3e-8).
__global__ void pack_weight_tiles(const __nv_bfloat16* __restrict__ w, long long ld, int N, int K, uint4* __restrict__ out,
                                  long long chunks, int to_fp16) {
    const int kchunks = K / 8, ntiles = (N + 127) / 128;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / kchunks), kc = (int)(i % kchunks);
        const int j = row >> 7, r = row & 127, t = kc >> 3, c = kc & 7;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < N) v = __ldg(reinterpret_cast<const uint4*>(w + (long long)row * ld + (long long)kc * 8));
        if (to_fp16) v = make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
        out[((long long)t * ntiles + j) * (kTcTileBytes / 16) + r * 8 + (c ^ (r & 7))] = v;
    }
}

}  // namespace mk

// =================================================================================================
// Host side: C ABI
// =================================================================================================

struct mk_program {
    int device = 0;
    int grid = 0;
    int n_insts = 0, n_waits = 0, n_arrives = 0, n_counters = 0, n_ops = 0, trace_cap = 0;
    int32_t* d_insts = nullptr;
    int32_t* d_waits = nullptr;
    int32_t* d_arrives = nullptr;
    int32_t* d_counters = nullptr;
    mk_op_desc* d_ops = nullptr;
    uint8_t* d_tmaps = nullptr;      // per op: kMapBytes of 128-byte tensor maps (tile GEMM: activations, weights; attention: q, k, v)
    // Two pinned staging copies of the descriptor and tensor-map tables, used in turn: a rebind fills
    // the one whose upload (two rebinds ago) has completed -- its event says so -- instead of
    // synchronising the stream, so a caller that binds a fresh input tensor every call never
    // waits for the previous launch.
    mk_op_desc* h_ops[2] = {nullptr, nullptr};
    uint8_t* h_tmaps[2] = {nullptr, nullptr};
    cudaEvent_t staged[2] = {nullptr, nullptr};
    int stage_turn = 0;
    std::vector<int32_t> h_insts;    // host copy of the instruction words (argument checks at bind time)
    struct Packed {                  // tile-image copy of one weight matrix (see pack_weight_tiles)
        uint64_t src; int N, K, ld;
        uint8_t* buf; size_t bytes; bool used, fresh;
        bool fp16;                   // weights converted to fp16 (the ops reading it have fp16 activations)
    };
    std::vector<Packed> packed;
    struct Retired { uint8_t* buf; cudaEvent_t done; };   // packed copies no longer bound: freed once `done` has passed
    std::vector<Retired> retired;
    cudaStream_t last_stream = nullptr;                   // stream of the latest launch
    int64_t* d_trace = nullptr;
    int32_t* d_status = nullptr;
    int32_t* h_status = nullptr;     // pinned
    int epoch = 0;
    int max_target = 1;
    unsigned long long timeout_ns = 2000000000ull;
    int tcgen05_ops = 0;             // tile GEMMs bound to the tcgen05 body by the last set_ops
    int tcgen05_attn_ops = 0;        // ... prefill attention ops
    int pf_stages = 0;               // L2 prefetch distance of the producer warp, in ring stages (0 = off)
};

static const size_t kMapBytes = 512;       // tensor-map space per op
static thread_local char g_cuda_err[256] = "";

static int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_cuda_err, sizeof g_cuda_err, "%s: %s", what, cudaGetErrorString(e));
    return MK_E_CUDA;
}
#define MK_CUDA(call)                                        \
    do {                                                     \
        cudaError_t e_ = (call);                             \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call);  \
    } while (0)

// Makes `device` current for the lifetime of the object and puts the caller's device back after.
// Every entry point that allocates, copies or launches runs under one: a program belongs to one GPU,
// but the calling thread's current device is the caller's business (torch keeps its own notion of it).
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; (void)cudaGetLastError(); }
        if (prev != device) {
            cudaError_t e = cudaSetDevice(device);
            if (e != cudaSuccess) { cuda_fail(e, "cudaSetDevice"); ok = false; prev = -1; }
        } else {
            prev = -1;                                  // nothing to restore
        }
    }
    ~DeviceGuard() {
        if (prev >= 0) (void)cudaSetDevice(prev);
    }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};
#define MK_ON_DEVICE(dev)            \
    DeviceGuard guard_(dev);         \
    if (!guard_.ok) return MK_E_CUDA

// Tensor map over a row-major bf16 matrix {cols, rows} with row pitch `ld` elements: boxes of 64
// columns x `box_rows` rows, stored with the 128-byte swizzle (the operand tile layout of the tcgen05 tile
// GEMM), rows outside the matrix read as zero.  The driver entry point is looked up once; false
// when it is missing or refuses the arguments (the kernel then runs its mma.sync body).
static bool encode_tile_map(void* out, uint64_t base, long long rows, long long cols, long long ld, int box_rows, bool streamed,
                            bool fp16 = false) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn fn = nullptr;
    static bool looked = false;
    if (!looked) {
        looked = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_fn>(ptr);
        (void)cudaGetLastError();
    }
    if (!fn || (base & 15) || (ld % 8) || rows <= 0 || cols < 64 || ld < cols) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    alignas(64) CUtensorMap m;
    if (fn(&m, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, reinterpret_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           streamed ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(out, &m, sizeof(m));
    return true;
}

// Can the tcgen05 body run this tile GEMM?  K range of an instruction in whole 64-element k-tiles,
// and every operand the epilogue touches with 16-byte vectors aligned for them.
static bool tile_gemm_on_tcgen05(const mk_op_desc& d) {
    const int N = d.i[1], K = d.i[2], splits = d.i[4], odt = d.i[5], rdt = d.i[7], swi = d.i[8];
    if (splits <= 0 || K % splits || (K / splits) % 64) return false;
    const int n_out = swi ? N / 2 : N;
    if (n_out % 8 || (swi && N % 128)) return false;
    auto vec_ok = [](uint64_t ptr, int ld, int dt) { return !(ptr & 15) && ld % (dt == 1 ? 4 : 8) == 0; };
    if (!vec_ok(d.ptr[2], d.ld[2], odt)) return false;
    if (d.ptr[3] && (d.ptr[3] & 15)) return false;
    if (d.ptr[4] && !vec_ok(d.ptr[4], d.ld[4], rdt)) return false;
    return true;
}

// Bind-time check of the instruction table against the op descriptors: every argument an op body
// turns into an address (tile, row-group, head, split indices; output-column ranges) must lie inside
// the extents the descriptor states.  The kernel trusts its tables; this is where a table built for
// another graph, or a descriptor with a shrunken extent, is caught -- as an error code here instead of
// an out-of-bounds access on the device.  On failure the message names the instruction.
static int verify_tables(const mk_program* p, const mk_op_desc* ops) {
    const int W = MK_INST_WORDS;
    auto ceil_div = [](long long a, long long b) { return (a + b - 1) / b; };
    for (int k = 0; k < p->n_insts; ++k) {
        const int32_t* w = p->h_insts.data() + (size_t)k * W;
        const int opi = w[0] - 1;
        const char* why = nullptr;
        if (opi < 0 || opi >= p->n_ops) {
            why = "op index out of range";
        } else {
            const mk_op_desc& d = ops[opi];
            const long long a0 = w[1], a1 = w[2], a2 = w[3];
            switch (d.kind) {
                case MK_OP_GEMV:
                    if (!(0 <= a0 && a0 < a1 && a1 <= d.i[1])) why = "streaming linear: output range outside [0, N)";
                    break;
                case MK_OP_GEMM:
                    if (d.i[4] <= 0) why = "tile GEMM: split count";
                    else if (a0 < 0 || a0 * 128 >= d.i[0]) why = "tile GEMM: m tile outside M";
                    else if (d.i[10] != 0 && d.i[10] != 128 && !(d.i[10] == 256 && d.i[1] % 256 == 0)) why = "tile GEMM: weight rows per tile";
                    else if (a1 < 0 || a1 * (long long)(d.i[10] == 256 ? 256 : 128) >= d.i[1]) why = "tile GEMM: n tile outside N";
                    else if (a2 < 0 || a2 >= d.i[4]) why = "tile GEMM: K split index";
                    break;
                case MK_OP_FINALIZE:
                    if (d.i[5] <= 0 || a0 < 0 || a0 >= ceil_div(d.i[0], d.i[5]) || a1 < 0 || a1 * 512 >= d.i[1]) why = "finalize: tile outside the output";
                    break;
                case MK_OP_ELTWISE:
                    if (a0 < 0 || a0 * 32 >= d.i[0] || a1 < 0 || a1 * 512 >= d.i[1]) why = "pointwise: tile outside the output";
                    break;
                case MK_OP_NORM:
                    if (d.i[3] <= 0 || a0 < 0 || a0 * d.i[3] >= d.i[0]) why = "norm: row group outside the rows";
                    break;
                case MK_OP_ATTENTION:
                    if (a0 < 0 || a0 >= d.i[0] || a1 < 0 || a1 >= d.i[3] || a2 < 0 || a2 * 128 >= d.i[1]) why = "attention: (batch, head, query tile)";
                    break;
                case MK_OP_ROPE_APPEND:
                    if (a0 < 0 || a0 * 8 >= d.i[0]) why = "rope_append: row group outside the batch";
                    break;
                case MK_OP_DECODE_ATTN: {
                    const int hp = d.i[10] > 0 ? d.i[10] : 1;
                    if (a0 < 0 || a0 >= d.i[0] || a1 < 0 || a1 + hp > d.i[2] || a2 < 0 || a2 >= (d.i[5] > 0 ? d.i[5] : 1))
                        why = "decode attention: (sequence, kv head, split)";
                    break;
                }
                case MK_OP_INCREMENT: break;
                case MK_OP_GATHER:
                    if (a0 < 0 || a0 * 8 >= d.i[0] || a1 < 0 || a1 * 512 >= d.i[1]) why = "gather: tile outside the output";
                    break;
                case MK_OP_ARGMAX:
                    if (a0 < 0 || a0 >= d.i[0] || a1 < 0 || a1 >= d.i[2] || d.i[2] > 256 || d.i[3] % 8 || (long long)d.i[2] * d.i[3] < d.i[1])
                        why = "argmax: (row, chunk)";
                    break;
                default: why = "unknown op kind";
            }
        }
        if (why) {
            snprintf(g_cuda_err, sizeof g_cuda_err, "instruction %d (op %d): %s", k, opi, why);
            return MK_E_ARG;
        }
    }
    return MK_OK;
}

static void free_retired(mk_program* p, bool wait) {
    for (size_t e = 0; e < p->retired.size();) {
        auto& r = p->retired[e];
        if (wait) (void)cudaEventSynchronize(r.done);
        else if (cudaEventQuery(r.done) != cudaSuccess) { (void)cudaGetLastError(); ++e; continue; }
        cudaFree(r.buf);
        cudaEventDestroy(r.done);
        p->retired.erase(p->retired.begin() + e);
    }
}

extern "C" {

const char* mk_strerror(int code) {
    switch (code) {
        case MK_OK: return "ok";
        case MK_E_CUDA: return "CUDA runtime error";
        case MK_E_ARG: return "invalid argument";
        case MK_E_ARCH: return "device is not compute capability 10.x (sm_100a kernel)";
        case MK_E_DEVICE: return "megakernel reported a device-side error (see status words)";
        case MK_E_NOMEM: return "out of memory";
        case MK_E_TOO_LARGE: return "graph needs more dependency counters than MK_NOALLOC_MAX_COUNTERS (static scratch of mk_launch_noalloc)";
        default: return "unknown error";
    }
}

const char* mk_last_cuda_error(void) { return g_cuda_err; }

int mk_query(int device, mk_caps* caps) {
    if (!caps) return MK_E_ARG;
    cudaDeviceProp prop;
    MK_CUDA(cudaGetDeviceProperties(&prop, device));
    memset(caps, 0, sizeof *caps);
    caps->sm_count = prop.multiProcessorCount;
    caps->cc_major = prop.major;
    caps->cc_minor = prop.minor;
    caps->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    caps->kernel_smem = mk::kSmemBytes;
    caps->kernel_threads = mk::kThreads;
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, mk::megakernel<false>) == cudaSuccess) caps->kernel_regs = fa.numRegs;
    else (void)cudaGetLastError();
    if (prop.major != 10) return MK_E_ARCH;
    return MK_OK;
}

// The schedule is deadlock-free only if every CTA of the grid is resident at once (a CTA waits on
// counters that CTAs with lower instruction numbers publish): one CTA per SM with this kernel's
// shared memory, so a grid larger than the device's SM count is an argument error, not a timeout.
static int check_grid(int device, int grid) {
    mk_caps caps;
    int rc = mk_query(device, &caps);
    if (rc != MK_OK) return rc;
    if (caps.max_smem_optin < mk::kSmemBytes) return MK_E_ARCH;
    if (grid <= 0 || grid > caps.sm_count) {
        snprintf(g_cuda_err, sizeof g_cuda_err, "grid %d: must be 1..%d (the device's SM count; all CTAs must be co-resident)", grid, caps.sm_count);
        return MK_E_ARG;
    }
    return MK_OK;
}

int mk_program_create(int device, const int32_t* insts, int n_insts, const int32_t* waits, int n_waits,
                      const int32_t* arrives, int n_arrives, int n_counters, int n_ops, int grid, int trace_cap,
                      mk_program** out) {
    g_cuda_err[0] = 0;
    if (!out || !insts || n_insts <= 0 || n_ops <= 0 || grid <= 0 || n_waits < 0 || n_arrives < 0) return MK_E_ARG;
    if ((n_waits && !waits) || (n_arrives && !arrives)) return MK_E_ARG;
    int rc = check_grid(device, grid);
    if (rc != MK_OK) return rc;
    MK_ON_DEVICE(device);
    mk_program* p = new (std::nothrow) mk_program();
    if (!p) return MK_E_NOMEM;
    p->device = device; p->grid = grid; p->n_insts = n_insts; p->n_waits = n_waits; p->n_arrives = n_arrives;
    p->n_counters = n_counters > 0 ? n_counters : 1; p->n_ops = n_ops; p->trace_cap = trace_cap;
    for (int k = 0; k < n_waits; ++k) {
        if (waits[2 * k] < 0 || waits[2 * k] >= p->n_counters) { delete p; return MK_E_ARG; }
        if (waits[2 * k + 1] > p->max_target) p->max_target = waits[2 * k + 1];
    }
    for (int k = 0; k < n_arrives; ++k)
        if (arrives[k] < 0 || arrives[k] >= p->n_counters) { delete p; return MK_E_ARG; }
    // every instruction's wait and arrival slices must lie inside their tables
    for (int k = 0; k < n_insts; ++k) {
        const int32_t* w = insts + (size_t)k * MK_INST_WORDS;
        if (w[8] < 0 || w[9] < 0 || (long long)w[8] + w[9] > n_waits || w[10] < 0 || w[11] < 0 || (long long)w[10] + w[11] > n_arrives) {
            delete p;
            snprintf(g_cuda_err, sizeof g_cuda_err, "instruction %d: wait / arrival slice outside its table", k);
            return MK_E_ARG;
        }
    }
    p->h_insts.assign(insts, insts + (size_t)n_insts * MK_INST_WORDS);
#define MK_TRY(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { cuda_fail(e_, #call); mk_program_destroy(p); return MK_E_CUDA; } } while (0)
    MK_TRY(cudaMalloc(&p->d_insts, (size_t)n_insts * MK_INST_WORDS * 4));
    MK_TRY(cudaMemcpy(p->d_insts, insts, (size_t)n_insts * MK_INST_WORDS * 4, cudaMemcpyHostToDevice));
    MK_TRY(cudaMalloc(&p->d_waits, (size_t)(n_waits > 0 ? n_waits : 1) * 8));
    if (n_waits) MK_TRY(cudaMemcpy(p->d_waits, waits, (size_t)n_waits * 8, cudaMemcpyHostToDevice));
    MK_TRY(cudaMalloc(&p->d_arrives, (size_t)(n_arrives > 0 ? n_arrives : 1) * 4));
    if (n_arrives) MK_TRY(cudaMemcpy(p->d_arrives, arrives, (size_t)n_arrives * 4, cudaMemcpyHostToDevice));
    MK_TRY(cudaMalloc(&p->d_counters, (size_t)p->n_counters * 4));
    MK_TRY(cudaMemset(p->d_counters, 0, (size_t)p->n_counters * 4));
    MK_TRY(cudaMalloc(&p->d_ops, (size_t)n_ops * sizeof(mk_op_desc)));
    MK_TRY(cudaMalloc(&p->d_tmaps, (size_t)n_ops * kMapBytes));
    for (int b = 0; b < 2; ++b) {
        MK_TRY(cudaMallocHost(&p->h_ops[b], (size_t)n_ops * sizeof(mk_op_desc)));
        MK_TRY(cudaMallocHost(&p->h_tmaps[b], (size_t)n_ops * kMapBytes));
        MK_TRY(cudaEventCreateWithFlags(&p->staged[b], cudaEventDisableTiming));
    }
    MK_TRY(cudaMalloc(&p->d_status, MK_ST_WORDS * 4));
    MK_TRY(cudaMemset(p->d_status, 0, MK_ST_WORDS * 4));
    MK_TRY(cudaMallocHost(&p->h_status, MK_ST_WORDS * 4));
    if (trace_cap > 0) {
        size_t words = (size_t)grid * mk::kTraceRoles * trace_cap * 4;
        MK_TRY(cudaMalloc(&p->d_trace, words * 8));
        MK_TRY(cudaMemset(p->d_trace, 0, words * 8));
    }
    MK_TRY(cudaFuncSetAttribute(mk::megakernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, mk::kSmemBytes));
    MK_TRY(cudaFuncSetAttribute(mk::megakernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, mk::kSmemBytes));
#undef MK_TRY
    if (const char* e = getenv("MEGACUTE_B200_PF_STAGES")) p->pf_stages = atoi(e);
    *out = p;
    return MK_OK;
}

int mk_program_set_ops(mk_program* p, const mk_op_desc* ops, int n_ops, void* stream) {
    g_cuda_err[0] = 0;
    if (!p || !ops || n_ops != p->n_ops) return MK_E_ARG;
    int rc = verify_tables(p, ops);
    if (rc != MK_OK) return rc;
    MK_ON_DEVICE(p->device);
    cudaStream_t st = (cudaStream_t)stream;
    // this turn's staging copy was last uploaded two rebinds ago; wait for that upload only
    const int turn = p->stage_turn;
    p->stage_turn ^= 1;
    MK_CUDA(cudaEventSynchronize(p->staged[turn]));
    mk_op_desc* h_ops = p->h_ops[turn];
    uint8_t* h_tmaps = p->h_tmaps[turn];
    memcpy(h_ops, ops, (size_t)n_ops * sizeof(mk_op_desc));
    // Tile GEMMs get tensor maps over their activations and weights (ptr 11): with them the kernel
    // runs the tcgen05 body and streams the weight tiles through the producer warp's ring.
    bool any_map = false;
    int n_tc = 0;
    const bool tc_off = getenv("MEGACUTE_B200_NO_TCGEN05") != nullptr;
    const bool pack_off = getenv("MEGACUTE_B200_NO_WEIGHT_PACK") != nullptr;
    for (auto& e : p->packed) e.used = false;
    int n_attn = 0;
    for (int k = 0; k < n_ops; ++k) {
        mk_op_desc& d = h_ops[k];
        if (d.kind == MK_OP_ATTENTION) {
            // head_dim 64: tensor maps over q, k, v select the tcgen05 body (op_attention_tc.cuh)
            d.ptr[11] = 0;
            uint8_t* maps = h_tmaps + (size_t)k * kMapBytes;
            const long long B = d.i[0], Sq = d.i[1], Sk = d.i[2], H = d.i[3], KVH = d.i[4];
            // On unless MEGACUTE_B200_ATTN_TCGEN05=0: measured on 4 x 4096 causal tokens (32 heads, 8 kv heads, 16 layers)
            // the tcgen05 body (softmax on all eight compute warps, tiles and MMAs fed by the producer warp) takes
            // 14.5 ms of attention against the mma.sync body's 31 ms.
            const char* attn_tc = getenv("MEGACUTE_B200_ATTN_TCGEN05");
            if (attn_tc && attn_tc[0] == '0') continue;
            if (tc_off || d.i[5] != 64 || (d.ptr[3] & 15) || d.ld[3] % 8) continue;
            const bool h16 = d.i[8] == mk::DT_F16;
            if (encode_tile_map(maps, d.ptr[0], B * Sq, H * 64, d.ld[0], 128, false, h16) &&
                encode_tile_map(maps + 128, d.ptr[1], B * Sk, KVH * 64, d.ld[1], 128, false, h16) &&
                encode_tile_map(maps + 256, d.ptr[2], B * Sk, KVH * 64, d.ld[2], 128, false, h16)) {
                d.ptr[11] = reinterpret_cast<uint64_t>(p->d_tmaps + (size_t)k * kMapBytes);
                any_map = true;
                ++n_attn;
            }
            continue;
        }
        if (d.kind != MK_OP_GEMM) continue;
        d.ptr[11] = 0;
        if (tc_off || !tile_gemm_on_tcgen05(d)) continue;
        uint8_t* maps = h_tmaps + (size_t)k * kMapBytes;
        d.ptr[10] = 0;
        if (d.i[9] != mk::DT_BF16 && d.i[9] != mk::DT_F16) continue;
        const bool xh = d.i[9] == mk::DT_F16;
        // fp16 activations need fp16 weights (the tensor core takes one 16-bit type per instruction;
        // mixing fp16 activations with bf16 weights raised an illegal-instruction fault): only the packed
        // copy can provide them.  Without one, the op runs the mma.sync body, which converts in registers.
        if (xh && (pack_off || (d.ptr[1] & 15) || d.ld[1] % 8 != 0)) continue;
        if (!encode_tile_map(maps, d.ptr[0], d.i[0], d.i[2], d.ld[0], d.i[0] <= 64 ? 64 : 128, false, d.i[9] == mk::DT_F16)) continue;
        // weights: the packed copy, made when a matrix (address, shape, pitch) is bound for the first
        // time and kept while it stays bound -- rebinding other operands (a new input tensor every
        // call) must not copy gigabytes of weights again; weights changed in place need
        // mk_program_refresh_weights -- else a tensor map over the matrix
        if (!pack_off && !(d.ptr[1] & 15) && d.ld[1] % 8 == 0) {
            mk_program::Packed* hit = nullptr;
            for (auto& e : p->packed)
                if (e.src == d.ptr[1] && e.N == d.i[1] && e.K == d.i[2] && e.ld == d.ld[1] && e.fp16 == xh) hit = &e;
            if (!hit) {
                free_retired(p, false);
                mk_program::Packed e{d.ptr[1], d.i[1], d.i[2], d.ld[1], nullptr, 0, false, true, xh};
                e.bytes = (size_t)((d.i[1] + 127) / 128) * 128 * (size_t)d.i[2] * 2;
                cudaError_t err = cudaMalloc(&e.buf, e.bytes);
                if (err != cudaSuccess && !p->retired.empty()) {       // out of memory with copies waiting to be freed
                    (void)cudaGetLastError();
                    free_retired(p, true);
                    err = cudaMalloc(&e.buf, e.bytes);
                }
                if (err == cudaSuccess) {
                    p->packed.push_back(e);
                    hit = &p->packed.back();
                } else {
                    (void)cudaGetLastError();
                }
            }
            if (hit) {
                if (hit->fresh) {       // a copy made by this call: fill it (once, however many ops share the matrix)
                    const long long chunks = (long long)(hit->bytes / 16);
                    const int blocks = (int)((chunks + 255) / 256 < 4096 ? (chunks + 255) / 256 : 4096);
                    mk::pack_weight_tiles<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(hit->src), hit->ld, hit->N,
                                                                  hit->K, reinterpret_cast<uint4*>(hit->buf), chunks, hit->fp16 ? 1 : 0);
                    MK_CUDA(cudaGetLastError());
                    hit->fresh = false;
                }
                hit->used = true;
                d.ptr[10] = reinterpret_cast<uint64_t>(hit->buf);
            }
        }
        if (xh && !d.ptr[10]) continue;                 // (the copy could not be allocated)
        if (d.ptr[10] || encode_tile_map(maps + 128, d.ptr[1], d.i[1], d.i[2], d.ld[1], 128, true)) {
            d.ptr[11] = reinterpret_cast<uint64_t>(p->d_tmaps + (size_t)k * kMapBytes);
            any_map = true;
            ++n_tc;
        }
    }
    p->tcgen05_ops = n_tc;
    p->tcgen05_attn_ops = n_attn;
    // Packed copies of matrices that are no longer bound are retired, not freed: launches enqueued
    // before this rebind may still read them.  An event on `stream` (and on the stream of the latest
    // launch, if another) marks the point after which they are free; they are released by a later
    // rebind that finds the event passed, by mk_program_refresh_weights or by mk_program_destroy.
    for (size_t e = 0; e < p->packed.size();) {
        if (p->packed[e].used) { ++e; continue; }
        mk_program::Retired r{p->packed[e].buf, nullptr};
        MK_CUDA(cudaEventCreateWithFlags(&r.done, cudaEventDisableTiming));
        if (p->last_stream != st) {
            // order this stream behind the latest launch, so that one event covers both
            cudaEvent_t ev;
            MK_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            MK_CUDA(cudaEventRecord(ev, p->last_stream));
            MK_CUDA(cudaStreamWaitEvent(st, ev, 0));
            MK_CUDA(cudaEventDestroy(ev));
        }
        MK_CUDA(cudaEventRecord(r.done, st));
        p->retired.push_back(r);
        p->packed.erase(p->packed.begin() + e);
    }
    free_retired(p, false);
    if (any_map) MK_CUDA(cudaMemcpyAsync(p->d_tmaps, h_tmaps, (size_t)n_ops * kMapBytes, cudaMemcpyHostToDevice, st));
    MK_CUDA(cudaMemcpyAsync(p->d_ops, h_ops, (size_t)n_ops * sizeof(mk_op_desc), cudaMemcpyHostToDevice, st));
    MK_CUDA(cudaEventRecord(p->staged[turn], st));
    return MK_OK;
}

int mk_program_set_timeout(mk_program* p, uint64_t ns) {
    if (!p || ns == 0) return MK_E_ARG;
    p->timeout_ns = ns;
    return MK_OK;
}

int mk_launch(mk_program* p, void* stream) {
    if (!p) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int max_epoch = 0x7fffffff / (p->max_target > 0 ? p->max_target : 1) - 1;
    if (p->epoch >= max_epoch) {
        MK_CUDA(cudaMemsetAsync(p->d_counters, 0, (size_t)p->n_counters * 4, st));
        p->epoch = 0;
    }
    p->epoch += 1;
    p->last_stream = st;
    mk::Params prm;
    prm.insts = reinterpret_cast<const int4*>(p->d_insts);
    prm.n_insts = p->n_insts;
    prm.waits = reinterpret_cast<const int2*>(p->d_waits);
    prm.arrives = p->d_arrives;
    prm.counters = p->d_counters;
    prm.ops = p->d_ops;
    prm.n_ops = p->n_ops;
    prm.trace = reinterpret_cast<long long*>(p->d_trace);
    prm.trace_cap = p->trace_cap;
    prm.status = p->d_status;
    prm.epoch = p->epoch;
    prm.timeout_ns = p->timeout_ns;
    prm.pf_stages = p->pf_stages;
    if (p->trace_cap > 0) mk::megakernel<true><<<p->grid, mk::kThreads, mk::kSmemBytes, st>>>(prm);
    else mk::megakernel<false><<<p->grid, mk::kThreads, mk::kSmemBytes, st>>>(prm);
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

int mk_program_status(mk_program* p, void* stream, int32_t status[MK_ST_WORDS]) {
    if (!p) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    cudaStream_t st = (cudaStream_t)stream;
    MK_CUDA(cudaMemcpyAsync(p->h_status, p->d_status, MK_ST_WORDS * 4, cudaMemcpyDeviceToHost, st));
    MK_CUDA(cudaStreamSynchronize(st));
    if (status) memcpy(status, p->h_status, MK_ST_WORDS * 4);
    if (p->h_status[MK_ST_CODE] != 0) {
        MK_CUDA(cudaMemsetAsync(p->d_status, 0, MK_ST_WORDS * 4, st));
        return MK_E_DEVICE;
    }
    return MK_OK;
}

int mk_program_reset(mk_program* p, void* stream) {
    if (!p) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    cudaStream_t st = (cudaStream_t)stream;
    MK_CUDA(cudaMemsetAsync(p->d_counters, 0, (size_t)p->n_counters * 4, st));
    MK_CUDA(cudaMemsetAsync(p->d_status, 0, MK_ST_WORDS * 4, st));
    p->epoch = 0;
    return MK_OK;
}

int mk_program_epoch(mk_program* p) { return p ? p->epoch : MK_E_ARG; }

int mk_program_tcgen05_ops(mk_program* p) { return p ? p->tcgen05_ops : MK_E_ARG; }

int mk_program_tcgen05_attention_ops(mk_program* p) { return p ? p->tcgen05_attn_ops : MK_E_ARG; }

int mk_program_refresh_weights(mk_program* p, void* stream) {
    if (!p) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    MK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));       // no launch may still be reading the copies
    if (p->last_stream != (cudaStream_t)stream) MK_CUDA(cudaStreamSynchronize(p->last_stream));
    for (auto& e : p->packed) cudaFree(e.buf);
    p->packed.clear();
    free_retired(p, true);
    return MK_OK;
}

long long mk_program_packed_bytes(mk_program* p) {
    if (!p) return MK_E_ARG;
    long long total = 0;
    for (auto& e : p->packed) total += (long long)e.bytes;
    return total;
}

int mk_program_read_counters(mk_program* p, int32_t* out, int n) {
    if (!p || !out || n < 0 || n > p->n_counters) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    MK_CUDA(cudaMemcpy(out, p->d_counters, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return MK_OK;
}

int mk_program_read_trace(mk_program* p, int64_t* out, size_t n_words) {
    if (!p || !out || !p->d_trace) return MK_E_ARG;
    if (n_words > (size_t)p->grid * mk::kTraceRoles * p->trace_cap * 4) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    MK_CUDA(cudaMemcpy(out, p->d_trace, n_words * 8, cudaMemcpyDeviceToHost));
    return MK_OK;
}

int mk_program_clear_trace(mk_program* p, void* stream) {
    if (!p) return MK_E_ARG;
    if (!p->d_trace) return MK_OK;
    MK_ON_DEVICE(p->device);
    MK_CUDA(cudaMemsetAsync(p->d_trace, 0, (size_t)p->grid * mk::kTraceRoles * p->trace_cap * 4 * 8, (cudaStream_t)stream));
    return MK_OK;
}

int mk_program_poke_wait(mk_program* p, int wait_index, int counter, int target) {
    if (!p || wait_index < 0 || wait_index >= p->n_waits || counter < 0 || counter >= p->n_counters) return MK_E_ARG;
    MK_ON_DEVICE(p->device);
    int32_t pair[2] = {counter, target};
    MK_CUDA(cudaMemcpy(p->d_waits + 2 * wait_index, pair, 8, cudaMemcpyHostToDevice));
    return MK_OK;
}

void mk_program_destroy(mk_program* p) {
    if (!p) return;
    DeviceGuard guard(p->device);
    free_retired(p, true);
    cudaFree(p->d_insts); cudaFree(p->d_waits); cudaFree(p->d_arrives); cudaFree(p->d_counters);
    cudaFree(p->d_ops); cudaFree(p->d_trace); cudaFree(p->d_status); cudaFree(p->d_tmaps);
    for (auto& e : p->packed) cudaFree(e.buf);
    for (int b = 0; b < 2; ++b) {
        if (p->h_ops[b]) cudaFreeHost(p->h_ops[b]);
        if (p->h_tmaps[b]) cudaFreeHost(p->h_tmaps[b]);
        if (p->staged[b]) cudaEventDestroy(p->staged[b]);
    }
    if (p->h_status) cudaFreeHost(p->h_status);
    delete p;
}

}  // extern "C"

// -------------------------------------------------------------------------------------------------
// mk_launch_noalloc: the same kernel for hosts that must not allocate device memory.
//
// The megakernel needs scratch beyond the caller's tensors: its dependency counters and its status
// words.  mk_program_create() gets them from cudaMalloc.  Some hosts cannot do that -- an inference
// server that has already handed all of HBM to its own pool, or a latency-critical loop that cannot
// afford the device-wide synchronisation a cudaMalloc / cudaFree implies.  For them the scratch
// lives in this file-scope device array: MK_NOALLOC_MAX_COUNTERS counters + MK_ST_WORDS status
// words, about 64 KB that every GPU which loads the library holds until the process exits.
//
// `g_noalloc_scratch` below is, in host code, only a handle for the symbol -- not a device
// address.  The address is looked up once per device with cudaGetSymbolAddress (that device
// current) and cached; kernels are only ever given that looked-up pointer.
// -------------------------------------------------------------------------------------------------
static __device__ __align__(256) int32_t g_noalloc_scratch[MK_NOALLOC_MAX_COUNTERS + MK_ST_WORDS];

static const int kMaxDevices = 64;
static int32_t* g_noalloc_ptr[kMaxDevices];          // per device: looked-up address of the array, or null

extern "C" int mk_launch_noalloc(int device, const int32_t* d_insts, int n_insts, const int32_t* d_waits, int n_waits,
                                 const int32_t* d_arrives, int n_arrives, const mk_op_desc* d_ops, int n_ops,
                                 int n_counters, int grid, void* stream, int32_t status[MK_ST_WORDS]) {
    g_cuda_err[0] = 0;
    if (device < 0 || device >= kMaxDevices || !d_insts || n_insts <= 0 || !d_ops || n_ops <= 0 || grid <= 0 ||
        n_waits < 0 || n_arrives < 0 || n_counters < 0 || (n_waits && !d_waits) || (n_arrives && !d_arrives))
        return MK_E_ARG;
    if (n_counters > MK_NOALLOC_MAX_COUNTERS) return MK_E_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    MK_ON_DEVICE(device);                               // the caller's current device is put back on return
    if (!g_noalloc_ptr[device]) {
        // one-time set-up for this device (do this first call outside any stream capture)
        int rc = check_grid(device, grid);
        if (rc != MK_OK) return rc;
        int32_t* ptr = nullptr;
        MK_CUDA(cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch));
        MK_CUDA(cudaFuncSetAttribute(mk::megakernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, mk::kSmemBytes));
        g_noalloc_ptr[device] = ptr;
    } else {
        int sms = 0;
        MK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        if (grid > sms) return MK_E_ARG;               // all CTAs must be co-resident (see check_grid)
    }
    int32_t* scratch = g_noalloc_ptr[device];
    int32_t* d_status = scratch + MK_NOALLOC_MAX_COUNTERS;
    // the array keeps the previous call's contents: counters and status must start at zero
    if (n_counters > 0) MK_CUDA(cudaMemsetAsync(scratch, 0, (size_t)n_counters * 4, st));
    MK_CUDA(cudaMemsetAsync(d_status, 0, MK_ST_WORDS * 4, st));
    mk::Params prm;
    prm.insts = reinterpret_cast<const int4*>(d_insts);
    prm.n_insts = n_insts;
    prm.waits = reinterpret_cast<const int2*>(d_waits);
    prm.arrives = d_arrives;
    prm.counters = scratch;
    prm.ops = d_ops;
    prm.n_ops = n_ops;
    prm.trace = nullptr;
    prm.trace_cap = 0;
    prm.status = d_status;
    prm.epoch = 1;
    prm.timeout_ns = 2000000000ull;
    prm.pf_stages = 0;
    mk::megakernel<false><<<grid, mk::kThreads, mk::kSmemBytes, st>>>(prm);
    MK_CUDA(cudaGetLastError());
    if (status) {
        MK_CUDA(cudaMemcpyAsync(status, d_status, MK_ST_WORDS * 4, cudaMemcpyDeviceToHost, st));
        MK_CUDA(cudaStreamSynchronize(st));
        if (status[MK_ST_CODE] != 0) return MK_E_DEVICE;
    }
    return MK_OK;
}

// Status of the latest mk_launch_noalloc on `device` for callers that passed status == NULL: waits for
// `stream`, copies the static status words out.  Allocates nothing.
extern "C" int mk_noalloc_status(int device, void* stream, int32_t status[MK_ST_WORDS]) {
    if (device < 0 || device >= kMaxDevices || !status) return MK_E_ARG;
    if (!g_noalloc_ptr[device]) return MK_E_ARG;        // no mk_launch_noalloc on this device yet
    MK_ON_DEVICE(device);
    cudaStream_t st = (cudaStream_t)stream;
    MK_CUDA(cudaMemcpyAsync(status, g_noalloc_ptr[device] + MK_NOALLOC_MAX_COUNTERS, MK_ST_WORDS * 4, cudaMemcpyDeviceToHost, st));
    MK_CUDA(cudaStreamSynchronize(st));
    return status[MK_ST_CODE] != 0 ? MK_E_DEVICE : MK_OK;
}
