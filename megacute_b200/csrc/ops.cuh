// Entry points of the op bodies.  Every op body lives in its own translation unit and the library
// is built as relocatable device code: measured on sm_100a, when the bodies share one translation
// unit with the kernel, ptxas' whole-program register allocation spills the inner loop of the
// streaming linear to local memory (with 227 KB of the SM given to shared memory almost no L1 is
// left, so each spill is an L2 round trip: 6x slower), however the calls are arranged.  Compiled
// separately, each body gets its own allocation under the 168-register cap of a 9-warp CTA.
//
// All take the op descriptor and the instruction's arguments by value and find the CTA's shared
// memory through the kernel's dynamic shared-memory window.
#pragma once
#include "mk_device.cuh"

namespace mk {

// ring position in / out is packed as stage | phase << 8
// (this op waits for its own dependencies and publishes its own arrivals; returns -1 when aborting)
__device__ int mk_op_gemv_units(const Params& p, const mk_op_desc* op, int o0, int o1, int seq, int packed_pos, int nwait,
                                int wait_off, int narrive, int arrive_off);
// body of the finisher warp (op_gemv_mma.cuh): runs until the CTA's instruction list ends
__device__ void mk_gemv_finisher(const Params& p);
__device__ int mk_op_gemv_general(const Params& p, const mk_op_desc* op, int o0, int o1, int seq, int packed_pos);
// Tile GEMM.  The kernel's loop has fetched instruction `idx` and chosen this body; the body runs it and every
// following instruction of the CTA that is its own (walk.cuh), waiting for the dependencies and publishing the
// arrivals of each itself (begin_op says why).  Returns the index of the last instruction executed, -1 when the CTA is
// aborting.  (The ring position is untouched: the weight tiles have slots of their own.)
__device__ int mk_run_gemm(const Params& p, int idx);
// (the same with 128 x 256 output tiles; only for ops the host library bound to the tcgen05 body)
__device__ int mk_run_gemm_wide(const Params& p, int idx);
__device__ void mk_op_attention(const mk_op_desc* op, int a0, int a1, int a2);
// (the tcgen05 body, for ops the host library attached tensor maps to; returns -1 when aborting)
__device__ int mk_op_attention_tc(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int seq);
// body of the feeder warp: walks the CTA's instruction list and, for every prefill attention bound to the tcgen05 body,
// requests its tiles and issues its MMAs (one thread); runs until the list ends or the CTA aborts
__device__ void mk_attention_feeder(const Params& p);
// (waits for its own dependencies and publishes its own arrivals; returns whether the CTA is aborting)
__device__ bool mk_op_decode_attn(const Params& p, const mk_op_desc* op, int a0, int a1, int a2, int nwait, int wait_off,
                                  int seq, int narrive, int arrive_off);
// (many-sequence form: all kv heads of a sequence per instruction, whole cache rows through bulk copies)
__device__ bool mk_op_decode_bulk(const Params& p, const mk_op_desc* op, int b, int s, int nwait, int wait_off, int seq,
                                  int narrive, int arrive_off);
// finalize / eltwise / norm / rope_append / increment / gather / argmax; returns false for an unknown kind
__device__ bool mk_op_pointwise(const mk_op_desc* op, int a0, int a1);

struct SmemMap {
    uint8_t* ring;
    uint8_t* work;
    Ctrl* ctrl;
};
__device__ __forceinline__ SmemMap smem_map() {
    extern __shared__ __align__(1024) uint8_t mk_smem[];
    SmemMap m;
    m.ring = mk_smem;
    m.work = mk_smem + kRingBytes;
    m.ctrl = reinterpret_cast<Ctrl*>(mk_smem + kRingBytes + kWorkBytes);
    return m;
}

}  // namespace mk
