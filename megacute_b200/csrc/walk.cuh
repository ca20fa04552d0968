// A tile-GEMM body keeps the CTA's walk through its instruction list for as long as the next instruction is its own.
//
// The body is a function of another translation unit than the kernel, called through the ABI: on entry it saves the
// callee-saved registers it is going to use to local memory and on return it loads them back (62 registers of 256
// threads, 63 KB each way, with almost no L1 to hold them: 1.5 us measured on entry).  Behind a dependency hop that
// time is hidden in the wait (begin_op / end_op); a prefill or DiT graph, though, gives an SM some two thousand tile
// GEMM instructions whose dependencies are already met, many of them in a row.  So the body does not return after
// one: it does for the next instruction what the kernel's loop would do (metadata staging, dependency wait, arrivals,
// trace records) and goes on, until the CTA's next instruction belongs to another body.
// Nothing of the walk lives in registers across an instruction: its index is parked in shared memory and everything
// else is read again from the staged metadata, so that the walk adds nothing to the body's register allocation (with
// the index and the ring position held in registers the body's frame grew by 80 bytes, and a graph with one tile GEMM
// instruction per SM and op paid for it: 57 -> 60 us for the MLP block).
#pragma once
#include "mk_device.cuh"

namespace mk {

// The kernel's loop has fetched instruction `idx` (its metadata is staged, the staging for the following ones is
// under way) and chosen this body for it.  mine(op): does the body run this op too?  body(op, a0, a1, a2, seq) runs
// one instruction between its dependency wait and its arrivals, < 0 when the CTA is aborting.
// Returns the index of the last instruction executed, or -1 when aborting.  All compute threads call this together;
// every decision in it is made on words that change only behind a barrier.
template <class Mine, class Body>
__device__ __forceinline__ int run_own_insts(const Params& p, Ctrl* c, int idx, Mine mine, Body body) {
    Meta* mt = &c->meta;
    for (;;) {
        if (threadIdx.x == 0) c->run_idx = idx;                 // (read back behind the barrier of publish())
        {
            const int slot = (idx - (int)blockIdx.x) / (int)gridDim.x, s3 = slot % 3, s2 = slot & 1;
            if (p.trace_cap > 0 && threadIdx.x == 0) c->t_fetch = (long long)globaltimer();
            const int4 w2 = mt->inst[s3][2];
            const Sync sy{w2.x, w2.x <= kMetaWaits ? -1 - s2 : w2.y, 0, 0};
            if (begin_op(p, c, sy, mt->inst[s3][3].x)) return -1;
            const int4 w0 = mt->inst[s3][0];
            if (body(&mt->desc[s2], w0.y, w0.z, w0.w, mt->inst[s3][3].x) < 0) return -1;
        }
        idx = *(volatile int*)&c->run_idx;                      // (the same value: not kept in a register across the body)
        const int slot = (idx - (int)blockIdx.x) / (int)gridDim.x, s3 = slot % 3, s2 = slot & 1;
        const int seq = mt->inst[s3][3].x;                       // (behind the barrier of publish() warp 1 may already be staging over this row)
        {
            const int4 w2 = mt->inst[s3][2];
            if (publish(p, c, w2.z, w2.z <= kMetaArrives ? -1 - s2 : w2.w)) return -1;
        }
        if (p.trace_cap > 0 && threadIdx.x == 0) {
            trace_rec_rt(p, 1, slot, seq, c->t_fetch, c->t_dep, (long long)globaltimer());
            trace_rec_rt(p, 2, slot, seq, c->t_phase[0], c->t_phase[1], c->t_phase[2]);
        }
        // the CTA's next instruction: staged during this one, visible behind the barrier of publish()
        const int next = idx + (int)gridDim.x;
        if (next >= p.n_insts) break;
        const int opi = mt->inst[(slot + 1) % 3][0].x - 1;
        if (opi < 0 || opi >= p.n_ops || !mine(&mt->desc[s2 ^ 1])) break;
        idx = next;
        if ((threadIdx.x >> 5) == 1) {           // what the kernel's loop does when it fetches an instruction
            const int lane = threadIdx.x & 31;
            stage_row(p, mt, idx + 2 * (int)gridDim.x, (slot + 3) % 3, lane);
            if (idx + (int)gridDim.x < p.n_insts) stage_op(p, mt, (slot + 2) % 3, s2, lane);
            cp_async_commit();
        }
    }
    return idx;
}

}  // namespace mk
