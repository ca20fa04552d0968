// MK_OP_GEMV: linear with <= 8 activation rows, out = act(norm(x) @ w^T + bias) + residual.
//
// Pure weight streaming.  The producer warp copies weight rows into a ring of 32 KB stages with
// 1-D bulk copies (one per row, completion counted on the stage's mbarrier) and runs ahead of the
// compute warps across instruction boundaries, because weights never depend on anything in the
// launch.  A stage holds 8 row slots x 2048 K-elements; compute thread t owns K-elements
// [8t, 8t+8) of every slot, so its slice of the activation is loaded once per stage and reused
// for the 8 rows.  Partial dot products are reduced across the CTA once per group of 8 rows.
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
// A stage is 16 weight rows x one 1024-element K segment.  Each compute warp multiplies a 128-wide
// K slice of the 16 rows with warp-level MMAs (weights are the A operand straight from the stage via
// ldmatrix; the <= 8 activation rows are the B operand, split into bf16 high and low parts so the
// product keeps ~16 mantissa bits of the activation), accumulates over the segments of the row
// group, and the 8 warps combine through shared memory: the last to arrive writes the 16 outputs.
// About 12 instructions per 512 bytes of weights, so the warps mostly wait for HBM.
constexpr int GEMV_F_UNITS = 4;

struct RingPos {
    int stage = 0;
    uint32_t phase = 0;
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

// Producer warp: issue every stage of one GEMV instruction.  Returns false if a wait gave up.
__device__ __forceinline__ bool gemv_produce(const Params& p, Ctrl* c, uint8_t* ring, const mk_op_desc* op,
                                             int o0, int o1, int seq, RingPos& pos) {
    const int lane = threadIdx.x & 31;
    const int K = op->i[2];
    const bool swi = op->flags & GEMV_F_SWIGLU;
    const int per = swi ? 4 : 8;
    const int groups = (o1 - o0 + per - 1) / per;
    const int nkc = (K + kGemvKChunk - 1) / kGemvKChunk;
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]);
    const long long ldw = op->ld[1];
    if (op->flags & GEMV_F_UNITS) {
        // stage = 16 rows x K segment `seg`; segments of a row group are consecutive stages; swiglu
        // alternates a group of 16 gate rows with the group of the matching 16 up rows
        const int S = (K + kSegElems - 1) / kSegElems;
        const int n = o1 - o0;
        const int ngroups = (swi ? 2 : 1) * ((n + 15) / 16);
        const int r = lane & 15;
        for (int g = 0; g < ngroups; ++g) {
            const int o = o0 + (swi ? g >> 1 : g) * 16 + r;
            const int row = swi ? 128 * (o >> 6) + (o & 63) + ((g & 1) << 6) : o;
            const bool valid = lane < 16 && o < o1;
            for (int seg = 0; seg < S; ++seg) {
                const int k0 = seg * kSegElems;
                const int bytes = valid ? min(kSegElems, K - k0) * 2 : 0;
                const int total = __reduce_add_sync(0xffffffffu, bytes);
                bool ok = true;
                if (lane == 0) {
                    ok = wait_barrier(p, c, &c->empty[pos.stage], pos.phase ^ 1u, seq, WHERE_RING_EMPTY);
                    if (ok) mbar_arrive_expect_tx(&c->full[pos.stage], (uint32_t)total);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) return false;
                if (valid)
                    bulk_g2s(ring + pos.stage * kStageBytes + r * kSegStride, w + row * ldw + k0, (uint32_t)bytes,
                             &c->full[pos.stage]);
                pos.advance();
            }
        }
        return true;
    }
    for (int g = 0; g < groups; ++g) {
        int col;
        const int row = gemv_weight_row(swi, o0, g, lane & 7, &col);
        const bool valid = lane < 8 && col < o1;
        const int nvalid = swi ? 2 * min(4, o1 - o0 - g * 4) : min(8, o1 - o0 - g * 8);
        for (int kc = 0; kc < nkc; ++kc) {
            const int k0 = kc * kGemvKChunk;
            const int kl = min(kGemvKChunk, K - k0);
            bool ok = true;
            if (lane == 0) {
                ok = wait_barrier(p, c, &c->empty[pos.stage], pos.phase ^ 1u, seq, WHERE_RING_EMPTY);
                if (ok) mbar_arrive_expect_tx(&c->full[pos.stage], (uint32_t)(nvalid * kl * 2));
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) return false;
            if (valid)
                bulk_g2s(ring + pos.stage * kStageBytes + (lane & 7) * (kGemvKChunk * 2), w + row * ldw + k0,
                         (uint32_t)(kl * 2), &c->full[pos.stage]);
            pos.advance();
        }
    }
    return true;
}

}  // namespace mk
