// Vectorised (128-bit) pointwise, norm and small decode ops.  All read and write global memory
// directly with 16-byte accesses: they are bandwidth / latency bound and need no staging.
#pragma once
#include <type_traits>
#include "mk_device.cuh"

namespace mk {

constexpr int kEwRows = 32, kEwCols = 512;                 // config.py EW_ROWS / EW_COLS
enum { EW_UNARY = 0, EW_BINARY, EW_SWIGLU, EW_MODULATE, EW_ROPE, EW_GATED };
enum { BIN_ADD = 0, BIN_SUB, BIN_MUL, BIN_MAX, BIN_MIN };

__device__ __forceinline__ float apply_bin(int fn, float a, float b) {
    switch (fn) {
        case BIN_ADD: return a + b;
        case BIN_SUB: return a - b;
        case BIN_MUL: return a * b;
        case BIN_MAX: return fmaxf(a, b);
        default: return fminf(a, b);
    }
}

// MK_OP_FINALIZE: out = act(ws + bias) + residual; ws = 0.
// ptr 0 ws (fp32), 1 out, 2 bias, 3 residual; i 0 R, 1 C, 2 act, 3 out dtype, 4 residual dtype,
// 5 rows per instruction (schedule.py finalize_rows; 0 = kEwRows)
// args: 0 row tile, 1 col tile (i5 x kEwCols)
static __device__ __noinline__ void op_finalize(const mk_op_desc* op, int a0, int a1) {
    const int R = op->i[0], Cc = op->i[1], act = op->i[2];
    const int tr = op->i[5] > 0 ? op->i[5] : kEwRows;
    const int r0 = a0 * tr, c0 = a1 * kEwCols;
    const int rows = min(tr, R - r0), cols = min(kEwCols, Cc - c0);
    const int vpr = cols >> 3;
    float* ws = reinterpret_cast<float*>(op->ptr[0]);
    for (int v = threadIdx.x; v < rows * vpr; v += kComputeThreads) {
        const int r = r0 + v / vpr, cidx = c0 + (v % vpr) * 8;
        float f[8], b[8];
        load8(ws, (long long)r * op->ld[0] + cidx, 1, f);
        if (op->ptr[2]) {
            load8(reinterpret_cast<const void*>(op->ptr[2]), cidx, 0, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] += b[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = apply_act(act, f[e]);
        if (op->ptr[3]) {
            load8(reinterpret_cast<const void*>(op->ptr[3]), (long long)r * op->ld[3] + cidx, op->i[4], b);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] += b[e];
        }
        store8(reinterpret_cast<void*>(op->ptr[1]), (long long)r * op->ld[1] + cidx, op->i[3], f);
        const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        store8(ws, (long long)r * op->ld[0] + cidx, 1, z);
    }
}

// a raw vector of 8 elements: 16 bytes when the element type is known to be 16-bit, else room for fp32
template <bool SIXTEEN> struct Raw8x;
template <> struct Raw8x<true> {
    uint4 v;
    __device__ __forceinline__ void load(const void* base, long long elem, int) { v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + elem)); }
    __device__ __forceinline__ void unpack(int dtype, float* f) const { Raw8 r; r.lo = v; r.hi = v; unpack8_raw(r, dtype == DT_F16 ? DT_F16 : DT_BF16, f); }
};
template <> struct Raw8x<false> {
    Raw8 v;
    __device__ __forceinline__ void load(const void* base, long long elem, int dtype) { v = load8_raw(base, elem, dtype); }
    __device__ __forceinline__ void unpack(int dtype, float* f) const { unpack8_raw(v, dtype, f); }
};

// Binary / modulate tile whose rows all read ONE row of the second (and third) operand -- a per-image gate, scale or
// shift over that image's tokens: the thread keeps its 8 columns of them and streams a, eight rows in flight when a is 16-bit.
template <int MODE>
static __device__ __noinline__ void eltwise_tile_one_group(const mk_op_desc* op, int r0, int col, int rows, int rowp, int rpp) {
    const int fn = op->i[3], group = op->i[4];
    const int adt = op->i[6], bdt = op->i[7], cdt = op->i[8], odt = op->i[9];
    const void* A = reinterpret_cast<const void*>(op->ptr[0]);
    void* O = reinterpret_cast<void*>(op->ptr[3]);
    const long long grow = r0 / group;
    float b[8], cc[8];
    load8(reinterpret_cast<const void*>(op->ptr[1]), grow * op->ld[1] + col, bdt, b);
    if (MODE == EW_MODULATE) {
        load8(reinterpret_cast<const void*>(op->ptr[2]), grow * op->ld[2] + col, cdt, cc);
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] += 1.0f;
    }
    auto body = [&](auto tag) {
        constexpr bool S16 = decltype(tag)::value;
        constexpr int UN = S16 ? 8 : 4;
        for (int rr = rowp; rr < rows; rr += UN * rpp) {
            Raw8x<S16> ra[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u)
                if (rr + u * rpp < rows) ra[u].load(A, (long long)(r0 + rr + u * rpp) * op->ld[0] + col, adt);
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                if (rr + u * rpp >= rows) continue;
                float a[8];
                ra[u].unpack(adt, a);
                if (MODE == EW_MODULATE) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] = fmaf(a[e], b[e], cc[e]);
                } else if (fn == BIN_MUL) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] *= b[e];
                } else if (fn == BIN_ADD) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] += b[e];
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] = apply_bin(fn, a[e], b[e]);
                }
                store8(O, (long long)(r0 + rr + u * rpp) * op->ld[3] + col, odt, a);
            }
        }
    };
    if (adt != DT_F32) body(std::true_type{});
    else body(std::false_type{});
}

// One tile of a pointwise op other than rope.  A pointwise instruction is a few thousand elements; with the mode, the
// function and the tile geometry as run-time switches and divisions inside the vector loop it was instruction-bound
// (8.7 us for a 32 x 512 modulate tile: ~300 instructions per 8-element vector at a fraction of an instruction per
// cycle; more loads in flight changed nothing).  Here the mode is a template parameter, the function is switched once
// per vector, a thread keeps its columns and walks rows (no division in the loop), and two rows are in flight.
template <int MODE, bool SIXTEEN>
static __device__ __noinline__ void eltwise_tile(const mk_op_desc* op, int r0, int c0, int rows, int cols) {
    const int fn = op->i[3], group = op->i[4];
    const int adt = op->i[6], bdt = op->i[7], cdt = op->i[8], odt = op->i[9];
    const void* A = reinterpret_cast<const void*>(op->ptr[0]);
    const void* B = reinterpret_cast<const void*>(op->ptr[1]);
    const void* Cp = reinterpret_cast<const void*>(op->ptr[2]);
    void* O = reinterpret_cast<void*>(op->ptr[3]);
    constexpr bool HASB = MODE != EW_UNARY, HASC = MODE == EW_MODULATE, GROUPED = MODE == EW_BINARY || MODE == EW_MODULATE;
    const int vpr = cols >> 3;                                   // vectors per row: at most 64
    // threads cover whole rows side by side: thread -> (row of the pass, vector of the row)
    const int tpr = vpr <= 1 ? 1 : vpr <= 2 ? 2 : vpr <= 4 ? 4 : vpr <= 8 ? 8 : vpr <= 16 ? 16 : vpr <= 32 ? 32 : 64;   // threads per row
    const int rpp = kComputeThreads / tpr;                       // rows per pass
    const int vec = threadIdx.x & (tpr - 1), rowp = threadIdx.x / tpr;
    if (vec >= vpr) return;
    const int col = c0 + vec * 8;
    if (GROUPED && (r0 / group) == ((r0 + rows - 1) / group)) {
        // every row of the tile reads the same row of b (and c): a thread's column of them is loaded once, and only a streams
        eltwise_tile_one_group<MODE>(op, r0, col, rows, rowp, rpp);
        return;
    }
    // rows in flight per thread: with 16-bit operands a vector is four registers and a thread's whole share of the tile
    // (eight rows) fits; otherwise two (more spill, and a spill is an L2 round trip like the loads it was to hide)
    constexpr int UN = SIXTEEN ? (HASC ? 2 : HASB ? 4 : 8) : 2;
    for (int rr = rowp; rr < rows; rr += UN * rpp) {
        Raw8x<SIXTEEN> ra[UN], rb[HASB ? UN : 1], rc[HASC ? UN : 1];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int r = r0 + rr + u * rpp;
            if (rr + u * rpp >= rows) continue;
            ra[u].load(A, (long long)r * op->ld[0] + col, adt);
            const long long rb_row = GROUPED ? r / group : r;
            if (HASB) rb[u].load(B, rb_row * op->ld[1] + col, bdt);
            if (HASC) rc[u].load(Cp, rb_row * op->ld[2] + col, cdt);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int r = r0 + rr + u * rpp;
            if (rr + u * rpp >= rows) continue;
            float a[8], b[8], cc[8];
            ra[u].unpack(adt, a);
            if (HASB) rb[u].unpack(bdt, b);
            if (MODE == EW_UNARY) {
                switch (fn) {
                    case ACT_NONE: break;
                    case ACT_SILU:
#pragma unroll
                        for (int e = 0; e < 8; ++e) a[e] = a[e] * sigmoidf_(a[e]);
                        break;
                    default:
#pragma unroll
                        for (int e = 0; e < 8; ++e) a[e] = apply_act(fn, a[e]);
                }
            } else if (MODE == EW_BINARY) {
                switch (fn) {
                    case BIN_ADD:
#pragma unroll
                        for (int e = 0; e < 8; ++e) a[e] += b[e];
                        break;
                    case BIN_MUL:
#pragma unroll
                        for (int e = 0; e < 8; ++e) a[e] *= b[e];
                        break;
                    default:
#pragma unroll
                        for (int e = 0; e < 8; ++e) a[e] = apply_bin(fn, a[e], b[e]);
                }
            } else if (MODE == EW_SWIGLU) {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = apply_act(fn, a[e]) * b[e];
            } else {  // EW_MODULATE: x * (1 + scale[g]) + shift[g]
                rc[u].unpack(cdt, cc);
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = fmaf(a[e], 1.0f + b[e], cc[e]);
            }
            store8(O, (long long)r * op->ld[3] + col, odt, a);
        }
    }
}

// EW_GATED: out = fn(a, b * c[r / group]) -- a gated residual, x + y * gate[image] (passes.fuse_pointwise).  a and b
// stream (two rows in flight), the gate row of a tile is loaded once when the tile lies in one group.
static __device__ __noinline__ void eltwise_tile_gated(const mk_op_desc* op, int r0, int c0, int rows, int cols) {
    const int fn = op->i[3], group = op->i[4];
    const int adt = op->i[6], bdt = op->i[7], cdt = op->i[8], odt = op->i[9];
    const void* A = reinterpret_cast<const void*>(op->ptr[0]);
    const void* B = reinterpret_cast<const void*>(op->ptr[1]);
    const void* G = reinterpret_cast<const void*>(op->ptr[2]);
    void* O = reinterpret_cast<void*>(op->ptr[3]);
    const int vpr = cols >> 3;
    const int tpr = vpr <= 1 ? 1 : vpr <= 2 ? 2 : vpr <= 4 ? 4 : vpr <= 8 ? 8 : vpr <= 16 ? 16 : vpr <= 32 ? 32 : 64;
    const int rpp = kComputeThreads / tpr;
    const int vec = threadIdx.x & (tpr - 1), rowp = threadIdx.x / tpr;
    if (vec >= vpr) return;
    const int col = c0 + vec * 8;
    const bool one = (r0 / group) == ((r0 + rows - 1) / group);
    float gt[8];
    if (one) load8(G, (long long)(r0 / group) * op->ld[2] + col, cdt, gt);
    constexpr int UN = 2;
    for (int rr = rowp; rr < rows; rr += UN * rpp) {
        Raw8 ra[UN], rb[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int r = r0 + rr + u * rpp;
            if (rr + u * rpp >= rows) continue;
            ra[u] = load8_raw(A, (long long)r * op->ld[0] + col, adt);
            rb[u] = load8_raw(B, (long long)r * op->ld[1] + col, bdt);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int r = r0 + rr + u * rpp;
            if (rr + u * rpp >= rows) continue;
            float a[8], b[8];
            unpack8_raw(ra[u], adt, a);
            unpack8_raw(rb[u], bdt, b);
            if (!one) load8(G, (long long)(r / group) * op->ld[2] + col, cdt, gt);
            if (fn == BIN_ADD) {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = fmaf(b[e], gt[e], a[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = apply_bin(fn, a[e], b[e] * gt[e]);
            }
            store8(O, (long long)r * op->ld[3] + col, odt, a);
        }
    }
}

// MK_OP_ELTWISE.  ptr 0 a (x / gate), 1 b (b / up / scale / cos), 2 c (shift / sin), 3 out
// i 0 R, 1 C, 2 mode, 3 fn (activation or binary code), 4 group (rows of a per row of b; rope: seq),
//   5 head_dim (rope), 6..9 dtypes of a, b, c, out (DT_*).  args: 0 row tile, 1 col tile.
static __device__ __noinline__ void op_eltwise(const mk_op_desc* op, int a0, int a1) {
    const int R = op->i[0], Cc = op->i[1], mode = op->i[2], fn = op->i[3], group = op->i[4];
    const int adt = op->i[6], bdt = op->i[7], cdt = op->i[8], odt = op->i[9];
    const int r0 = a0 * kEwRows, c0 = a1 * kEwCols;
    const int rows = min(kEwRows, R - r0), cols = min(kEwCols, Cc - c0);
    const void* A = reinterpret_cast<const void*>(op->ptr[0]);
    const void* B = reinterpret_cast<const void*>(op->ptr[1]);
    const void* Cp = reinterpret_cast<const void*>(op->ptr[2]);
    void* O = reinterpret_cast<void*>(op->ptr[3]);
    if (mode == EW_ROPE) {
        const int D = op->i[5], half = D >> 1, hv = half >> 3;        // vectors per half head
        const int heads = cols / D;
        const int units = rows * heads * hv;
        for (int u = threadIdx.x; u < units; u += kComputeThreads) {
            const int r = r0 + u / (heads * hv);
            const int rem = u % (heads * hv);
            const int col = c0 + (rem / hv) * D + (rem % hv) * 8;
            const int tok = r % group, dc = (rem % hv) * 8;
            float x1[8], x2[8], c1[8], c2[8], s1[8], s2[8], o1[8], o2[8];
            load8(A, (long long)r * op->ld[0] + col, adt, x1);
            load8(A, (long long)r * op->ld[0] + col + half, adt, x2);
            load8(B, (long long)tok * op->ld[1] + dc, bdt, c1);
            load8(B, (long long)tok * op->ld[1] + dc + half, bdt, c2);
            load8(Cp, (long long)tok * op->ld[2] + dc, cdt, s1);
            load8(Cp, (long long)tok * op->ld[2] + dc + half, cdt, s2);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                o1[e] = x1[e] * c1[e] - x2[e] * s1[e];
                o2[e] = x2[e] * c2[e] + x1[e] * s2[e];
            }
            store8(O, (long long)r * op->ld[3] + col, odt, o1);
            store8(O, (long long)r * op->ld[3] + col + half, odt, o2);
        }
        return;
    }
    if (mode == EW_GATED) { eltwise_tile_gated(op, r0, c0, rows, cols); return; }
    const bool all16 = adt != DT_F32 && (mode == EW_UNARY || bdt != DT_F32) && (mode != EW_MODULATE || cdt != DT_F32);
    if (all16) {
        switch (mode) {
            case EW_UNARY: eltwise_tile<EW_UNARY, true>(op, r0, c0, rows, cols); break;
            case EW_BINARY: eltwise_tile<EW_BINARY, true>(op, r0, c0, rows, cols); break;
            case EW_SWIGLU: eltwise_tile<EW_SWIGLU, true>(op, r0, c0, rows, cols); break;
            default: eltwise_tile<EW_MODULATE, true>(op, r0, c0, rows, cols); break;
        }
        return;
    }
    switch (mode) {
        case EW_UNARY: eltwise_tile<EW_UNARY, false>(op, r0, c0, rows, cols); break;
        case EW_BINARY: eltwise_tile<EW_BINARY, false>(op, r0, c0, rows, cols); break;
        case EW_SWIGLU: eltwise_tile<EW_SWIGLU, false>(op, r0, c0, rows, cols); break;
        default: eltwise_tile<EW_MODULATE, false>(op, r0, c0, rows, cols); break;
    }
}

// (Each instance is a function of its own: inlined into one body, the longer variants' registers and spills fell on
// the one-vector-per-thread case too, which is the norm of every decode step.)
// A row (or a lane's share of it) of at most NPER vectors per thread stays in registers between the two passes: every
// vector is requested before the first is used, and gain and bias come in pairs.  (Requested one by one,
// the vectors of a 2048-column row cost eight L2 round trips in each pass: 11 us per 8-row instruction.)
template <int NPER, bool MOD, bool X16 = false>
static __device__ __noinline__ void norm_kept(const mk_op_desc* op, int r, int first, int step, int nvec, bool live, uint8_t* work) {
    const int Cc = op->i[1], rms = op->i[2], rpi = op->i[3], xdt = op->i[4], odt = op->i[5];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const void* X = reinterpret_cast<const void*>(op->ptr[0]);
    void* O = reinterpret_cast<void*>(op->ptr[1]);
    const void* W = reinterpret_cast<const void*>(op->ptr[2]);
    const void* Bv = reinterpret_cast<const void*>(op->ptr[3]);
    const void* Sc = reinterpret_cast<const void*>(op->ptr[4]);          // adaLN modulation fused in (passes.fuse_pointwise), or null
    const void* Sh = reinterpret_cast<const void*>(op->ptr[5]);
    const long long grow = live ? r / max(1, op->i[6]) : 0;
    Raw8x<X16> kr[NPER];                                  // (a 16-bit row: four registers per vector, eight vectors per lane fit)
#pragma unroll
    for (int u = 0; u < NPER; ++u) {
        const int v = first + u * step;
        if (live && v < nvec) kr[u].load(X, (long long)r * op->ld[0] + v * 8, xdt);
    }
    // gain, bias (and modulation) of the first batch are requested with the row: for a row of one vector per thread --
    // the norm of a decode step -- that is ONE L2 round trip on the instruction's critical path instead of two
    constexpr int NB = (NPER < 2 || MOD) ? 1 : 2;                  // (with the modulation's two more operands: one at a time)
    Raw8 gw[NB], bw[NB], sw[MOD ? NB : 1], tw[MOD ? NB : 1];
    auto request = [&](int u0) {
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            const int v = first + (u0 + u) * step;
            if (live && v < nvec) {
                if (W) gw[u] = load8_raw(W, v * 8, 0);
                if (Bv) bw[u] = load8_raw(Bv, v * 8, 0);
                if (MOD) {
                    sw[u] = load8_raw(Sc, grow * op->ld[4] + v * 8, op->i[7]);
                    tw[u] = load8_raw(Sh, grow * op->ld[5] + v * 8, op->i[8]);
                }
            }
        }
    };
    request(0);
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int u = 0; u < NPER; ++u) {
        if (live && first + u * step < nvec) {
            float f[8];
            kr[u].unpack(xdt, f);
#pragma unroll
            for (int e = 0; e < 8; ++e) { s += f[e]; ss += f[e] * f[e]; }
        }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    if (rpi == 1) {
        float* sh = reinterpret_cast<float*>(work);
        if (lane == 0) { sh[warp * 2] = s; sh[warp * 2 + 1] = ss; }
        compute_sync();
        s = 0.f; ss = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kComputeWarps; ++w8) { s += sh[w8 * 2]; ss += sh[w8 * 2 + 1]; }
    }
    if (!live) return;
    const float mean = rms ? 0.f : s / (float)Cc;
    const float var = ss / (float)Cc - mean * mean;
    const float rstd = rsqrt_approx(var + op->f[0]);
#pragma unroll
    for (int u0 = 0; u0 < NPER; u0 += NB) {
        if (u0 > 0) request(u0);
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            const int v = first + (u0 + u) * step;
            if (v >= nvec) continue;
            float f[8], g[8];
            kr[u0 + u].unpack(xdt, f);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = (f[e] - mean) * rstd;
            if (W) {
                unpack8_raw(gw[u], 0, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] *= g[e];
            }
            if (Bv) {
                unpack8_raw(bw[u], 0, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += g[e];
            }
            if (MOD) {
                float h[8];
                unpack8_raw(sw[u], op->i[7], g);
                unpack8_raw(tw[u], op->i[8], h);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = fmaf(f[e], 1.0f + g[e], h[e]);
            }
            store8(O, (long long)r * op->ld[1] + v * 8, odt, f);
        }
    }
}

// MK_OP_NORM.  ptr 0 x, 1 out, 2 weight, 3 bias, 4 scale, 5 shift (adaLN modulation of the normalised row fused in:
// out = norm(x) * (1 + scale[r / group]) + shift[r / group]; or null); i 0 R, 1 C, 2 rms, 3 rows per instruction (8: one
// row per warp, 1: one row over the whole CTA), 4 x dtype, 5 out dtype, 6 group, 7 scale dtype, 8 shift dtype; f 0 eps.
// args: 0 row tile.
// var = E[x^2] - mean^2 in fp32 (as the reference's norm kernel, megacute/ops/norm.py:94-114).
static __device__ __noinline__ void op_norm(const mk_op_desc* op, int a0, uint8_t* work) {
    const int R = op->i[0], Cc = op->i[1], rms = op->i[2], rpi = op->i[3], xdt = op->i[4], odt = op->i[5];
    const float eps = op->f[0];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const void* X = reinterpret_cast<const void*>(op->ptr[0]);
    void* O = reinterpret_cast<void*>(op->ptr[1]);
    const void* W = reinterpret_cast<const void*>(op->ptr[2]);
    const void* Bv = reinterpret_cast<const void*>(op->ptr[3]);
    const int nvec = Cc >> 3;
    int r, first, step;
    if (rpi == 1) { r = a0; first = threadIdx.x; step = kComputeThreads; }
    else { r = a0 * kComputeWarps + warp; first = lane; step = 32; }
    const bool live = r < R;
    const int nper = (nvec + step - 1) / step;          // vectors per thread
    if (op->ptr[4] && nper <= 4) { norm_kept<4, true>(op, r, first, step, nvec, live, work); return; }
    if (nper <= 1) {
        // one vector per thread -- the norm of every decode step -- is done here, without a further call: the row's
        // vector, its gain and its bias are requested together (one L2 round trip on the instruction's critical path)
        float keep[8], gk[8], bk[8];
        float s = 0.f, ss = 0.f;
        if (live && first < nvec) {
            load8(X, (long long)r * op->ld[0] + first * 8, xdt, keep);
            if (W) load8(W, first * 8, 0, gk);
            if (Bv) load8(Bv, first * 8, 0, bk);
#pragma unroll
            for (int e = 0; e < 8; ++e) { s += keep[e]; ss += keep[e] * keep[e]; }
        }
        s = warp_sum(s);
        ss = warp_sum(ss);
        if (rpi == 1) {
            float* sh = reinterpret_cast<float*>(work);
            if (lane == 0) { sh[warp * 2] = s; sh[warp * 2 + 1] = ss; }
            compute_sync();
            s = 0.f; ss = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kComputeWarps; ++w8) { s += sh[w8 * 2]; ss += sh[w8 * 2 + 1]; }
        }
        if (!live || first >= nvec) return;
        const float mean = rms ? 0.f : s / (float)Cc;
        const float rstd = rsqrt_approx(ss / (float)Cc - mean * mean + eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            keep[e] = (keep[e] - mean) * rstd;
            if (W) keep[e] *= gk[e];
            if (Bv) keep[e] += bk[e];
        }
        store8(O, (long long)r * op->ld[1] + first * 8, odt, keep);
        return;
    }
    if (nper <= 2) { norm_kept<2, false>(op, r, first, step, nvec, live, work); return; }
    if (nper <= 4) { norm_kept<4, false>(op, r, first, step, nvec, live, work); return; }
    if (nper <= 8 && xdt != DT_F32 && !op->ptr[4]) { norm_kept<8, false, true>(op, r, first, step, nvec, live, work); return; }
    // longer rows: two passes over global memory, four vectors requested at a time
    float s = 0.f, ss = 0.f;
    constexpr int UN = 4;
    if (live)
        for (int v0 = first; v0 < nvec; v0 += UN * step) {
            Raw8 rx[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u)
                if (v0 + u * step < nvec) rx[u] = load8_raw(X, (long long)r * op->ld[0] + (v0 + u * step) * 8, xdt);
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                if (v0 + u * step >= nvec) continue;
                float f[8];
                unpack8_raw(rx[u], xdt, f);
#pragma unroll
                for (int e = 0; e < 8; ++e) { s += f[e]; ss += f[e] * f[e]; }
            }
        }
    s = warp_sum(s);
    ss = warp_sum(ss);
    if (rpi == 1) {
        float* sh = reinterpret_cast<float*>(work);
        if (lane == 0) { sh[warp * 2] = s; sh[warp * 2 + 1] = ss; }
        compute_sync();
        s = 0.f; ss = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kComputeWarps; ++w8) { s += sh[w8 * 2]; ss += sh[w8 * 2 + 1]; }
    }
    if (!live) return;
    const float mean = rms ? 0.f : s / (float)Cc;
    const float var = ss / (float)Cc - mean * mean;
    const float rstd = rsqrt_approx(var + eps);
    for (int v0 = first; v0 < nvec; v0 += 2 * step) {
        Raw8 rx[2], gw[2], bw[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = v0 + u * step;
            if (v >= nvec) continue;
            rx[u] = load8_raw(X, (long long)r * op->ld[0] + v * 8, xdt);
            if (W) gw[u] = load8_raw(W, v * 8, 0);
            if (Bv) bw[u] = load8_raw(Bv, v * 8, 0);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = v0 + u * step;
            if (v >= nvec) continue;
            float f[8], g[8];
            unpack8_raw(rx[u], xdt, f);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = (f[e] - mean) * rstd;
            if (W) {
                unpack8_raw(gw[u], 0, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] *= g[e];
            }
            if (Bv) {
                unpack8_raw(bw[u], 0, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += g[e];
            }
            if (op->ptr[4]) {                                   // adaLN modulation fused in
                const long long grow = r / max(1, op->i[6]);
                float h[8];
                load8(reinterpret_cast<const void*>(op->ptr[4]), grow * op->ld[4] + v * 8, op->i[7], g);
                load8(reinterpret_cast<const void*>(op->ptr[5]), grow * op->ld[5] + v * 8, op->i[8], h);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = fmaf(f[e], 1.0f + g[e], h[e]);
            }
            store8(O, (long long)r * op->ld[1] + v * 8, odt, f);
        }
    }
}

// Rotate-half of one 8-wide chunk pair.  x1/x2: chunks at d and d + D/2; result rounded to bf16.
__device__ __forceinline__ void rope8(const float* x1, const float* x2, const void* cosr, const void* sinr, int d,
                                      int half, float* o1, float* o2) {
    float c1[8], c2[8], s1[8], s2[8];
    load8(cosr, d, 0, c1); load8(cosr, d + half, 0, c2);
    load8(sinr, d, 0, s1); load8(sinr, d + half, 0, s2);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        o1[e] = round_bf16(x1[e] * c1[e] - x2[e] * s1[e]);
        o2[e] = round_bf16(x2[e] * c2[e] + x1[e] * s2[e]);
    }
}

// MK_OP_ROPE_APPEND.  ptr 0 qkv, 1 cos, 2 sin, 3 pos, 4 q_out, 5 k_cache, 6 v_cache
// i 0 B, 1 H, 2 KVH, 3 D, 4 max_seq, 5 qkv dtype, 6 pos stride.  args: 0 row tile (8 sequences).
// Cache row written for sequence b: b * max_seq + pos (reference: graph.py:375-379).
static __device__ __noinline__ void op_rope_append(const mk_op_desc* op, int a0) {
    const int B = op->i[0], H = op->i[1], KVH = op->i[2], D = op->i[3], L = op->i[4], qdt = op->i[5];
    const int* posp = reinterpret_cast<const int*>(op->ptr[3]);
    const long long pstride = op->i[6];                                   // 0: one position for the batch, else one per sequence
    const int half = D >> 1, hv = half >> 3;
    const int r0 = a0 * kComputeWarps;
    const int rows = min(kComputeWarps, B - r0);
    const void* qkv = reinterpret_cast<const void*>(op->ptr[0]);
    const int units = (H + KVH) * hv;
    for (int u = threadIdx.x; u < rows * units; u += kComputeThreads) {
        const int b = r0 + u / units, rem = u % units;
        const int hh = rem / hv, d = (rem % hv) * 8;
        const int pos = posp[b * pstride];
        const __nv_bfloat16* cosr = reinterpret_cast<const __nv_bfloat16*>(op->ptr[1]) + (long long)pos * op->ld[1];
        const __nv_bfloat16* sinr = reinterpret_cast<const __nv_bfloat16*>(op->ptr[2]) + (long long)pos * op->ld[2];
        float x1[8], x2[8], o1[8], o2[8];
        load8(qkv, (long long)b * op->ld[0] + hh * D + d, qdt, x1);
        load8(qkv, (long long)b * op->ld[0] + hh * D + d + half, qdt, x2);
        rope8(x1, x2, cosr, sinr, d, half, o1, o2);
        if (hh < H) {
            store8(reinterpret_cast<void*>(op->ptr[4]), (long long)b * op->ld[4] + hh * D + d, 0, o1);
            store8(reinterpret_cast<void*>(op->ptr[4]), (long long)b * op->ld[4] + hh * D + d + half, 0, o2);
        } else {
            const long long row = (long long)b * L + pos;
            store8(reinterpret_cast<void*>(op->ptr[5]), row * op->ld[5] + (hh - H) * D + d, 0, o1);
            store8(reinterpret_cast<void*>(op->ptr[5]), row * op->ld[5] + (hh - H) * D + d + half, 0, o2);
        }
    }
    const int nv = (KVH * D) >> 3;
    for (int u = threadIdx.x; u < rows * nv; u += kComputeThreads) {
        const int b = r0 + u / nv, v = u % nv;
        float f[8];
        load8(qkv, (long long)b * op->ld[0] + (H + KVH) * D + v * 8, qdt, f);
        store8(reinterpret_cast<void*>(op->ptr[6]), ((long long)b * L + posp[b * pstride]) * op->ld[6] + v * 8, 0, f);
    }
}

// MK_OP_GATHER: out[r] = table[ids[r]] -- the embedding lookup of a decode step as the launch's first
// instructions (the reference's step calls torch.index_select before its launch,
// examples/llama/llama1b.py:103-104).  An index outside the table reads row 0.
// ptr 0 table (bf16), 1 ids (int32 column), 2 out; i 0 rows, 1 cols, 2 table rows, 3 out dtype
// args: 0 row tile (8 rows, one per warp), 1 col tile (kEwCols)
static __device__ __noinline__ void op_gather(const mk_op_desc* op, int a0, int a1) {
    const int R = op->i[0], Cc = op->i[1], T = op->i[2], odt = op->i[3];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = a0 * kComputeWarps + warp;
    if (r >= R) return;
    int id = __ldcg(reinterpret_cast<const int*>(op->ptr[1]) + (long long)r * op->ld[1]);
    if (id < 0 || id >= T) id = 0;
    const int c0 = a1 * kEwCols, cols = min(kEwCols, Cc - c0);
    const void* row = reinterpret_cast<const __nv_bfloat16*>(op->ptr[0]) + (long long)id * op->ld[0];
    for (int v = lane; v < (cols >> 3); v += 32) {
        float f[8];
        load8(row, c0 + v * 8, DT_BF16, f);
        store8(reinterpret_cast<void*>(op->ptr[2]), (long long)r * op->ld[2] + c0 + v * 8, odt, f);
    }
}

// MK_OP_ARGMAX: ids[r] = argmax(x[r]), ties to the lowest index, NaN never selected -- greedy sampling as
// the launch's last instructions (the reference's step calls torch's argmax after its launch,
// examples/llama/llama1b.py:105).  A row is cut into `chunks` column ranges, one instruction each;
// every instruction leaves its best (value, index) in `part` and bumps the row's arrival count; the
// last to arrive picks the winner (one partial per thread) and resets the count.
// ptr 0 x, 1 ids (int32 column), 2 part (fp32, per row: `chunks` values, then from column ceil4(chunks) on the bits
// of their indices), 3 count
// i 0 rows, 1 cols, 2 chunks, 3 columns per chunk (multiple of 8), 4 x dtype.  args: 0 row, 1 chunk.
struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {        // NaN never wins; equal values: lower index
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, other);
    }
    return b;
}
static __device__ __noinline__ void op_argmax(const mk_op_desc* op, int a0, int a1, Ctrl* c, uint8_t* work) {
    const int Cc = op->i[1], chunks = op->i[2], width = op->i[3], xdt = op->i[4];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int r = a0, c0 = a1 * width, c1 = min(Cc, c0 + width);
    const void* X = reinterpret_cast<const void*>(op->ptr[0]);
    Best best{-__builtin_huge_valf(), 0x7fffffff};
    for (int col = c0 + t * 8; col < c1; col += kComputeThreads * 8) {
        float f[8];
        load8(X, (long long)r * op->ld[0] + col, xdt, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) best = better(best, Best{f[e], col + e});
    }
    best = warp_best(best);
    float* sv = reinterpret_cast<float*>(work);
    int* si = reinterpret_cast<int*>(work) + kComputeWarps;
    if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
    compute_sync();
    int* ids = reinterpret_cast<int*>(op->ptr[1]) + (long long)r * op->ld[1];
    if (warp == 0) {
        best = lane < kComputeWarps ? Best{sv[lane], si[lane]} : Best{-__builtin_huge_valf(), 0x7fffffff};
        best = warp_best(best);
        if (lane == 0) {
            if (chunks == 1) {
                *ids = best.i == 0x7fffffff ? 0 : best.i;
            } else {
                float* part = reinterpret_cast<float*>(op->ptr[2]) + (long long)r * op->ld[2];
                part[a1] = best.v;
                part[((chunks + 3) & ~3) + a1] = __int_as_float(best.i);
                __threadfence();
                int* count = reinterpret_cast<int*>(op->ptr[3]) + (long long)r * op->ld[3];
                const int old = atomicAdd(count, 1);
                c->flag = (old == chunks - 1);
                if (old == chunks - 1) *count = 0;            // back to zero for the next launch
            }
        }
    }
    if (chunks == 1) return;
    compute_sync();
    if (!c->flag) return;
    __threadfence();
    const float* part = reinterpret_cast<const float*>(op->ptr[2]) + (long long)r * op->ld[2];
    best = Best{-__builtin_huge_valf(), 0x7fffffff};
    if (t < chunks) best = Best{__ldcg(part + t), __float_as_int(__ldcg(part + ((chunks + 3) & ~3) + t))};
    best = warp_best(best);
    compute_sync();                                           // sv / si of the first pass have been read
    if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
    compute_sync();
    if (warp == 0) {
        best = lane < kComputeWarps ? Best{sv[lane], si[lane]} : Best{-__builtin_huge_valf(), 0x7fffffff};
        best = warp_best(best);
        if (lane == 0) *ids = best.i == 0x7fffffff ? 0 : best.i;
    }
}

// MK_OP_INCREMENT.  ptr 0 pos; i 0 rows of pos, 1 their stride.  One instruction.
__device__ __forceinline__ void op_increment(const mk_op_desc* op) {
    int* pos = reinterpret_cast<int*>(op->ptr[0]);
    const int rows = max(1, op->i[0]);
    for (int r = threadIdx.x; r < rows; r += kComputeThreads) pos[(long long)r * op->i[1]] += 1;
}

}  // namespace mk
