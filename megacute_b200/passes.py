"""Graph rewrites applied by ``compile`` before scheduling: Graph -> Graph, each on a derived copy.

Same pass names and intent as the reference (``megacute/runtime.py:44-199``), re-decided for this
runtime's kernel:

  fold_norms           few-row RMSNorm feeding only linears -> computed inside those linears.
                       The reference folds the gain into a derived copy of the weights and applies
                       rstd in the GEMM epilogue; here the consuming instruction normalises its own
                       copy of the (<= 8 row) activation in shared memory before streaming weights,
                       so no second copy of any weight (e.g. the 525 MB lm_head) is made.
  split_k              tile GEMMs that cannot fill the SMs are split along K into partial
                       instructions that reduce-add into an fp32 workspace (+ SplitFinalize) or, for
                       a residual linear, straight into the residual stream.
  fuse_rope_attention  RopeAppend feeding only the next DecodeAttention -> one fused op.
  split_kv             decode attention instructions are multiplied along the key axis so that every
                       SM streams keys; the last split of a (sequence, kv head) pair to finish
                       combines the partials inside the op.
"""

from __future__ import annotations

import os

import torch

from . import config as C
from .graph import Buffer, Graph, Op, View


def _reads_buffer(ops, buf, outputs=()) -> bool:
    return any(v.buf is buf for op in ops for v in op.reads) or any(v.buf is buf for v in outputs)


def gemv_eligible(M: int, K: int) -> bool:
    """Does a linear with M activation rows of length K run on the weight-streaming GEMV path?
    The whole activation is kept in shared memory as fp32."""
    return M <= C.GEMV_MAX_ROWS and M * K * 4 <= C.GEMV_XBUF_BYTES


def fold_norms(g: Graph) -> Graph:
    out = g.derive()
    ops = list(g.ops)
    drop = set()
    for i, op in enumerate(ops):
        if not (op.kind == "Norm" and op.rms and op.bias is None and op.out.buf.kind == "temp"):
            continue
        if not gemv_eligible(op.x.rows, op.x.cols):
            continue
        users = [j for j in range(i + 1, len(ops)) if any(v.buf is op.out.buf for v in ops[j].reads)]
        ok = bool(users) and not _reads_buffer((), op.out.buf, g.outputs)
        for j in users:
            u = ops[j]
            ok = ok and u.kind == "Linear" and op.out.same(u.x) and u.rms_eps is None
            ok = ok and all(v is None or v.buf is not op.out.buf for v in (u.residual, u.bias))
        # the raw input must not be rewritten between the norm and its last user
        if ok:
            between = ops[i + 1:users[-1]]
            ok = not any(w.buf is op.x.buf for o in between for w in o.writes)
        if not ok:
            continue
        for j in users:
            ops[j] = ops[j].clone(x=op.x, norm_w=op.weight, rms_eps=float(op.eps))
        drop.add(i)
    out.ops = [o for i, o in enumerate(ops) if i not in drop]
    return out


def fuse_rope_attention(g: Graph) -> Graph:
    out = g.derive()
    ops: list[Op] = []
    for i, op in enumerate(g.ops):
        prev = ops[-1] if ops else None
        if (op.kind == "DecodeAttention" and op.k_new is None and prev is not None and prev.kind == "RopeAppend"
                and op.q.same(prev.q_out) and op.k_cache.same(prev.k_cache) and op.v_cache.same(prev.v_cache)
                and op.pos.same(prev.pos) and prev.q_out.buf.kind == "temp"
                and not _reads_buffer(g.ops[i + 1:], prev.q_out.buf, g.outputs)):
            H, KVH, D = prev.heads, prev.kv_heads, prev.head_dim
            qkv = prev.qkv
            ops[-1] = op.clone(q=qkv.cols_slice(0, H * D), k_new=qkv.cols_slice(H * D, KVH * D),
                               v_new=qkv.cols_slice((H + KVH) * D, KVH * D), cos=prev.cos, sin=prev.sin)
            continue
        ops.append(op)
    out.ops = ops
    return out


def kv_splits(pairs: int, max_seq: int, sm_count: int, head_dim: int = 64) -> int:
    """Instructions per (sequence, kv head) pair: the split count with the lowest modelled time
    waves x (fixed cost per instruction [+ partials and merge when split] + key tiles per split x time per tile),
    with constants measured on B200 (config.DEC_*).  The kernel works in tiles of 128 keys (64 for
    head_dim 128), so splitting below one tile buys nothing and only adds partials to merge.  Few
    pairs (batch 1) spread over one wave of SMs; many pairs stay unsplit until the cache is long
    enough to pay for the partials.  A split keeps at least MIN_SPLIT_KEYS keys of room.
    MEGACUTE_B200_KV_SPLITS overrides the choice (experiments)."""
    cap = max(1, min(max_seq // C.MIN_SPLIT_KEYS, C.MAX_KV_SPLITS))
    if os.environ.get("MEGACUTE_B200_KV_SPLITS"):
        return max(1, min(cap, int(os.environ["MEGACUTE_B200_KV_SPLITS"])))
    tile = 128 if head_dim <= 64 else 64
    best, best_cost = 1, float("inf")
    for s in range(1, cap + 1):
        waves = -(-(pairs * s) // sm_count)
        tiles = -(-(-(-max_seq // s)) // tile)
        merge = C.DEC_MERGE_US + C.DEC_MERGE_US_PER_SPLIT * s if s > 1 else 0.0
        cost = waves * (C.DEC_FIXED_US + merge + tiles * C.DEC_TILE_US)
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def kv_heads_per_instruction(pairs: int, kv_heads: int, max_seq: int, sm_count: int, head_dim: int = 64) -> int:
    """Unsplit decode attention with more (sequence, kv head) pairs than SMs (batched decode): how many
    kv heads of a sequence one instruction handles, one after the other.  An instruction's fetch,
    dependency wait and arrival are paid once, so fewer and longer instructions win as long as they
    still fill the SMs evenly: waves x (shared cost + heads x (per-head cost + tiles x time per tile)).
    MEGACUTE_B200_ATT_HEADS overrides the choice (experiments)."""
    if os.environ.get("MEGACUTE_B200_ATT_HEADS"):
        h = int(os.environ["MEGACUTE_B200_ATT_HEADS"])
        return h if h >= 1 and kv_heads % h == 0 else 1
    tiles = -(-max_seq // (128 if head_dim <= 64 else 64))
    best, best_cost = 1, float("inf")
    for h in (1, 2, 4, 8):
        if kv_heads % h:
            continue
        waves = -(-(pairs // h) // sm_count)
        cost = waves * (C.DEC_SHARED_US + h * (C.DEC_FIXED_US - C.DEC_SHARED_US + tiles * C.DEC_TILE_US))
        if cost < best_cost - 1e-9:
            best, best_cost = h, cost
    return best


def bulk_eligible(op: Op) -> bool:
    """Can this decode attention run in the many-sequence form (csrc/op_decode_bulk.cuh)?  One warp per
    kv head, head_dim 64, and cache views that are whole rows of their buffers, 128 bytes per kv head,
    so that consecutive rows are one contiguous run of memory."""
    if os.environ.get("MEGACUTE_B200_ATT_BULK") == "0" or getattr(op, "window", 0):      # (no sliding window in that form)
        return False
    whole = all(v.col0 == 0 and v.cols == v.buf.cols for v in (op.k_cache, op.v_cache))
    ok = op.head_dim == 64 and op.kv_heads <= C.COMPUTE_WARPS and whole and op.k_cache.cols == op.kv_heads * 64
    if os.environ.get("MEGACUTE_B200_ATT_BULK") == "1":
        return ok
    return ok and (op.batch >= C.BULK_MIN_BATCH or (op.batch >= C.BULK_MIN_BATCH_LONG and op.max_seq >= C.BULK_LONG_SEQ))


def bulk_kv_splits(batch: int, kv_heads: int, max_seq: int, sm_count: int) -> int:
    """KV splits per sequence in the many-sequence form: the count with the lowest modelled time
    rounds x (cost per instruction + 16-row tiles per split x time per tile), rounds = instructions per
    SM.  Long contexts want enough instructions to fill the last round evenly (batch 64: 2 splits
    leave 20 SMs idle, 9 splits fill 3.9 rounds of 4); the measured cost per instruction grows with
    the split count, which caps it.  MEGACUTE_B200_KV_SPLITS overrides the choice."""
    cap = max(1, min(max_seq // C.MIN_SPLIT_KEYS, C.MAX_KV_SPLITS))
    if os.environ.get("MEGACUTE_B200_KV_SPLITS"):
        return max(1, min(cap, int(os.environ["MEGACUTE_B200_KV_SPLITS"])))
    tile_us = C.BULK_TILE_US_PER_KB * kv_heads * 128 / 1024
    best, best_cost = 1, float("inf")
    for s in range(1, cap + 1):
        waves = -(-(batch * s) // sm_count)
        tiles = -(-(-(-max_seq // s)) // C.BULK_TILE_ROWS)
        cost = waves * (max(C.BULK_FIXED_US, C.BULK_US_PER_SPLIT * s - 3.0) + tiles * tile_us)
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def split_kv(g: Graph, sm_count: int) -> Graph:
    out = g.derive()
    ops = []
    for op in g.ops:
        if op.kind == "DecodeAttention" and op.splits == 1 and bulk_eligible(op):
            s = bulk_kv_splits(op.batch, op.kv_heads, op.max_seq, sm_count)
            op = op.clone(heads_per_inst=op.kv_heads, bulk=True)
            if s > 1:
                G, D = op.heads // op.kv_heads, op.head_dim
                cols = -(-(G * D + 2 * G) // 4) * 4          # per (kv head, split): O (G x D), running max (G), sum (G)
                part = out.workspace((op.batch * op.kv_heads * s, cols), torch.float32)
                count = out.workspace((op.batch * op.kv_heads, 1), torch.int32)
                op = op.clone(splits=s, part=part, count=count)
            ops.append(op)
            continue
        if op.kind == "DecodeAttention" and op.splits == 1:
            pairs = op.batch * op.kv_heads
            s = kv_splits(pairs, op.max_seq, sm_count, op.head_dim)
            if s == 1 and (pairs > sm_count or os.environ.get("MEGACUTE_B200_ATT_HEADS")):
                hpi = kv_heads_per_instruction(pairs, op.kv_heads, op.max_seq, sm_count, op.head_dim)
                if hpi > 1:
                    op = op.clone(heads_per_inst=hpi)
            if s > 1:
                G, D = op.heads // op.kv_heads, op.head_dim
                cols = -(-(G * D + 2 * G) // 4) * 4          # per split: O (G x D), running max (G), sum (G)
                s = min(s, C.DECODE_MERGE_BYTES // (cols * 4))   # the merging split holds all partial rows in shared memory
                if s < 2:
                    ops.append(op)
                    continue
                part = out.workspace((pairs * s, cols), torch.float32)
                count = out.workspace((pairs, 1), torch.int32)
                op = op.clone(splits=s, part=part, count=count)
        ops.append(op)
    out.ops = ops
    return out


def _retarget(v, alias):
    if v is None or v.buf.id not in alias:
        return v
    r = alias[v.buf.id]
    return View(r.buf, r.row0 + v.row0, r.col0 + v.col0, v.rows, v.cols)


def choose_k_splits(M: int, N: int, K: int, sm_count: int) -> int:
    """Split count for a tile GEMM.  Cost of a plan = waves x (fixed cost per instruction + operand
    bytes of one instruction at one SM's share of HBM bandwidth)."""
    bm, bn, bk = C.GEMM_BM, C.GEMM_BN, C.GEMM_BK
    mt, nt, kt = -(-M // bm), -(-N // bn), K // bk
    rows = min(M, bm)

    def cost(n_inst, k):
        return -(-n_inst // sm_count) * (C.INST_US + (bn + rows) * k * 2 / (C.SM_GBPS * 1e3))

    best, best_cost = 1, cost(mt * nt, K)
    if mt * nt >= sm_count:
        return 1
    for s in range(2, C.MAX_K_SPLITS + 1):
        if kt % s or kt // s < C.MIN_SPLIT_KTILES:
            continue
        c = cost(mt * nt * s, K // s)
        if c < best_cost:
            best, best_cost = s, c
    return best


def split_k(g: Graph, sm_count: int) -> Graph:
    out = g.derive()
    alias: dict[int, View] = {}      # id of a dropped output buffer -> residual view that now holds it
    ops: list[Op] = []
    src = list(g.ops)
    for i, op0 in enumerate(src):
        op = op0.clone(**{k: _retarget(v, alias) for k, v in op0.view_fields()}) if alias else op0
        if op.kind == "Linear" and op.act != "swiglu" and not gemv_eligible(op.x.rows, op.x.cols):
            M, K = op.x.shape
            s = choose_k_splits(M, op.w.rows, K, sm_count)
            if s > 1:
                r = op.residual
                whole = op.out.rect == (0, op.out.buf.rows, 0, op.out.buf.cols)
                inplace = (r is not None and op.bias is None and op.act is None and op.norm_w is None
                           and r.buf.kind == "temp" and op.out.buf.kind == "temp" and whole
                           and not _reads_buffer(src[i + 1:], r.buf))
                if inplace:
                    alias[op.out.buf.id] = r
                    new = Op("LinearSplit", x=op.x, w=op.w, ws=r, splits=s)
                    new.layer = op.layer
                    ops.append(new)
                    continue
                ws = out.workspace(op.out.shape, torch.float32)
                part = Op("LinearSplit", x=op.x, w=op.w, ws=ws, splits=s)
                fin = Op("SplitFinalize", ws=ws, out=op.out, bias=op.bias, act=op.act, residual=op.residual)
                part.layer = fin.layer = op.layer
                ops += [part, fin]
                continue
        ops.append(op)
    out.ops = ops
    out.outputs = [_retarget(v, alias) for v in g.outputs]
    return out


def _accepts(op: Op, field: str, dtype) -> bool:
    """Can the kernel read / write operand `field` of `op` in `dtype` (fp32 or fp16) instead of bf16?"""
    k = op.kind
    f32 = dtype == torch.float32
    if k == "Linear":
        streaming = gemv_eligible(op.x.rows, op.x.cols)
        if field == "x":                                # the tensor core takes 16-bit operands; the streaming linear converts
            return streaming or not f32
        return field in ("out", "residual")
    if k == "LinearSplit":
        return (field == "ws" and f32) or (field == "x" and not f32)
    if k == "SplitFinalize":
        return field in ("out", "residual") or (field == "ws" and f32)
    if k == "Norm":
        return field in ("x", "out")
    if k in ("Unary", "Binary", "SwiGLU", "Modulate"):
        return True
    if k == "Rope":
        return field in ("x", "out")
    if k == "Attention":                              # (q, k and v must end up with one dtype: promote_temps checks the trio)
        return not f32
    if k == "RopeAppend":
        return field == "qkv"
    if k == "Gather":
        return field == "out"
    if k == "Argmax":
        return field == "x"
    if k == "DecodeAttention":
        if field in ("q", "k_new", "v_new"):          # one dtype code covers all three
            return op.k_new is None or (op.q.buf is op.k_new.buf is op.v_new.buf)
        return field == "out"
    return False


# runtime-private activations up to this size are kept in fp32 when every op touching them can; larger
# ones (prefill, DiT: megabytes per tensor, streamed through L2 by bandwidth-bound pointwise ops) in fp16
F32_TEMP_BYTES = 4 << 20


def promote_temps(g: Graph) -> Graph:
    """Keep runtime-private activations in more than bf16's 8 significant bits wherever every op that
    touches them can: the residual stream, the QKV row, the attention output and the MLP hidden of a
    step are never seen by the caller, and rounding each of them to bf16 at every layer is the main
    source of drift against an fp32 evaluation (16 layers of the 1B shape: 1.5e-2 to 2.5e-2 rel-L2 on
    the logits with bf16 intermediates, ~2e-3 without).  fp32 for small tensors when every user
    accepts it (decode); otherwise fp16 -- the same bytes as bf16, 11 significant bits, accepted by the
    tensor cores as the A operand of a tile GEMM beside bf16 weights; conversions saturate at +-65504.
    Buffers the caller sees (inputs, params, states, outputs) keep their dtype.
    MEGACUTE_B200_BF16_TEMPS=1 leaves every temp in bf16."""
    out = g.derive()
    if os.environ.get("MEGACUTE_B200_BF16_TEMPS") == "1":
        return out
    users: dict[int, list] = {}
    for op in g.ops:
        for name, v in op.view_fields():
            users.setdefault(v.buf.id, []).append((op, name))
    swap: dict[int, Buffer] = {}
    for b in g.buffers:
        if b.kind != "temp" or b.dtype != torch.bfloat16 or b.id not in users:
            continue
        if any(v.buf is b for v in g.outputs):
            continue
        for dt in (torch.float32, torch.float16):
            if dt == torch.float32 and b.rows * b.cols * 4 > F32_TEMP_BYTES:
                continue
            if all(_accepts(op, name, dt) for op, name in users[b.id]):
                swap[b.id] = Buffer(b.name, b.rows, b.cols, dt, "temp")
                break
    # an attention's q, k and v share one dtype (one tensor-core instruction takes one operand type): a trio of
    # which not every member changes to fp16 stays as it was
    changed = True
    while changed:
        changed = False
        for op in g.ops:
            if op.kind != "Attention":
                continue
            new = [swap[v.buf.id].dtype if v.buf.id in swap else v.buf.dtype for v in (op.q, op.k, op.v)]
            if len(set(new)) > 1:
                for v in (op.q, op.k, op.v):
                    if swap.pop(v.buf.id, None) is not None:
                        changed = True
    if not swap:
        return out
    move = lambda v: View(swap[v.buf.id], v.row0, v.col0, v.rows, v.cols) if v is not None and v.buf.id in swap else v
    out.ops = [op.clone(**{k: move(v) for k, v in op.view_fields()}) for op in g.ops]
    out.buffers = [swap.get(b.id, b) for b in g.buffers]
    return out


def fuse_finalize_attention(g: Graph) -> Graph:
    """A split-K QKV projection leaves its sums in an fp32 workspace; when the SplitFinalize behind it
    is a plain copy (no bias, activation or residual, fp32 output) whose only reader is the fused
    decode attention, the attention reads the workspace itself and zeroes what it has read (the
    finalize's other duty), and the copy -- a dependency hop of ~9 us per layer in batched decode --
    is dropped."""
    if os.environ.get("MEGACUTE_B200_KEEP_FINALIZE"):
        return g
    out = g.derive()
    ops: list[Op] = []
    for i, op in enumerate(g.ops):
        prev = ops[-1] if ops else None
        if (op.kind == "DecodeAttention" and op.k_new is not None and prev is not None and prev.kind == "SplitFinalize"
                and prev.bias is None and prev.act is None and prev.residual is None
                and prev.out.buf.kind == "temp" and prev.out.buf.dtype == torch.float32
                and all(v.buf is prev.out.buf and v.rows == prev.out.rows and prev.out.row0 == v.row0
                        and prev.out.col0 <= v.col0 and v.col0 + v.cols <= prev.out.col0 + prev.out.cols
                        for v in (op.q, op.k_new, op.v_new))
                and not _reads_buffer(g.ops[i + 1:], prev.out.buf, g.outputs)):
            move = lambda v: prev.ws.cols_slice(v.col0 - prev.out.col0, v.cols)
            ops[-1] = op.clone(q=move(op.q), k_new=move(op.k_new), v_new=move(op.v_new), zero_inputs=True)
            continue
        ops.append(op)
    out.ops = ops
    return out


def wide_tiles(g: Graph, sm_count: int) -> Graph:
    """Tile linears with many rows get 128 x 256 output tiles when that is modelled faster: the main
    loop of a tile GEMM is bound by the operand bytes an SM draws from L2, and a 256-wide tile reuses
    each activation k-tile for two weight tiles (48 KB instead of 64 KB per 128 x 256 x 64 block).
    rounds x (k-tiles x time per k-tile + epilogue), rounds = instructions per SM.
    MEGACUTE_B200_WIDE_TILES=0 / 1 forces the choice where the shape allows it."""
    force = os.environ.get("MEGACUTE_B200_WIDE_TILES")
    out = g.derive()
    ops = []
    for op in g.ops:
        if op.kind in ("Linear", "LinearSplit") and not gemv_eligible(op.x.rows, op.x.cols) and not op.bn:
            M, K = op.x.shape
            N = op.w.rows
            splits = op.splits if op.kind == "LinearSplit" else 1
            if N % C.GEMM_BN_WIDE == 0 and K % (64 * splits) == 0 and M > C.WIDE_MIN_ROWS and force != "0":
                mt, kt = -(-M // C.GEMM_BM), K // 64 // splits
                narrow = -(-(mt * (N // C.GEMM_BN) * splits) // sm_count) * (kt * C.KTILE_US + C.EPILOGUE_US)
                wide = -(-(mt * (N // C.GEMM_BN_WIDE) * splits) // sm_count) * (kt * C.KTILE_US_WIDE + C.EPILOGUE_US_WIDE)
                if wide < narrow or force == "1":
                    op = op.clone(bn=C.GEMM_BN_WIDE)
        ops.append(op)
    out.ops = ops
    return out


def split_argmax(g: Graph, sm_count: int) -> Graph:
    """An argmax over few long rows is cut into column chunks, about two instructions per SM in all;
    every chunk leaves its best (value, index) in a workspace and the last chunk of a row to arrive
    picks the winner (the scheme of the split decode attention)."""
    out = g.derive()
    ops = []
    for op in g.ops:
        if op.kind == "Argmax" and op.part is None:
            rows, cols = op.x.shape
            chunks = max(1, min(C.ARGMAX_MAX_CHUNKS, -(-2 * sm_count // rows), cols // 1024))
            if chunks > 1:
                # per row: the chunks' best values, then (from a 16-byte boundary on) the bits of their indices
                op = op.clone(chunks=chunks, part=out.workspace((rows, 2 * (-(-chunks // 4) * 4)), torch.float32),
                              count=out.workspace((rows, 1), torch.int32))
        ops.append(op)
    out.ops = ops
    return out


def fuse_pointwise(g: Graph) -> Graph:
    """Two pointwise pairs of an adaLN block become one op each (no counterpart among the reference's passes; its graphs
    run them as written, examples/dit/model.py):

    * ``Norm -> Modulate``: ``norm(x) * (1 + scale[g]) + shift[g]`` in the norm's own pass over the row;
    * ``Binary(mul, y, gate[g]) -> Binary(add, x, .)``: ``x + y * gate[g]`` (a gated residual).

    Each pair's intermediate is a runtime-private tensor nothing else reads.  A pointwise op over an activation costs
    one read and one write of it plus a dependency hop: a DiT block drops from eight such ops to four.
    MEGACUTE_B200_NO_POINTWISE_FUSION=1 keeps the ops apart."""
    if os.environ.get("MEGACUTE_B200_NO_POINTWISE_FUSION") == "1":
        return g
    out = g.derive()
    ops: list[Op] = []
    for i, op in enumerate(g.ops):
        prev = ops[-1] if ops else None
        private = lambda v: v.buf.kind == "temp" and not _reads_buffer(g.ops[i + 1:], v.buf, g.outputs)
        if (op.kind == "Modulate" and prev is not None and prev.kind == "Norm" and prev.scale is None
                and op.x.same(prev.out) and private(prev.out)):
            ops[-1] = prev.clone(out=op.out, scale=op.scale, shift=op.shift, group=op.group)
            continue
        if (op.kind == "Binary" and op.fn == "add" and op.b_group == 1 and op.gate is None and prev is not None
                and prev.kind == "Binary" and prev.fn == "mul" and prev.gate is None and prev.b_group > 1):
            for mine, other in ((op.b, op.a), (op.a, op.b)):
                if mine.same(prev.out) and private(prev.out) and other.shape == op.out.shape:
                    ops[-1] = op.clone(a=other, b=prev.a, gate=prev.b, gate_group=prev.b_group)
                    break
            else:
                ops.append(op)
            continue
        ops.append(op)
    out.ops = ops
    return out


def run_all(g: Graph, sm_count: int) -> Graph:
    """The pass pipeline of ``compile`` (reference order: runtime.py:235, plus wide_tiles, split_argmax,
    fuse_pointwise, promote_temps and fuse_finalize_attention)."""
    g = split_argmax(split_kv(fuse_rope_attention(wide_tiles(split_k(fold_norms(g), sm_count), sm_count)), sm_count), sm_count)
    return fuse_finalize_attention(promote_temps(fuse_pointwise(g)))
