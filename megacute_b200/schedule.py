"""Scheduler: graph -> instruction stream, dependency counters and the encoded tables.

Plays the role of the reference's ``megacute/schedule.py`` (tile_op :62-199, schedule :281-339,
Schedule.encode :249-271) with a different construction:

1. ``tile_op`` cuts every op into instructions.  Each instruction has up to 7 integer arguments
   and, per operand, the rectangle of the buffer it reads or writes.  Linears with <= 8 activation
   rows are cut into one contiguous range of output columns per SM (weight streaming); everything
   else is cut into fixed tiles.
2. Instructions are numbered in program order; CTA ``c`` of a grid of ``G`` executes numbers
   ``c, c + G, c + 2G, ...`` in order, so every dependency points backwards and no cycle of waits
   can form.
3. Hazards (RAW / WAR / WAW, with commuting accumulations) are found per pair of ops with
   vectorised rectangle intersection.  For each operand the earlier accesses of the same buffer
   are walked newest to oldest and the walk stops as soon as an access that is already ordered
   before the instruction covers the operand -- everything older is then ordered transitively.
   This is what keeps a buffer that every layer rewrites (the residual stream) from collecting
   one wait per earlier layer.
4. All consumers that need the same set of producer instructions share one counter: the members
   arrive on it (release add), the consumers wait until it reaches ``len(members) * epoch``
   (acquire load).  Counters are never reset between launches.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from . import config as C
from .graph import Graph, Op, View
from .passes import gemv_eligible

READ, WRITE, ACCUM = "R", "W", "A"
CONFLICTS = {READ: {WRITE, ACCUM}, WRITE: {READ, WRITE, ACCUM}, ACCUM: {READ, WRITE}}


def _ceil(a, b):
    return -(-a // b)


@dataclasses.dataclass
class Access:
    buf: object
    kind: str               # READ / WRITE / ACCUM
    boxes: np.ndarray       # [n, 4] int64: r0, r1, c0, c1 (half open, buffer coordinates) per instruction
    covers: bool            # the instructions together touch every cell of `rect`
    rect: tuple             # bounding rectangle of all boxes


@dataclasses.dataclass
class Tiled:
    args: np.ndarray        # [n, N_ARGS] int32
    accesses: list


def _boxes(v: View, r0, r1, c0, c1):
    """Rectangles in view coordinates (arrays or scalars), clipped to the view -> buffer coordinates."""
    r0, r1, c0, c1 = np.broadcast_arrays(*(np.asarray(a, dtype=np.int64) for a in (r0, r1, c0, c1)))
    out = np.stack([v.row0 + np.minimum(r0, v.rows), v.row0 + np.minimum(r1, v.rows),
                    v.col0 + np.minimum(c0, v.cols), v.col0 + np.minimum(c1, v.cols)], axis=1)
    return out


def _acc(v: View, kind, r0=None, r1=None, c0=None, c1=None, n=1, covers=True):
    if v is None:
        return None
    if r0 is None:
        r0, r1 = np.zeros(n, np.int64), np.full(n, v.rows, np.int64)
    if c0 is None:
        c0, c1 = np.zeros(n, np.int64), np.full(n, v.cols, np.int64)
    b = _boxes(v, r0, r1, c0, c1)
    if len(b) != n:
        b = np.broadcast_to(b, (n, 4)).copy()
    rect = (int(b[:, 0].min()), int(b[:, 1].max()), int(b[:, 2].min()), int(b[:, 3].max()))
    return Access(v.buf, kind, b, covers, rect)


def _args(n, *cols):
    a = np.zeros((n, C.N_ARGS), np.int32)
    for k, col in enumerate(cols):
        a[:, k] = col
    return a


def gemv_ranges(n_out: int, sm_count: int):
    """Output-column ranges of a streaming linear: as even as possible, one per SM."""
    n = max(1, min(sm_count, n_out))
    base, rem = divmod(n_out, n)
    sizes = np.full(n, base, np.int64)
    sizes[:rem] += 1
    ends = np.cumsum(sizes)
    return ends - sizes, ends


def gemm_raster(mt: int, nt: int, group: int = 8):
    """(m, n) tile order: `group` row blocks at a time so neighbouring instructions share weights in L2."""
    ms, ns = [], []
    for g0 in range(0, mt, group):
        rows = np.arange(g0, min(g0 + group, mt))
        ms.append(np.tile(rows, nt))
        ns.append(np.repeat(np.arange(nt), len(rows)))
    return np.concatenate(ms), np.concatenate(ns)


def is_gemv(op: Op) -> bool:
    return op.kind == "Linear" and gemv_eligible(op.x.rows, op.x.cols)


def tile_op(op: Op, sm_count: int) -> Tiled:
    k = op.kind
    if k == "Linear" and is_gemv(op):
        n_out = op.out.cols
        o0, o1 = gemv_ranges(n_out, sm_count)
        n = len(o0)
        if op.act == "swiglu":           # weight rows of output columns [o0, o1): 64-row gate / up blocks
            w0, w1 = (o0 // 64) * 128, _ceil(o1, 64) * 128
        else:
            w0, w1 = o0, o1
        acc = [_acc(op.x, READ, n=n), _acc(op.w, READ, w0, w1, n=n, covers=False), _acc(op.norm_w, READ, n=n),
               _acc(op.bias, READ, 0, 1, o0, o1, n=n), _acc(op.residual, READ, None, None, o0, o1, n=n),
               _acc(op.out, WRITE, None, None, o0, o1, n=n)]
        return Tiled(_args(n, o0, o1), [a for a in acc if a is not None])
    if k in ("Linear", "LinearSplit"):
        assert op.x.cols % C.GEMM_BK == 0, f"linear K={op.x.cols} must be a multiple of {C.GEMM_BK}"
        assert getattr(op, "norm_w", None) is None or k == "Linear"
        out = op.out if k == "Linear" else op.ws
        M = out.rows
        swi = k == "Linear" and op.act == "swiglu"
        BN = op.bn or C.GEMM_BN                       # weight rows per tile: 128, or 256 (passes.wide_tiles)
        on = BN // 2 if swi else BN
        m, nn = gemm_raster(_ceil(M, C.GEMM_BM), _ceil(out.cols, on))
        splits = op.splits if k == "LinearSplit" else 1
        kc = op.x.cols // splits
        m, nn, ks = np.repeat(m, splits), np.repeat(nn, splits), np.tile(np.arange(splits), len(m))
        n = len(m)
        r0, r1 = m * C.GEMM_BM, (m + 1) * C.GEMM_BM
        acc = [_acc(op.x, READ, r0, r1, ks * kc, (ks + 1) * kc, n=n),
               _acc(op.w, READ, nn * BN, (nn + 1) * BN, ks * kc, (ks + 1) * kc, n=n),
               _acc(out, ACCUM if k == "LinearSplit" else WRITE, r0, r1, nn * on, (nn + 1) * on, n=n)]
        if k == "Linear":
            acc += [_acc(op.bias, READ, 0, 1, nn * on, (nn + 1) * on, n=n),
                    _acc(op.residual, READ, r0, r1, nn * on, (nn + 1) * on, n=n)]
            assert op.norm_w is None and op.rms_eps is None, "norm folding is only done on the streaming path"
        return Tiled(_args(n, m, nn, ks), [a for a in acc if a is not None])
    if k in ("SplitFinalize", "Unary", "Binary", "SwiGLU", "Modulate", "Rope"):
        R, Cc = op.out.shape
        TR, TC = C.EW_ROWS, C.EW_COLS
        if k == "SplitFinalize":
            TR = finalize_rows(R, Cc)
        if k == "Rope":
            assert TC % op.head_dim == 0, "rope: head_dim must divide the pointwise tile width"
        rt, ct = np.divmod(np.arange(_ceil(R, TR) * _ceil(Cc, TC)), _ceil(Cc, TC))
        n = len(rt)
        r0, r1, c0, c1 = rt * TR, (rt + 1) * TR, ct * TC, (ct + 1) * TC
        t = lambda v, kind=READ: _acc(v, kind, r0, r1, c0, c1, n=n)
        if k == "SplitFinalize":
            acc = [t(op.ws), _acc(op.bias, READ, 0, 1, c0, c1, n=n), t(op.residual), t(op.out, WRITE), t(op.ws, WRITE)]
        elif k == "Unary":
            acc = [t(op.x), t(op.out, WRITE)]
        elif k == "Binary":
            gq = op.b_group
            acc = [t(op.a), _acc(op.b, READ, r0 // gq, -(-np.minimum(r1, R) // gq), c0, c1, n=n, covers=False),
                   t(op.out, WRITE)]
            if op.gate is not None:
                gg = op.gate_group
                acc.append(_acc(op.gate, READ, r0 // gg, -(-np.minimum(r1, R) // gg), c0, c1, n=n, covers=False))
        elif k == "SwiGLU":
            acc = [t(op.gate), t(op.up), t(op.out, WRITE)]
        elif k == "Modulate":
            gq = op.group
            bro = lambda v: _acc(v, READ, r0 // gq, -(-np.minimum(r1, R) // gq), c0, c1, n=n, covers=False)
            acc = [t(op.x), bro(op.scale), bro(op.shift), t(op.out, WRITE)]
        else:
            acc = [t(op.x), _acc(op.cos, READ, n=n), _acc(op.sin, READ, n=n), t(op.out, WRITE)]
        return Tiled(_args(n, rt, ct), [a for a in acc if a is not None])
    if k == "Norm":
        R = op.x.rows
        rows = norm_rows(R)
        rt = np.arange(_ceil(R, rows))
        n = len(rt)
        acc = [_acc(op.x, READ, rt * rows, (rt + 1) * rows, n=n), _acc(op.weight, READ, n=n), _acc(op.bias, READ, n=n),
               _acc(op.out, WRITE, rt * rows, (rt + 1) * rows, n=n)]
        if op.scale is not None:
            gq = op.group
            for v in (op.scale, op.shift):
                acc.append(_acc(v, READ, rt * rows // gq, -(-np.minimum((rt + 1) * rows, R) // gq), n=n, covers=False))
        return Tiled(_args(n, rt), [a for a in acc if a is not None])
    if k == "Attention":
        D, QP = op.head_dim, C.ATTN_BQ
        qt = _ceil(op.seq_q, QP)
        # causal: longest query tiles first so the long diagonal ones do not trail the launch
        q_order = np.arange(qt)[::-1] if op.causal else np.arange(qt)
        qi, b, h = (a.ravel() for a in np.meshgrid(q_order, np.arange(op.batch), np.arange(op.heads), indexing="ij"))
        n = len(qi)
        q0 = b * op.seq_q + qi * QP
        q1 = np.minimum(q0 + QP, (b + 1) * op.seq_q)
        k0 = b * op.seq_k
        k1 = k0 + (np.minimum(op.seq_k, (qi + 1) * QP) if op.causal else op.seq_k)
        hk = h // (op.heads // op.kv_heads)
        acc = [_acc(op.q, READ, q0, q1, h * D, (h + 1) * D, n=n),
               _acc(op.k, READ, k0, k1, hk * D, (hk + 1) * D, n=n, covers=False),
               _acc(op.v, READ, k0, k1, hk * D, (hk + 1) * D, n=n, covers=False),
               _acc(op.out, WRITE, q0, q1, h * D, (h + 1) * D, n=n)]
        return Tiled(_args(n, b, h, qi), acc)
    if k == "RopeAppend":
        B, L, RR = op.qkv.rows, op.max_seq, C.ROPE_APPEND_ROWS
        rt = np.arange(_ceil(B, RR))
        n = len(rt)
        r0, r1 = rt * RR, np.minimum((rt + 1) * RR, B)
        acc = [_acc(op.qkv, READ, r0, r1, n=n), _acc(op.cos, READ, n=n, covers=False),
               _acc(op.sin, READ, n=n, covers=False), _acc(op.pos, READ, n=n), _acc(op.q_out, WRITE, r0, r1, n=n),
               _acc(op.k_cache, WRITE, r0 * L, r1 * L, n=n, covers=False),
               _acc(op.v_cache, WRITE, r0 * L, r1 * L, n=n, covers=False)]
        return Tiled(_args(n, rt), acc)
    if k == "DecodeAttention":
        D, G, L, S = op.head_dim, op.heads // op.kv_heads, op.max_seq, op.splits
        hp = op.heads_per_inst or 1          # kv heads h .. h + hp - 1 per instruction (unsplit batched decode)
        b, h, s = (a.ravel() for a in np.meshgrid(np.arange(op.batch), np.arange(0, op.kv_heads, hp), np.arange(S),
                                                  indexing="ij"))
        n = len(b)
        cache = lambda v, kind: _acc(v, kind, b * L, (b + 1) * L, h * D, (h + hp) * D, n=n, covers=False)
        qcols = (h * G * D, (h + hp) * G * D)
        acc = [_acc(op.q, READ, b, b + 1, *qcols, n=n, covers=S == 1), _acc(op.pos, READ, n=n),
               cache(op.k_cache, READ), cache(op.v_cache, READ),
               _acc(op.out, WRITE, b, b + 1, *qcols, n=n, covers=S == 1)]
        if op.k_new is not None:
            acc += [_acc(op.k_new, READ, b, b + 1, h * D, (h + hp) * D, n=n, covers=S == 1),
                    _acc(op.v_new, READ, b, b + 1, h * D, (h + hp) * D, n=n, covers=S == 1),
                    _acc(op.cos, READ, n=n, covers=False), _acc(op.sin, READ, n=n, covers=False),
                    cache(op.k_cache, WRITE), cache(op.v_cache, WRITE)]
        if op.zero_inputs:      # q, k_new, v_new are a split-K workspace, zeroed by the pair's last instruction
            acc += [_acc(op.q, WRITE, b, b + 1, *qcols, n=n, covers=S == 1),
                    _acc(op.k_new, WRITE, b, b + 1, h * D, (h + hp) * D, n=n, covers=S == 1),
                    _acc(op.v_new, WRITE, b, b + 1, h * D, (h + hp) * D, n=n, covers=S == 1)]
        if S > 1:
            r = b * op.kv_heads + h
            acc += [_acc(op.part, WRITE, r * S, (r + hp) * S, n=n, covers=False),
                    _acc(op.count, WRITE, r, r + hp, n=n, covers=False)]
        return Tiled(_args(n, b, h, s), acc)
    if k == "Increment":
        return Tiled(_args(1), [_acc(op.pos, WRITE, n=1)])
    if k == "Gather":
        R, Cc = op.out.shape
        rt, ct = np.divmod(np.arange(_ceil(R, C.GATHER_ROWS) * _ceil(Cc, C.EW_COLS)), _ceil(Cc, C.EW_COLS))
        n = len(rt)
        r0, r1, c0, c1 = rt * C.GATHER_ROWS, (rt + 1) * C.GATHER_ROWS, ct * C.EW_COLS, (ct + 1) * C.EW_COLS
        return Tiled(_args(n, rt, ct), [_acc(op.ids, READ, r0, r1, n=n), _acc(op.table, READ, n=n, covers=False),
                                        _acc(op.out, WRITE, r0, r1, c0, c1, n=n)])
    if k == "Argmax":
        R, Cc = op.x.shape
        ch = op.chunks
        width = argmax_chunk_cols(Cc, ch)
        r, cidx = np.divmod(np.arange(R * ch), ch)
        n = len(r)
        acc = [_acc(op.x, READ, r, r + 1, cidx * width, (cidx + 1) * width, n=n), _acc(op.ids, WRITE, r, r + 1, n=n, covers=ch == 1)]
        if ch > 1:
            acc += [_acc(op.part, WRITE, r, r + 1, n=n, covers=False), _acc(op.count, WRITE, r, r + 1, n=n, covers=False)]
        return Tiled(_args(n, r, cidx), acc)
    raise NotImplementedError(k)


def argmax_chunk_cols(cols: int, chunks: int) -> int:
    """Columns per chunk of a split argmax: a multiple of 8 (16-byte loads of bf16)."""
    return _ceil(_ceil(cols, chunks), 8) * 8


def finalize_rows(rows: int, cols: int) -> int:
    """Rows per SplitFinalize instruction.  The op sits between two dependent linears; with few
    rows (batched decode) whole pointwise tiles would leave it a dozen instructions of eight
    dependent round trips each, so the tile is shortened until the op has about one instruction
    per SM."""
    tr = C.EW_ROWS
    while tr > C.FINALIZE_MIN_ROWS and _ceil(rows, tr) * _ceil(cols, C.EW_COLS) < C.FINALIZE_MIN_INSTS:
        tr //= 2
    return tr


def norm_rows(rows: int) -> int:
    """Rows per norm instruction: one per compute warp, or a single row spread over the whole CTA
    when the op has few rows (decode)."""
    return 1 if rows <= C.WIDE_NORM_ROWS else C.NORM_ROWS


# --------------------------------------------------------------------------------------------
# dependencies
# --------------------------------------------------------------------------------------------

def _overlap(bb: np.ndarray, ba: np.ndarray) -> np.ndarray:
    """[nB, nA] bool: does consumer box i intersect producer box j?"""
    if len(ba) == 1 or len(bb) == 1 or len(bb) * len(ba) <= (1 << 22):
        return ((bb[:, None, 0] < ba[None, :, 1]) & (ba[None, :, 0] < bb[:, None, 1]) &
                (bb[:, None, 2] < ba[None, :, 3]) & (ba[None, :, 2] < bb[:, None, 3]))
    out = np.empty((len(bb), len(ba)), bool)
    step = max(1, (1 << 22) // len(ba))
    for i in range(0, len(bb), step):
        out[i:i + step] = _overlap(bb[i:i + step], ba)
    return out


def _rect_hits(a, b) -> bool:
    return a[0] < b[1] and b[0] < a[1] and a[2] < b[3] and b[2] < a[3]


def _rect_in(inner, outer) -> bool:
    return outer[0] <= inner[0] and inner[1] <= outer[1] and outer[2] <= inner[2] and inner[3] <= outer[3]


class Inst:
    """Read-only record of one instruction (``prog.sched.insts[i]``)."""
    __slots__ = ("node", "args", "waits", "arrives", "cta")

    def __init__(self, node, args, waits, arrives, cta):
        self.node, self.args, self.waits, self.arrives, self.cta = node, args, waits, arrives, cta

    def __repr__(self):
        return f"Inst(node={self.node}, args={self.args}, waits={self.waits}, arrives={self.arrives})"


class _InstList:
    def __init__(self, s):
        self.s = s

    def __len__(self):
        return self.s.n

    def __getitem__(self, i):
        s = self.s
        if i < 0:
            i += s.n
        w0, w1 = s.wait_ptr[i], s.wait_ptr[i + 1]
        a0, a1 = s.arr_ptr[i], s.arr_ptr[i + 1]
        return Inst(int(s.op_of[i]), tuple(int(a) for a in s.args[i]),
                    [(int(c), int(t)) for c, t in zip(s.wait_cnt[w0:w1], s.wait_tgt[w0:w1])],
                    [int(c) for c in s.arr_cnt[a0:a1]], int(i % s.sm_count))

    def __iter__(self):
        return (self[i] for i in range(self.s.n))


@dataclasses.dataclass
class Schedule:
    graph: Graph
    sm_count: int
    n: int
    op_of: np.ndarray                   # [n] op index of every instruction
    args: np.ndarray                    # [n, N_ARGS]
    node_ranges: list                   # [start, end) of each op's instructions
    wait_ptr: np.ndarray                # [n + 1] CSR into wait_cnt / wait_tgt
    wait_cnt: np.ndarray
    wait_tgt: np.ndarray
    arr_ptr: np.ndarray                 # [n + 1] CSR into arr_cnt
    arr_cnt: np.ndarray
    num_counters: int
    counter_target: np.ndarray          # [num_counters] arrivals per launch

    @property
    def insts(self):
        return _InstList(self)

    def encode(self):
        """-> (insts [n, IW] int32, waits [2W] int32 as (counter, target) pairs, arrives [A] int32)."""
        w = np.zeros((self.n, C.IW), np.int32)
        w[:, C.W_OP] = self.op_of + 1
        w[:, C.W_ARG0:C.W_ARG0 + C.N_ARGS] = self.args
        w[:, C.W_NWAIT] = np.diff(self.wait_ptr)
        w[:, C.W_WAIT_OFF] = self.wait_ptr[:-1]
        w[:, C.W_NARRIVE] = np.diff(self.arr_ptr)
        w[:, C.W_ARRIVE_OFF] = self.arr_ptr[:-1]
        w[:, C.W_SEQ] = np.arange(self.n)
        waits = np.stack([self.wait_cnt, self.wait_tgt], 1).reshape(-1).astype(np.int32)
        pad = lambda a: a if len(a) else np.zeros(1, np.int32)
        return (torch.from_numpy(w), torch.from_numpy(pad(waits)), torch.from_numpy(pad(self.arr_cnt.astype(np.int32))))

    def summary(self) -> str:
        lines = [f"{self.n} instructions, {self.num_counters} counters, {len(self.wait_cnt)} waits"]
        for k, (op, (a, b)) in enumerate(zip(self.graph.ops, self.node_ranges)):
            lines.append(f"  node {k} {op.kind:<16} insts [{a}, {b})")
        return "\n".join(lines)


def schedule(g: Graph, sm_count: int = 148) -> Schedule:
    tiled = [tile_op(op, sm_count) for op in g.ops]
    starts = np.concatenate([[0], np.cumsum([len(t.args) for t in tiled])]).astype(np.int64)
    n = int(starts[-1])
    node_ranges = [(int(starts[k]), int(starts[k + 1])) for k in range(len(tiled))]
    op_of = np.concatenate([np.full(len(t.args), k, np.int32) for k, t in enumerate(tiled)]) if n else np.zeros(0, np.int32)
    args = np.concatenate([t.args for t in tiled]) if n else np.zeros((0, C.N_ARGS), np.int32)

    records: dict[int, list] = {}                 # buffer id -> [(op index, Access)] in program order
    counter_key: dict[tuple, int] = {}
    counter_members: list[np.ndarray] = []        # global instruction ids
    waits_of = [[] for _ in range(n)]             # per instruction: [(counter, target)]

    for kb, tb in enumerate(tiled):
        nb = len(tb.args)
        dep: dict[int, np.ndarray] = {}           # producer op -> [nb, na] bool
        for acc in tb.accesses:
            if acc.buf.kind in ("input", "param"):
                continue
            ordered: set = set()
            need = CONFLICTS[acc.kind]
            for ka, ra in reversed(records.get(acc.buf.id, ())):
                if ka == kb:
                    continue
                collect = ra.kind in need and ra.kind not in ordered
                if collect and _rect_hits(acc.rect, ra.rect):
                    o = _overlap(acc.boxes, ra.boxes)
                    if o.any():
                        dep[ka] = o if ka not in dep else (dep[ka] | o)
                if (collect or ra.kind in ordered) and ra.covers and _rect_in(acc.rect, ra.rect):
                    ordered |= CONFLICTS[ra.kind]
                if need <= ordered:
                    break
        for ka, o in sorted(dep.items()):
            a0 = node_ranges[ka][0]
            packed = np.packbits(o, axis=1)
            # consumers with the same producer set share a counter: group the packed rows (a dict on
            # the rows' bytes, visited in lexicographic order as np.unique(axis=0) would return them;
            # its structured-dtype sort took most of the scheduling time of a prefill graph)
            groups: dict[bytes, list[int]] = {}
            for i, row in enumerate(packed):
                groups.setdefault(row.tobytes(), []).append(i)
            for row_bytes in sorted(groups):
                rows = groups[row_bytes]
                members = np.nonzero(o[rows[0]])[0]
                if len(members) == 0:
                    continue
                key = (ka, row_bytes)
                c = counter_key.get(key)
                if c is None:
                    c = counter_key[key] = len(counter_members)
                    counter_members.append(members + a0)
                b0 = node_ranges[kb][0]
                for r in rows:
                    waits_of[b0 + r].append((c, len(members)))
        for acc in tb.accesses:
            if acc.buf.kind not in ("input", "param"):
                records.setdefault(acc.buf.id, []).append((kb, acc))

    wait_ptr = np.zeros(n + 1, np.int64)
    wait_ptr[1:] = np.cumsum([len(w) for w in waits_of])
    flat = [cw for w in waits_of for cw in w]
    wait_cnt = np.array([c for c, _ in flat], np.int64)
    wait_tgt = np.array([t for _, t in flat], np.int64)
    arr_lists = [[] for _ in range(n)]
    for c, members in enumerate(counter_members):
        for j in members:
            arr_lists[int(j)].append(c)
    arr_ptr = np.zeros(n + 1, np.int64)
    arr_ptr[1:] = np.cumsum([len(a) for a in arr_lists])
    arr_cnt = np.array([c for a in arr_lists for c in a], np.int64)
    target = np.array([len(m) for m in counter_members], np.int64)
    return Schedule(g, sm_count, n, op_of, args, node_ranges, wait_ptr, wait_cnt, wait_tgt, arr_ptr, arr_cnt,
                    len(counter_members), target)
