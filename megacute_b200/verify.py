"""Deterministic host checks of a compiled program: they stand where a memory-checking tool would.

The reference has nothing of the kind (its debug aid is an in-kernel watchdog that prints stuck
waits, ``megacute/kernel.py:91,117-131``).  A persistent kernel that trusts its tables can go wrong
in two ways no output comparison is guaranteed to catch: an instruction that addresses memory
outside its operands, and two instructions that touch the same memory without an ordering between
them.  Both are properties of the tables, so both are decided here, on the host, exactly:

``check_tables(prog)``
    For every op, the window of each operand that the kernel's address arithmetic can reach -- restated
    here per op kind from the descriptor's integers -- must lie inside the view the descriptor was
    encoded from, row pitch included; and every instruction's arguments must lie inside the op's
    tiling.  (The C library repeats the argument check at bind time for callers of the C ABI.)

``check_hazards(sched, g)``
    Happens-before closure over the encoded wait / arrival tables.  Instruction j happens before i
    when the same CTA runs j earlier (CTA c runs c, c + grid, ... in order), or i waits on a counter
    that j arrives on (a wait's target is the number of arrivals on that counter, so it waits for
    all of them), transitively.  Every pair of instructions of different ops whose accesses
    conflict (read/write, write/write, accumulate/read-or-write on intersecting rectangles of one
    buffer) must be so ordered, earlier program position first.  Exact: no sampling of executions.

``Program(..., debug=True)`` and ``MEGACUTE_B200_VERIFY=1`` run both at compile time.
"""

from __future__ import annotations

import numpy as np
import torch

from . import config as C
from .graph import Graph
from .schedule import CONFLICTS, Schedule, finalize_rows, is_gemv, norm_rows, tile_op


class VerifyError(AssertionError):
    pass


def _ceil(a, b):
    return -(-a // b)


# ---------------------------------------------------------------------------------------------------
# operand windows
# ---------------------------------------------------------------------------------------------------

def operand_windows(op) -> dict:
    """name -> (rows, cols): the part of each operand view, counted from its first element, that the
    kernel's op body can address for any legal instruction of the op."""
    k = op.kind
    if k in ("Linear", "LinearSplit"):
        M, K = op.x.shape
        out = op.out if k == "Linear" else op.ws
        n_out = out.cols
        swi = k == "Linear" and op.act == "swiglu"
        w_rows = 2 * n_out if swi else n_out
        win = {"x": (M, K), "w": (w_rows, K), ("out" if k == "Linear" else "ws"): (M, n_out)}
        if k == "Linear":
            win.update(bias=(1, n_out), residual=(M, n_out), norm_w=(1, K))
        return win
    if k == "SplitFinalize":
        R, Cc = op.out.shape
        return {"ws": (R, Cc), "out": (R, Cc), "bias": (1, Cc), "residual": (R, Cc)}
    if k == "Unary":
        return {"x": op.out.shape, "out": op.out.shape}
    if k == "Binary":
        R, Cc = op.out.shape
        w = {"a": (R, Cc), "b": (_ceil(R, op.b_group), Cc), "out": (R, Cc)}
        if op.gate is not None:
            w["gate"] = (_ceil(R, op.gate_group), Cc)
        return w
    if k == "SwiGLU":
        return {"gate": op.out.shape, "up": op.out.shape, "out": op.out.shape}
    if k == "Modulate":
        R, Cc = op.out.shape
        g = (_ceil(R, op.group), Cc)
        return {"x": (R, Cc), "scale": g, "shift": g, "out": (R, Cc)}
    if k == "Rope":
        R, Cc = op.out.shape
        return {"x": (R, Cc), "cos": (min(op.seq, R), op.head_dim), "sin": (min(op.seq, R), op.head_dim), "out": (R, Cc)}
    if k == "Norm":
        R, Cc = op.x.shape
        w = {"x": (R, Cc), "out": (R, Cc), "weight": (1, Cc), "bias": (1, Cc)}
        if op.scale is not None:
            w["scale"] = w["shift"] = (_ceil(R, op.group), Cc)
        return w
    if k == "Attention":
        D = op.head_dim
        q = (op.batch * op.seq_q, op.heads * D)
        kv = (op.batch * op.seq_k, op.kv_heads * D)
        return {"q": q, "k": kv, "v": kv, "out": q}
    if k == "RopeAppend":
        B, D, L = op.qkv.rows, op.head_dim, op.max_seq
        return {"qkv": (B, (op.heads + 2 * op.kv_heads) * D), "cos": (L, D), "sin": (L, D), "pos": (op.pos.rows, 1),
                "q_out": (B, op.heads * D), "k_cache": (B * L, op.kv_heads * D), "v_cache": (B * L, op.kv_heads * D)}
    if k == "DecodeAttention":
        B, D, L, S = op.batch, op.head_dim, op.max_seq, op.splits or 1
        G = op.heads // op.kv_heads
        cache = (B * L, op.kv_heads * D)       # the append row is b * L + pos with pos <= L - 1
        win = {"q": (B, op.heads * D), "k_cache": cache, "v_cache": cache, "pos": (op.pos.rows, 1), "out": (B, op.heads * D)}
        if op.k_new is not None:
            win.update(k_new=(B, op.kv_heads * D), v_new=(B, op.kv_heads * D), cos=(L, D), sin=(L, D))
        if S > 1:
            win.update(part=(B * op.kv_heads * S, G * D + 2 * G), count=(B * op.kv_heads, 1))
        return win
    if k == "Increment":
        return {"pos": (op.pos.rows, 1)}
    if k == "Gather":
        return {"table": op.table.shape, "ids": op.ids.shape, "out": op.out.shape}
    if k == "Argmax":
        win = {"x": op.x.shape, "ids": op.ids.shape}
        if op.chunks > 1:
            win.update(part=(op.x.rows, _ceil(op.chunks, 4) * 4 + op.chunks), count=(op.x.rows, 1))
        return win
    raise NotImplementedError(k)


def op_grid(op, sm_count: int):
    """Exclusive upper bounds of the instruction arguments of an op (None = not an index)."""
    k = op.kind
    if k == "Linear" and is_gemv(op):
        return ("range", op.out.cols)
    if k in ("Linear", "LinearSplit"):
        out = op.out if k == "Linear" else op.ws
        swi = k == "Linear" and op.act == "swiglu"
        bn = op.bn or C.GEMM_BN
        return (_ceil(out.rows, C.GEMM_BM), _ceil(out.cols, bn // 2 if swi else bn),
                op.splits if k == "LinearSplit" else 1)
    if k == "SplitFinalize":
        return (_ceil(op.out.rows, finalize_rows(*op.out.shape)), _ceil(op.out.cols, C.EW_COLS))
    if k in ("Unary", "Binary", "SwiGLU", "Modulate", "Rope"):
        return (_ceil(op.out.rows, C.EW_ROWS), _ceil(op.out.cols, C.EW_COLS))
    if k == "Norm":
        return (_ceil(op.x.rows, norm_rows(op.x.rows)),)
    if k == "Attention":
        return (op.batch, op.heads, _ceil(op.seq_q, C.ATTN_BQ))
    if k == "RopeAppend":
        return (_ceil(op.qkv.rows, C.ROPE_APPEND_ROWS),)
    if k == "DecodeAttention":
        return (op.batch, op.kv_heads - (op.heads_per_inst or 1) + 1, op.splits or 1)
    if k == "Increment":
        return ()
    if k == "Gather":
        return (_ceil(op.out.rows, C.GATHER_ROWS), _ceil(op.out.cols, C.EW_COLS))
    if k == "Argmax":
        return (op.x.rows, op.chunks)
    raise NotImplementedError(k)


def check_tables(g: Graph, sched: Schedule, tensors: dict | None = None) -> None:
    """Operand windows inside their views, views inside their buffers (and, with ``tensors`` -- buffer id
    -> bound tensor -- inside the bound storage), instruction arguments inside the op's tiling."""
    for kk, op in enumerate(g.ops):
        win = operand_windows(op)
        for name, v in op.view_fields():
            if name not in win:
                raise VerifyError(f"op {kk} {op.kind}: operand {name} has no window rule")
            r, c = win[name]
            if r > v.rows or c > v.cols:
                raise VerifyError(f"op {kk} {op.kind}.{name}: kernel window {r} x {c} exceeds the view {v}")
            b = v.buf
            if v.row0 < 0 or v.col0 < 0 or v.row0 + v.rows > b.rows or v.col0 + v.cols > b.cols:
                raise VerifyError(f"op {kk} {op.kind}.{name}: view {v} outside its buffer ({b.rows} x {b.cols})")
            if tensors is not None and b.id in tensors:
                t = tensors[b.id]
                if tuple(t.shape) != (b.rows, b.cols) or t.stride() != (b.cols, 1):
                    raise VerifyError(f"op {kk} {op.kind}.{name}: bound tensor {tuple(t.shape)} / strides {t.stride()} "
                                      f"is not the buffer ({b.rows} x {b.cols}, row-major)")
        a0, a1 = sched.node_ranges[kk]
        args = sched.args[a0:a1].astype(np.int64)
        lim = op_grid(op, sched.sm_count)
        if lim and lim[0] == "range":
            ok = (0 <= args[:, 0]).all() and (args[:, 0] < args[:, 1]).all() and (args[:, 1] <= lim[1]).all()
            # one contiguous, non-overlapping cover of the outputs
            ok = ok and args[0, 0] == 0 and args[-1, 1] == lim[1] and (args[1:, 0] == args[:-1, 1]).all()
            if not ok:
                raise VerifyError(f"op {kk} {op.kind}: output ranges do not partition [0, {lim[1]})")
            continue
        for j, hi in enumerate(lim):
            col = args[:, j]
            if (col < 0).any() or (col >= hi).any():
                bad = int(np.nonzero((col < 0) | (col >= hi))[0][0])
                raise VerifyError(f"op {kk} {op.kind}: instruction {a0 + bad} argument {j} = {int(col[bad])} outside [0, {hi})")
        if (args[:, len(lim):] != 0).any():
            raise VerifyError(f"op {kk} {op.kind}: unused instruction arguments are not zero")


# ---------------------------------------------------------------------------------------------------
# happens-before
# ---------------------------------------------------------------------------------------------------

def happens_before(s: Schedule) -> np.ndarray:
    """[n, ceil(n / 8)] packed bits: bit j of row i is set when instruction j happens before i."""
    n, grid = s.n, s.sm_count
    nb = _ceil(n, 8)
    reach = np.zeros((n, nb), np.uint8)
    bit = lambda j: (j >> 3, np.uint8(0x80 >> (j & 7)))          # numpy's packbits order: bit 7 first
    members: list[list[int]] = [[] for _ in range(s.num_counters)]
    for i in range(n):
        for c in s.arr_cnt[s.arr_ptr[i]:s.arr_ptr[i + 1]]:
            members[int(c)].append(i)
    behind_counter: dict[int, np.ndarray] = {}                   # counter -> everything that happens before its last arrival
    for i in range(n):
        row = reach[i]
        if i >= grid:
            j = i - grid
            row |= reach[j]
            byte, m = bit(j)
            row[byte] |= m
        for c, tgt in zip(s.wait_cnt[s.wait_ptr[i]:s.wait_ptr[i + 1]], s.wait_tgt[s.wait_ptr[i]:s.wait_ptr[i + 1]]):
            c = int(c)
            mem = members[c]
            if int(tgt) != len(mem):
                raise VerifyError(f"instruction {i}: waits for {int(tgt)} arrivals on counter {c}, which gets {len(mem)}")
            if mem and mem[-1] >= i:
                raise VerifyError(f"instruction {i}: waits on counter {c} whose arrival {mem[-1]} is not earlier in program order")
            acc = behind_counter.get(c)
            if acc is None:
                acc = np.zeros(nb, np.uint8)
                for j in mem:
                    acc |= reach[j]
                    byte, m = bit(j)
                    acc[byte] |= m
                behind_counter[c] = acc
            row |= acc
    return reach


def check_hazards(s: Schedule, g: Graph) -> int:
    """Every conflicting pair of accesses by instructions of different ops is ordered by the tables.
    Returns the number of conflicting instruction pairs checked."""
    reach = happens_before(s)
    tiled = [tile_op(op, s.sm_count) for op in g.ops]
    per_buf: dict[int, list] = {}
    for k, t in enumerate(tiled):
        if len(t.args) != s.node_ranges[k][1] - s.node_ranges[k][0]:
            raise VerifyError(f"op {k}: the schedule holds another number of instructions than the tiling")
        for a in t.accesses:
            if a.buf.kind not in ("input", "param"):
                per_buf.setdefault(a.buf.id, []).append((k, a))
    checked = 0
    for accs in per_buf.values():
        for x in range(len(accs)):
            kb, ab = accs[x]
            for y in range(x):
                ka, aa = accs[y]
                if ka == kb or aa.kind not in CONFLICTS[ab.kind]:
                    continue
                ra, rb = aa.rect, ab.rect
                if not (ra[0] < rb[1] and rb[0] < ra[1] and ra[2] < rb[3] and rb[2] < ra[3]):
                    continue
                bb, ba = ab.boxes, aa.boxes
                o = ((bb[:, None, 0] < ba[None, :, 1]) & (ba[None, :, 0] < bb[:, None, 1]) &
                     (bb[:, None, 2] < ba[None, :, 3]) & (ba[None, :, 2] < bb[:, None, 3]))
                if not o.any():
                    continue
                lo, hi = sorted((ka, kb))                       # program order: op lo first
                first, later = (aa, ab) if ka < kb else (ab, aa)
                o = o if ka < kb else o.T                        # [later instruction, earlier instruction]
                l0, e0 = s.node_ranges[hi][0], s.node_ranges[lo][0]
                li, ei = np.nonzero(o)
                gi, gj = l0 + li, e0 + ei
                have = (reach[gi, gj >> 3] & (0x80 >> (gj & 7)).astype(np.uint8)) != 0
                checked += len(gi)
                if not have.all():
                    w = int(np.nonzero(~have)[0][0])
                    raise VerifyError(f"unordered hazard on buffer '{first.buf.name}': instruction {int(gj[w])} (op {lo} "
                                      f"{g.ops[lo].kind}, {first.kind}) and instruction {int(gi[w])} (op {hi} {g.ops[hi].kind}, "
                                      f"{later.kind}) touch intersecting rectangles with no happens-before between them")
    return checked


def verify_program(prog) -> None:
    check_tables(prog.g, prog.sched, getattr(prog, "_bufs", None) or None)
    check_hazards(prog.sched, prog.g)
