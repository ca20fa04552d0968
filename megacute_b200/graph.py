"""Graph IR of the megakernel runtime: 2-D buffers, rectangular views and the op set.

This module mirrors the public surface of the reference's ``megacute/graph.py`` (Buffer, View,
Graph and its builder methods, ``swiglu_weight``; reference lines 23-84 and 488-625) so graph
builders written for it run unchanged.  The internals are different: every op is an instance of
one ``Op`` class whose operands are described by a per-kind table (``OP_TABLE``), which is what
the passes, the scheduler and the device descriptor encoder walk.

Conventions shared with the reference:
  * a tensor is a row-major ``(rows, cols)`` buffer; higher-rank activations are flattened to
    ``(batch * seq, features)`` and heads are column ranges;
  * ops read and write *views* (windows of a buffer), so slicing is free and a dependency is an
    intersection of rectangles on one buffer;
  * buffer kinds: input / param (read only), state (caller owned, updated in place), temp / output
    (runtime owned), workspace (runtime owned, zero on entry to every launch).
"""

from __future__ import annotations

import itertools
from typing import Optional

import torch

ELEM_BYTES = {torch.bfloat16: 2, torch.float32: 4, torch.int32: 4, torch.float16: 2}
# device dtype codes of activations (csrc/mk_device.cuh DT_*).  fp16 is never a caller-visible dtype (the
# builder methods accept bf16 / fp32 / int32, as the reference does): only passes.promote_temps makes
# fp16 buffers, for runtime-private activations.
DTYPE_CODE = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2, torch.int32: 3}
USER_DTYPES = (torch.bfloat16, torch.float32, torch.int32)
BUFFER_KINDS = ("input", "param", "state", "temp", "output", "workspace")

UNARY_FNS = ("relu", "silu", "gelu_tanh", "gelu", "exp", "neg", "sigmoid", "square", "identity")
BINARY_FNS = ("add", "sub", "mul", "max", "min")
LINEAR_ACTS = (None, "relu", "silu", "gelu_tanh", "gelu", "swiglu")

_buffer_ids = itertools.count()


class Buffer:
    """A named 2-D row-major tensor slot.  (reference: graph.py:23-47)"""

    __slots__ = ("name", "rows", "cols", "dtype", "kind", "id")

    def __init__(self, name: str, rows: int, cols: int, dtype: torch.dtype, kind: str):
        if dtype not in ELEM_BYTES:
            raise TypeError(f"{name}: unsupported dtype {dtype}")
        if dtype != torch.int32 and (cols * ELEM_BYTES[dtype]) % 16 != 0:
            raise ValueError(f"{name}: row stride of {cols} elements is not 16-byte aligned")
        assert kind in BUFFER_KINDS, kind
        self.name, self.rows, self.cols, self.dtype, self.kind = name, int(rows), int(cols), dtype, kind
        self.id = next(_buffer_ids)

    @property
    def full(self) -> "View":
        return View(self, 0, 0, self.rows, self.cols)

    @property
    def nbytes(self) -> int:
        return self.rows * self.cols * ELEM_BYTES[self.dtype]

    def __repr__(self):
        return f"{self.name}[{self.rows}x{self.cols}]"


class View:
    """An immutable ``rows x cols`` window of a buffer.  (reference: graph.py:50-74)"""

    __slots__ = ("buf", "row0", "col0", "rows", "cols")

    def __init__(self, buf: Buffer, row0: int, col0: int, rows: int, cols: int):
        inside = 0 <= row0 and 0 <= col0 and row0 + rows <= buf.rows and col0 + cols <= buf.cols
        if not inside:
            raise ValueError(f"view [{row0}:{row0 + rows}, {col0}:{col0 + cols}] out of bounds of {buf}")
        for k, v in zip(self.__slots__, (buf, int(row0), int(col0), int(rows), int(cols))):
            object.__setattr__(self, k, v)

    def __setattr__(self, *_):
        raise AttributeError("View is immutable")

    def cols_slice(self, start: int, size: int) -> "View":
        return View(self.buf, self.row0, self.col0 + start, self.rows, size)

    def rows_slice(self, start: int, size: int) -> "View":
        return View(self.buf, self.row0 + start, self.col0, size, self.cols)

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def rect(self):
        """(r0, r1, c0, c1) in buffer coordinates, half open."""
        return (self.row0, self.row0 + self.rows, self.col0, self.col0 + self.cols)

    def same(self, other: Optional["View"]) -> bool:
        return other is not None and self.buf is other.buf and self.rect == other.rect

    def __repr__(self):
        r0, r1, c0, c1 = self.rect
        return f"{self.buf.name}[{r0}:{r1}, {c0}:{c1}]"


# --------------------------------------------------------------------------------------------
# ops
# --------------------------------------------------------------------------------------------
# kind -> (view operands that are read, view operands that are written, scalar attributes).
# An operand listed in both columns is updated in place by the op.  Optional operands may be
# None.  The semantic definition of each kind is in the builder method's docstring below.
OP_TABLE = {
    "Linear":          (("x", "w", "bias", "residual", "norm_w"), ("out",), ("act", "rms_eps", "bn")),
    "LinearSplit":     (("x", "w", "norm_w"), ("ws",), ("splits", "rms_eps", "bn")),
    "SplitFinalize":   (("ws", "bias", "residual"), ("out", "ws"), ("act",)),
    "Unary":           (("x",), ("out",), ("fn",)),
    "Binary":          (("a", "b", "gate"), ("out",), ("fn", "b_group", "gate_group")),
    "SwiGLU":          (("gate", "up"), ("out",), ("act",)),
    "Modulate":        (("x", "scale", "shift"), ("out",), ("group",)),
    "Norm":            (("x", "weight", "bias", "scale", "shift"), ("out",), ("eps", "rms", "group")),
    "Rope":            (("x", "cos", "sin"), ("out",), ("heads", "head_dim", "seq")),
    "Attention":       (("q", "k", "v"), ("out",),
                        ("batch", "seq_q", "seq_k", "heads", "head_dim", "causal", "scale", "kv_heads")),
    "RopeAppend":      (("qkv", "cos", "sin", "pos"), ("q_out", "k_cache", "v_cache"),
                        ("heads", "kv_heads", "head_dim", "max_seq")),
    "DecodeAttention": (("q", "k_cache", "v_cache", "pos", "k_new", "v_new", "cos", "sin", "part", "count"),
                        ("out", "part", "count"),
                        ("batch", "heads", "kv_heads", "head_dim", "max_seq", "scale", "splits", "zero_inputs", "heads_per_inst",
                         "bulk", "window")),
    "Increment":       ((), ("pos",), ()),
    # the two ends of a decode step, inside the launch (no counterpart among the reference's ops: its
    # step does them in torch around the launch, examples/llama/llama1b.py:103-105)
    "Gather":          (("table", "ids"), ("out",), ()),
    "Argmax":          (("x", "part", "count"), ("ids", "part", "count"), ("chunks",)),
}


class Op:
    """One graph operation: a kind plus named view operands and scalar attributes.

    ``reads`` / ``writes`` list the views the op touches (reference: the ``reads``/``writes``
    properties of each dataclass in graph.py:96-481).  ``accumulate`` marks ops whose writes are
    commutative adds (split-K partials); ``independent`` marks ops whose instructions coordinate
    among themselves (split-KV with an in-op combine)."""

    def __init__(self, kind: str, **fields):
        reads, writes, attrs = OP_TABLE[kind]
        self.kind = kind
        self.layer = None
        known = set(reads) | set(writes) | set(attrs)
        for k in known:
            setattr(self, k, None)
        for k, v in fields.items():
            if k not in known:
                raise TypeError(f"{kind}: unknown field {k}")
            setattr(self, k, v)
        _CHECKS[kind](self)

    def clone(self, **changes) -> "Op":
        reads, writes, attrs = OP_TABLE[self.kind]
        f = {k: getattr(self, k) for k in dict.fromkeys(reads + writes + attrs)}
        f.update(changes)
        new = Op(self.kind, **f)
        new.layer = self.layer
        return new

    def view_fields(self):
        reads, writes, _ = OP_TABLE[self.kind]
        return [(k, getattr(self, k)) for k in dict.fromkeys(reads + writes) if getattr(self, k) is not None]

    @property
    def reads(self):
        vs = [getattr(self, k) for k in OP_TABLE[self.kind][0]]
        return [v for v in vs if v is not None]

    @property
    def writes(self):
        vs = [getattr(self, k) for k in OP_TABLE[self.kind][1]]
        out = [v for v in vs if v is not None]
        if self.kind == "DecodeAttention" and self.k_new is not None:
            out += [self.k_cache, self.v_cache]          # fused rope+append writes the row at pos
        return out

    @property
    def accumulate(self) -> bool:
        return self.kind == "LinearSplit"

    @property
    def independent(self) -> bool:
        return self.kind == "DecodeAttention" and (self.splits or 1) > 1

    def __repr__(self):
        return f"{self.kind}({', '.join(f'{k}={v}' for k, v in self.view_fields())})"


def _chk_linear(o):
    M, K = o.x.shape
    N, K2 = o.w.shape
    assert K == K2, f"linear: K mismatch {K} vs {K2}"
    assert o.act in LINEAR_ACTS, o.act
    if o.act == "swiglu":
        assert N % 128 == 0 and o.bias is None and o.residual is None, "swiglu linear: N % 128, no bias/res"
        N //= 2
    assert o.out.shape == (M, N), f"linear: out {o.out.shape} != {(M, N)}"
    if o.bias is not None:
        assert o.bias.shape == (1, N), f"linear: bias must be (1, {N})"
    if o.residual is not None:
        assert o.residual.shape == (M, N)
    if o.norm_w is not None:
        assert o.norm_w.shape == (1, K) and o.rms_eps is not None


def _chk_linear_split(o):
    assert o.x.cols == o.w.cols and o.ws.shape == (o.x.rows, o.w.rows)
    assert o.splits >= 1 and o.x.cols % o.splits == 0


def _chk_finalize(o):
    assert o.ws.shape == o.out.shape and o.act in LINEAR_ACTS and o.act != "swiglu"
    if o.bias is not None:
        assert o.bias.shape == (1, o.out.cols)
    if o.residual is not None:
        assert o.residual.shape == o.out.shape


def _chk_unary(o):
    assert o.fn in UNARY_FNS, o.fn
    assert o.x.shape == o.out.shape


def _chk_binary(o):
    assert o.fn in BINARY_FNS, o.fn
    assert o.a.shape == o.out.shape
    assert o.b.cols == o.a.cols
    assert o.a.rows == o.b.rows * o.b_group, "binary: b rows * b_group must equal a rows"
    if o.gate is not None:          # set by passes.fuse_gated_residual only: out = fn(a, b * gate[r // gate_group])
        assert o.b_group == 1 and o.gate.shape == (o.a.rows // o.gate_group, o.a.cols)


def _chk_swiglu(o):
    assert o.gate.shape == o.up.shape == o.out.shape
    assert o.act in UNARY_FNS


def _chk_modulate(o):
    assert o.x.shape == o.out.shape
    assert o.scale.shape == o.shift.shape == (o.x.rows // o.group, o.x.cols)


def _chk_norm(o):
    assert o.x.shape == o.out.shape
    for p in (o.weight, o.bias):
        if p is not None:
            assert p.shape == (1, o.x.cols)
    if o.scale is not None:         # set by passes.fuse_norm_modulate only: out = norm(x) * (1 + scale[r // group]) + shift[r // group]
        assert o.scale.shape == o.shift.shape == (o.x.rows // o.group, o.x.cols)


def _chk_rope(o):
    assert o.x.shape == o.out.shape
    assert o.x.cols == o.heads * o.head_dim
    assert o.cos.shape == o.sin.shape == (o.seq, o.head_dim)
    assert o.x.rows % o.seq == 0 and o.head_dim % 16 == 0


def _chk_attention(o):
    D, H = o.head_dim, o.heads
    assert H % o.kv_heads == 0, "attention: heads must be a multiple of kv_heads"
    assert D in (64, 128), "attention: head_dim must be 64 or 128"
    assert o.q.shape == (o.batch * o.seq_q, H * D)
    assert o.k.shape == o.v.shape == (o.batch * o.seq_k, o.kv_heads * D)
    assert o.out.shape == o.q.shape
    if o.causal:
        assert o.seq_q == o.seq_k, "causal attention requires seq_q == seq_k"


def _chk_pos(pos, batch):
    """One position for the whole batch, (1, 1), or one per sequence, (batch, 1): the reference's decode ops know only the
    first (megacute README.md:225-227 lists per-sequence positions as a limitation)."""
    assert pos.shape in ((1, 1), (batch, 1)) and pos.buf.dtype == torch.int32, "pos is (1, 1) or (batch, 1) int32"


def _chk_rope_append(o):
    B, D = o.qkv.rows, o.head_dim
    assert o.qkv.cols == (o.heads + 2 * o.kv_heads) * D
    assert o.q_out.shape == (B, o.heads * D)
    assert o.k_cache.shape == o.v_cache.shape == (B * o.max_seq, o.kv_heads * D)
    assert o.cos.shape == o.sin.shape == (o.max_seq, D) and D % 16 == 0
    _chk_pos(o.pos, B)


def _chk_decode_attention(o):
    D = o.head_dim
    o.splits = o.splits or 1
    o.heads_per_inst = o.heads_per_inst or 1
    o.bulk = bool(o.bulk)
    # several kv heads per instruction: unsplit (one head after the other), or the many-sequence form (all of them at once)
    assert o.kv_heads % o.heads_per_inst == 0 and (o.heads_per_inst == 1 or o.splits == 1 or o.bulk)
    assert not o.bulk or (o.heads_per_inst == o.kv_heads and D == 64)
    assert o.heads % o.kv_heads == 0 and o.heads // o.kv_heads <= 8, "decode attention: GQA group <= 8"
    assert D in (64, 128) and o.max_seq % 128 == 0
    assert o.q.shape == o.out.shape == (o.batch, o.heads * D)
    assert o.k_cache.shape == o.v_cache.shape == (o.batch * o.max_seq, o.kv_heads * D)
    _chk_pos(o.pos, o.batch)
    o.window = int(o.window or 0)
    assert o.window >= 0, "decode attention: window is a number of tokens (0 or None: the whole context)"
    assert not (o.bulk and o.window), "the many-sequence form of decode attention has no sliding window"


def _chk_increment(o):
    assert o.pos.cols == 1 and o.pos.buf.dtype == torch.int32


def _chk_gather(o):
    assert o.ids.cols == 1 and o.ids.buf.dtype == torch.int32, "gather: ids is a (rows, 1) int32 column"
    assert o.out.shape == (o.ids.rows, o.table.cols) and o.table.cols % 8 == 0
    assert o.table.buf.dtype == torch.bfloat16, "gather: bf16 table"


def _chk_argmax(o):
    assert o.ids.shape == (o.x.rows, 1) and o.ids.buf.dtype == torch.int32, "argmax: ids is a (rows, 1) int32 column"
    assert o.x.cols % 8 == 0
    o.chunks = o.chunks or 1


_CHECKS = {"Linear": _chk_linear, "LinearSplit": _chk_linear_split, "SplitFinalize": _chk_finalize,
           "Unary": _chk_unary, "Binary": _chk_binary, "SwiGLU": _chk_swiglu, "Modulate": _chk_modulate,
           "Norm": _chk_norm, "Rope": _chk_rope, "Attention": _chk_attention, "RopeAppend": _chk_rope_append,
           "DecodeAttention": _chk_decode_attention, "Increment": _chk_increment, "Gather": _chk_gather,
           "Argmax": _chk_argmax}


def swiglu_weight(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Interleave (F, K) gate and up projections into the (2F, K) weight of ``linear(act="swiglu")``:
    rows [128j, 128j+64) are gate rows [64j, 64j+64) and rows [128j+64, 128j+128) the matching up
    rows.  (reference: graph.py:367-370)"""
    F, K = gate.shape
    assert up.shape == (F, K) and F % 64 == 0
    out = gate.new_empty(F // 64, 2, 64, K)
    out[:, 0] = gate.reshape(F // 64, 64, K)
    out[:, 1] = up.reshape(F // 64, 64, K)
    return out.reshape(2 * F, K)


# --------------------------------------------------------------------------------------------
# builder
# --------------------------------------------------------------------------------------------

class Graph:
    """A straight-line program of ops over buffers.  (reference: graph.py:488-625)

        g = Graph()
        x = g.input("x", (4096, 2048))
        w = g.param("w", (8192, 2048))
        g.output(g.linear(x, w, act="gelu_tanh"))
    """

    def __init__(self, dtype: torch.dtype = torch.bfloat16):
        self.dtype = dtype
        self.layer = None            # builders of repeated blocks tag ops with the block index
        self.buffers: list[Buffer] = []
        self.ops: list[Op] = []
        self.inputs: list[Buffer] = []
        self.params: list[Buffer] = []
        self.states: list[Buffer] = []
        self.outputs: list[View] = []

    def derive(self) -> "Graph":
        """A shallow copy whose op / buffer / output lists can be rewritten by a pass."""
        g = Graph(self.dtype)
        g.buffers, g.ops, g.outputs = list(self.buffers), list(self.ops), list(self.outputs)
        g.inputs, g.params, g.states = list(self.inputs), list(self.params), list(self.states)
        return g

    # ---- buffers
    def _new(self, name, shape, kind, dtype=None) -> View:
        rows, cols = shape
        if (dtype or self.dtype) not in USER_DTYPES:
            raise TypeError(f"{name}: unsupported dtype {dtype or self.dtype}")
        b = Buffer(name, rows, cols, dtype or self.dtype, kind)
        self.buffers.append(b)
        return b.full

    def input(self, name, shape, dtype=None) -> View:
        v = self._new(name, shape, "input", dtype)
        self.inputs.append(v.buf)
        return v

    def param(self, name, shape, dtype=None) -> View:
        v = self._new(name, shape, "param", dtype)
        self.params.append(v.buf)
        return v

    def state(self, name, shape, dtype=None) -> View:
        """A caller-owned tensor the launch reads and updates in place (KV cache, position)."""
        v = self._new(name, shape, "state", dtype)
        self.states.append(v.buf)
        return v

    def temp(self, shape, name=None, dtype=None) -> View:
        return self._new(name or f"t{len(self.buffers)}", shape, "temp", dtype)

    def workspace(self, shape, dtype) -> View:
        return self._new(f"ws{len(self.buffers)}", shape, "workspace", dtype)

    def output(self, *views: View):
        for v in views:
            if v.buf.kind == "temp":
                v.buf.kind = "output"
            self.outputs.append(v)

    def _emit(self, kind, **fields) -> Op:
        op = Op(kind, **fields)
        for w in op.writes:
            if w.buf.kind in ("input", "param"):
                raise ValueError(f"{kind} writes read-only buffer {w.buf}")
        op.layer = self.layer
        self.ops.append(op)
        return op

    # ---- ops
    def linear(self, x, w, bias=None, act=None, residual=None, out=None) -> View:
        """``act(x @ w.T + bias) + residual``; x (M,K), w (N,K), bias (1,N).  ``act="swiglu"``: w is
        interleaved by ``swiglu_weight`` and the output is (M, N/2) = silu(gate) * up."""
        out = out or self.temp((x.rows, w.rows // 2 if act == "swiglu" else w.rows))
        self._emit("Linear", x=x, w=w, out=out, bias=bias, act=act, residual=residual)
        return out

    def unary(self, x, fn, out=None) -> View:
        out = out or self.temp(x.shape)
        self._emit("Unary", x=x, out=out, fn=fn)
        return out

    def binary(self, a, b, fn, out=None, b_group=None) -> View:
        """``a <fn> b[r // b_group]``: b is broadcast over runs of ``b_group`` rows of a."""
        out = out or self.temp(a.shape)
        self._emit("Binary", a=a, b=b, out=out, fn=fn, b_group=b_group or a.rows // b.rows)
        return out

    def add(self, a, b, out=None):
        return self.binary(a, b, "add", out)

    def mul(self, a, b, out=None):
        return self.binary(a, b, "mul", out)

    def swiglu(self, gate, up, act="silu", out=None) -> View:
        out = out or self.temp(gate.shape)
        self._emit("SwiGLU", gate=gate, up=up, out=out, act=act)
        return out

    def modulate(self, x, scale, shift, group, out=None) -> View:
        """adaLN: ``x * (1 + scale[r // group]) + shift[r // group]``."""
        out = out or self.temp(x.shape)
        self._emit("Modulate", x=x, scale=scale, shift=shift, out=out, group=group)
        return out

    def rms_norm(self, x, weight=None, eps=1e-6, out=None) -> View:
        out = out or self.temp(x.shape)
        self._emit("Norm", x=x, out=out, weight=weight, bias=None, eps=eps, rms=True)
        return out

    def layer_norm(self, x, weight=None, bias=None, eps=1e-5, out=None) -> View:
        out = out or self.temp(x.shape)
        self._emit("Norm", x=x, out=out, weight=weight, bias=bias, eps=eps, rms=False)
        return out

    def rope(self, x, cos, sin, heads, head_dim, seq, out=None) -> View:
        """Rotate-half RoPE on ``heads`` heads stored side by side; row r is token ``r % seq``."""
        out = out or self.temp(x.shape)
        self._emit("Rope", x=x, cos=cos, sin=sin, out=out, heads=heads, head_dim=head_dim, seq=seq)
        return out

    def attention(self, q, k, v, *, batch, heads, head_dim, causal=False, scale=None, kv_heads=None,
                  out=None) -> View:
        out = out or self.temp(q.shape)
        self._emit("Attention", q=q, k=k, v=v, out=out, batch=batch, seq_q=q.rows // batch, seq_k=k.rows // batch,
                   heads=heads, head_dim=head_dim, causal=bool(causal),
                   scale=float(scale) if scale is not None else head_dim ** -0.5, kv_heads=kv_heads or heads)
        return out

    def rope_append(self, qkv, cos, sin, pos, k_cache, v_cache, *, heads, kv_heads, head_dim, max_seq,
                    out=None) -> View:
        """Decode: rotate q and k of one new token per sequence at position ``pos[0, 0]`` (or ``pos[b, 0]``
        when pos has one row per sequence); write ``k_cache[b*max_seq + pos] = rope(k)`` and
        ``v_cache[b*max_seq + pos] = v``; return rotated q."""
        out = out or self.temp((qkv.rows, heads * head_dim))
        self._emit("RopeAppend", qkv=qkv, cos=cos, sin=sin, pos=pos, q_out=out, k_cache=k_cache, v_cache=v_cache,
                   heads=heads, kv_heads=kv_heads, head_dim=head_dim, max_seq=max_seq)
        return out

    def decode_attention(self, q, k_cache, v_cache, pos, *, heads, kv_heads, head_dim, max_seq, scale=None,
                         out=None, window=None) -> View:
        """Decode: one query token per sequence against cache rows [0, pos] of its sequence, GQA.

        Beyond the reference (its README.md:225-228 names both as limitations): ``pos`` may be a
        (batch, 1) column, one position per sequence (a ragged batch; rope_append and increment take
        the same), and ``window`` = w restricts a sequence to its last w tokens, rows
        [max(0, pos + 1 - w), pos] (sliding-window attention)."""
        out = out or self.temp(q.shape)
        self._emit("DecodeAttention", q=q, k_cache=k_cache, v_cache=v_cache, pos=pos, out=out, batch=q.rows,
                   heads=heads, kv_heads=kv_heads, head_dim=head_dim, max_seq=max_seq,
                   scale=float(scale) if scale is not None else head_dim ** -0.5, splits=1, window=int(window or 0))
        return out

    def increment(self, pos):
        """``pos += 1`` (every row of it) on device after every reader of pos in the launch."""
        self._emit("Increment", pos=pos)

    def gather(self, table, ids, out=None) -> View:
        """``out[r] = table[ids[r, 0]]``: the embedding lookup of a decode step as the launch's first
        instructions.  ``ids`` is a (rows, 1) int32 view.  (The reference's step gathers in torch before
        the launch, examples/llama/llama1b.py:103-104; this op has no counterpart in its Graph.)"""
        out = out or self.temp((ids.rows, table.cols))
        self._emit("Gather", table=table, ids=ids, out=out)
        return out

    def argmax(self, x, ids) -> View:
        """``ids[r, 0] = argmax(x[r])`` (ties: lowest index; NaN never wins): greedy sampling as the
        launch's last instructions, into a (rows, 1) int32 view -- with ``gather`` reading the same view,
        a decode step feeds itself.  (The reference's step calls torch's argmax after the launch,
        examples/llama/llama1b.py:105.)"""
        self._emit("Argmax", x=x, ids=ids)
        return ids

    def __repr__(self):
        head = f"Graph({len(self.buffers)} buffers, {len(self.ops)} ops)"
        return "\n".join([head] + [f"  {op.kind}: {op.reads} -> {op.writes}" for op in self.ops])
