"""Graph op -> device descriptor (``mk_op_desc``).

One descriptor per op of the rewritten graph.  The reference has no such table: its per-op
parameters are Python constants traced into the JIT kernel by the node classes
(``megacute/ops/*.py`` ``__init__`` / ``host``).  Here the kernel is compiled once, ahead of time,
and reads shapes, strides, flags and operand addresses from this table at run time.

``fill(desc, op, addr)`` writes the fields; ``addr(view)`` returns the device byte address of the
view's first element.  Field meaning per kind (the kernel side repeats it next to the reader):

  GEMV         ptr x, w, out, bias, residual, norm gain; i M, N_out, K, act, x dtype, out dtype,
               residual dtype; f eps; flags 1 = swiglu, 2 = rms-normalise x, 4 = tensor-core streaming path
  GEMM         ptr x, w, out, bias, residual; i M, N (weight rows), K, act, splits, out dtype,
               accumulate, residual dtype, swiglu, x dtype (bf16 or fp16), weight rows per tile (128 / 256)  (ptr 10, 11: set by the C
               library when it binds the op to its tcgen05 body: packed weight tiles, tensor maps)
  FINALIZE     ptr ws, out, bias, residual; i R, C, act, out dtype, residual dtype, rows per instruction
  ELTWISE      ptr a, b, c, out; i R, C, mode, fn, group, head_dim, dtypes of a, b, c, out
               (mode EW_GATED: out = fn(a, b * c[r // group]), a gated residual)
  NORM         ptr x, out, weight, bias, scale, shift (adaLN modulation fused in, or none); i R, C, rms, rows per
               instruction, x dtype, out dtype, rows per scale / shift row, their dtypes; f eps
  ATTENTION    ptr q, k, v, out; i batch, seq_q, seq_k, heads, kv_heads, head_dim, causal, out dtype,
               dtype of q / k / v (one for all three: bf16 or fp16); f scale
  ROPE_APPEND  ptr qkv, cos, sin, pos, q_out, k_cache, v_cache; i B, H, KVH, D, max_seq, qkv dtype,
               pos stride (ints between the positions of consecutive sequences; 0: one position for all)
  DECODE_ATTN  ptr q, k_cache, v_cache, pos, out, k_new, v_new, cos, sin, part, count;
               i B, H, KVH, D, max_seq, splits, fused, q dtype, out dtype, zero inputs, kv heads per
               instruction, many-sequence form, pos stride (0: one position for all), window (0: whole context);
               f scale
  INCREMENT    ptr pos; i rows of pos, pos stride
  GATHER       ptr table, ids, out; i rows, cols, table rows, out dtype
  ARGMAX       ptr x, ids, part, count; i rows, cols, chunks, columns per chunk, x dtype
"""

from __future__ import annotations

import torch

from . import config as C
from .graph import DTYPE_CODE, ELEM_BYTES, Op, View
from .schedule import argmax_chunk_cols, finalize_rows, is_gemv, norm_rows

BF16 = torch.bfloat16
F16 = torch.float16
F32 = torch.float32


def _aligned(v: View, what: str):
    if (v.col0 * ELEM_BYTES[v.buf.dtype]) % 16:
        raise ValueError(f"{v}: column offset is not 16-byte aligned ({what})")


def _want(v, dtypes, what):
    if v is not None and v.buf.dtype not in dtypes:
        raise TypeError(f"{what}: operand {v} has dtype {v.buf.dtype}, supported: {dtypes}")


def validate(op: Op):
    """Alignment and dtype rules of the kernel, checked once at compile time."""
    for name, v in op.view_fields():
        if v.buf.dtype != torch.int32:
            _aligned(v, f"{op.kind}.{name}")
    k = op.kind
    if k in ("Linear", "LinearSplit"):
        _want(op.w, (BF16,), k)
        if op.x.cols % 8:
            raise ValueError(f"{k}: K={op.x.cols} must be a multiple of 8")
        if not is_gemv(op):
            _want(op.x, (BF16, F16), k)
        _want(getattr(op, "bias", None), (BF16,), k)
    if k in ("Unary", "Binary", "SwiGLU", "Modulate", "Rope", "Norm"):
        for name, v in op.view_fields():
            if k == "Norm" and name in ("weight", "bias"):
                _want(v, (BF16,), f"{k}.{name}")
            else:
                _want(v, (BF16, F16, F32), f"{k}.{name}")
        if op.out.cols % 8:
            raise ValueError(f"{k}: column count {op.out.cols} must be a multiple of 8")
    if k == "Attention":
        for name, v in op.view_fields():
            _want(v, (BF16, F16), f"{k}.{name}")


def _pos_stride(pos: View) -> int:
    """int32 elements between the positions of consecutive sequences: 0 when the batch shares one position."""
    return 0 if pos.rows == 1 else pos.buf.cols


def gemv_units(op: Op) -> bool:
    """Streaming linear whose K is a multiple of 16: the kernel's tensor-core path (GEMV_F_UNITS).
    Other K fall back to the general CUDA-core path."""
    return op.x.cols % 16 == 0


def fill(d, op: Op, addr) -> None:
    """Write op's descriptor into ``d`` (an ``_lib.OpDesc``)."""
    ptrs: list = []
    ints: list = []
    d.flags = 0
    dt = lambda v: DTYPE_CODE[v.buf.dtype] if v is not None else 0
    k = op.kind
    if k == "Linear" and is_gemv(op):
        d.kind = C.OP_GEMV
        ptrs = [op.x, op.w, op.out, op.bias, op.residual, op.norm_w]
        ints = [op.x.rows, op.out.cols, op.x.cols, C.ACT_CODE[op.act], dt(op.x), dt(op.out), dt(op.residual)]
        d.f[0] = float(op.rms_eps or 0.0)
        d.flags = (1 if op.act == "swiglu" else 0) | (2 if op.rms_eps is not None else 0) | (4 if gemv_units(op) else 0)
    elif k in ("Linear", "LinearSplit"):
        d.kind = C.OP_GEMM
        split = k == "LinearSplit"
        out = op.ws if split else op.out
        ptrs = [op.x, op.w, out, None if split else op.bias, None if split else op.residual]
        act = None if split else op.act
        ints = [op.x.rows, op.w.rows, op.x.cols, C.ACT_CODE[act], op.splits if split else 1, dt(out), int(split),
                0 if split else dt(op.residual), int(act == "swiglu"), dt(op.x), int(op.bn or C.GEMM_BN)]
    elif k == "SplitFinalize":
        d.kind = C.OP_FINALIZE
        ptrs = [op.ws, op.out, op.bias, op.residual]
        ints = [op.out.rows, op.out.cols, C.ACT_CODE[op.act], dt(op.out), dt(op.residual), finalize_rows(op.out.rows, op.out.cols)]
    elif k in ("Unary", "Binary", "SwiGLU", "Modulate", "Rope"):
        d.kind = C.OP_ELTWISE
        R, Cc = op.out.shape
        if k == "Unary":
            ptrs, ints = [op.x, None, None, op.out], [R, Cc, C.EW_UNARY, C.ACT_CODE[op.fn], 1, 0]
        elif k == "Binary" and op.gate is not None:         # out = fn(a, b * gate[r // gate_group])
            ptrs, ints = [op.a, op.b, op.gate, op.out], [R, Cc, C.EW_GATED, C.BINARY_CODE[op.fn], op.gate_group, 0]
        elif k == "Binary":
            ptrs, ints = [op.a, op.b, None, op.out], [R, Cc, C.EW_BINARY, C.BINARY_CODE[op.fn], op.b_group, 0]
        elif k == "SwiGLU":
            ptrs, ints = [op.gate, op.up, None, op.out], [R, Cc, C.EW_SWIGLU, C.ACT_CODE[op.act], 1, 0]
        elif k == "Modulate":
            ptrs, ints = [op.x, op.scale, op.shift, op.out], [R, Cc, C.EW_MODULATE, 0, op.group, 0]
        else:
            ptrs, ints = [op.x, op.cos, op.sin, op.out], [R, Cc, C.EW_ROPE, 0, op.seq, op.head_dim]
        ints += [dt(v) for v in ptrs]
    elif k == "Norm":
        d.kind = C.OP_NORM
        ptrs = [op.x, op.out, op.weight, op.bias, op.scale, op.shift]
        ints = [op.x.rows, op.x.cols, int(bool(op.rms)), norm_rows(op.x.rows), dt(op.x), dt(op.out),
                int(op.group or 1), dt(op.scale), dt(op.shift)]
        d.f[0] = float(op.eps)
    elif k == "Attention":
        d.kind = C.OP_ATTENTION
        ptrs = [op.q, op.k, op.v, op.out]
        ints = [op.batch, op.seq_q, op.seq_k, op.heads, op.kv_heads, op.head_dim, int(op.causal), dt(op.out), dt(op.q)]
        if not dt(op.q) == dt(op.k) == dt(op.v):
            raise TypeError(f"Attention: q, k and v must share one dtype, got {op.q.buf.dtype}, {op.k.buf.dtype}, {op.v.buf.dtype}")
        d.f[0] = float(op.scale)
    elif k == "RopeAppend":
        d.kind = C.OP_ROPE_APPEND
        ptrs = [op.qkv, op.cos, op.sin, op.pos, op.q_out, op.k_cache, op.v_cache]
        ints = [op.qkv.rows, op.heads, op.kv_heads, op.head_dim, op.max_seq, dt(op.qkv), _pos_stride(op.pos)]
    elif k == "DecodeAttention":
        d.kind = C.OP_DECODE_ATTN
        ptrs = [op.q, op.k_cache, op.v_cache, op.pos, op.out, op.k_new, op.v_new, op.cos, op.sin, op.part, op.count]
        ints = [op.batch, op.heads, op.kv_heads, op.head_dim, op.max_seq, op.splits, int(op.k_new is not None),
                dt(op.q), dt(op.out), int(bool(op.zero_inputs)), int(op.heads_per_inst or 1), int(bool(op.bulk)),
                _pos_stride(op.pos), int(op.window or 0)]
        assert not op.bulk or (op.heads_per_inst == op.kv_heads and op.head_dim == 64 and op.kv_heads <= C.COMPUTE_WARPS)
        assert not op.zero_inputs or dt(op.q) == 1
        assert op.k_new is None or dt(op.k_new) == dt(op.v_new) == dt(op.q)
        assert op.splits <= C.MAX_KV_SPLITS
        d.f[0] = float(op.scale)
    elif k == "Increment":
        d.kind = C.OP_INCREMENT
        ptrs = [op.pos]
        ints = [op.pos.rows, _pos_stride(op.pos)]
    elif k == "Gather":
        d.kind = C.OP_GATHER
        ptrs = [op.table, op.ids, op.out]
        ints = [op.out.rows, op.out.cols, op.table.rows, dt(op.out)]
    elif k == "Argmax":
        d.kind = C.OP_ARGMAX
        ptrs = [op.x, op.ids, op.part, op.count]
        ints = [op.x.rows, op.x.cols, op.chunks, argmax_chunk_cols(op.x.cols, op.chunks), dt(op.x)]
    else:
        raise NotImplementedError(k)
    for n, v in enumerate(ints):
        d.i[n] = int(v)
    for n, v in enumerate(ptrs):
        d.ptr[n] = addr(v) if v is not None else 0
        d.ld[n] = v.buf.cols if v is not None else 0
