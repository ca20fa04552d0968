"""Runtime: compile a Graph into tables for the persistent kernel and run it.

    prog = megacute_b200.compile(g)        # passes + schedule + table upload (no JIT)
    outs = prog(x=x, w=w, ...)             # one kernel launch per call

Mirrors the reference's ``Program`` (``megacute/runtime.py:227-400``): same constructor keywords,
same binding rules and exceptions, same ownership (caller owns inputs / params / states; the
program owns temps, outputs, workspaces, counters and the trace buffer; returned outputs alias
program buffers and are overwritten by the next call).  What differs is below the call: the
reference JIT-compiles a kernel per graph; here a prebuilt sm_100a kernel is driven through the C
ABI of ``include/megacute_b200.h`` with an op-descriptor table that is rewritten only when a bound
tensor moves.
"""

from __future__ import annotations

import ctypes
import os
import time

import numpy as np
import torch

from . import _lib, config as C, encode
from .graph import ELEM_BYTES, Graph
from .layers import merge_layers
from .passes import run_all
from .schedule import schedule


class Program:
    """A compiled graph bound to one GPU.

    Tile-GEMM weights (linears with more than 8 activation rows) are read from packed tile copies the
    library makes when a weight tensor is first bound.  The copies are snapshots: a parameter changed
    in place through torch is noticed at the next call (its version counter moved) and packed again;
    a change torch cannot see (a raw pointer write, another process) needs ``refresh_weights()``.
    Linears with at most 8 rows stream the caller's tensors directly.
    """

    def __init__(self, g: Graph, *, sm_count: int | None = None, verbose: bool = False, debug: bool = False,
                 trace: bool = False, device: int | None = None):
        t0 = time.time()
        self.debug = debug or os.environ.get("MEGACUTE_DEBUG") == "1"   # check the device status after every launch
        self.trace = trace
        self.verbose = verbose
        self.device = device
        if sm_count is None:
            caps = _lib.Caps()
            dev = device if device is not None else torch.cuda.current_device()
            _lib.check(_lib.load().mk_query(dev, ctypes.byref(caps)), "mk_query")
            sm_count = caps.sm_count
        self.sm_count = int(sm_count)
        self.source = g
        self.g = run_all(g, self.sm_count)
        for op in self.g.ops:
            encode.validate(op)
        self.sched = schedule(self.g, self.sm_count)
        if self.debug or os.environ.get("MEGACUTE_B200_VERIFY") == "1":
            # exact host checks of the tables (see verify.py); the happens-before closure keeps
            # n^2 / 8 bytes, so very long instruction streams (full prefill) get the table check only
            from . import verify
            verify.check_tables(self.g, self.sched)
            if self.sched.n <= 40000:
                verify.check_hazards(self.sched, self.g)
        groups = [[k] for k in range(len(self.g.ops))] if os.environ.get("MEGACUTE_NO_MERGE") == "1" \
            else merge_layers(self.g)
        self.node_of = [None] * len(self.g.ops)
        for n, ks in enumerate(groups):
            for layer, k in enumerate(ks):
                self.node_of[k] = (n, layer)
        self.nodes = [[self.g.ops[k] for k in ks] for ks in groups]
        self.epoch = 0
        self._handle = None
        self._bufs: dict[int, torch.Tensor] = {}
        self._desc = (_lib.OpDesc * max(1, len(self.g.ops)))()
        self._desc_key = None
        self._ops_of_buf: dict[int, list[int]] = {}        # buffer id -> ops with an operand in it
        for k, op in enumerate(self.g.ops):
            for _, v in op.view_fields():
                self._ops_of_buf.setdefault(v.buf.id, []).append(k)
        self.trace_cap = 0
        self.schedule_seconds = time.time() - t0
        self.compile_seconds = self.schedule_seconds

    # ---- compile: upload the tables
    def compile(self):
        t0 = time.time()
        lib = _lib.load()
        if self.device is None:
            self.device = torch.cuda.current_device()
        insts, waits, arrives = self.sched.encode()
        n = self.sched.n
        if n == 0:
            raise ValueError("graph has no ops")
        self.trace_cap = -(-n // self.sm_count) if self.trace else 0
        self._tables = (insts.contiguous(), waits.contiguous(), arrives.contiguous())
        h = ctypes.c_void_p()
        _lib.check(lib.mk_program_create(self.device, insts.data_ptr(), n, waits.data_ptr(), len(self.sched.wait_cnt),
                                         arrives.data_ptr(), len(self.sched.arr_cnt), self.sched.num_counters,
                                         len(self.g.ops), self.sm_count, self.trace_cap, ctypes.byref(h)),
                   "mk_program_create")
        self._handle = h
        self.compile_seconds = self.schedule_seconds + time.time() - t0
        if self.verbose:
            print(f"[megacute_b200] {len(self.nodes)} nodes, {n} insts, {self.sched.num_counters} counters, "
                  f"compiled in {self.compile_seconds:.2f}s")
        return self

    def __del__(self):
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            try:
                _lib.load().mk_program_destroy(h)
            except Exception:
                pass

    # ---- buffers
    def buffer(self, buf) -> torch.Tensor:
        return self._bufs[buf.id]

    def _bind(self, bindings: dict):
        dev = torch.device("cuda", self.device)
        for b in self.g.inputs + self.g.params + self.g.states:
            if b.name not in bindings:
                raise KeyError(f"missing tensor for {b.kind} '{b.name}'")
            t = bindings[b.name]
            if (tuple(t.shape) != (b.rows, b.cols) or t.dtype != b.dtype or not t.is_contiguous() or not t.is_cuda
                    or t.device != dev):
                raise ValueError(f"'{b.name}': expected contiguous {dev} {b.dtype} {(b.rows, b.cols)}, "
                                 f"got {t.device} {t.dtype} {tuple(t.shape)}")
            self._bufs[b.id] = t
        for b in self.g.buffers:
            if b.id in self._bufs:
                continue
            if b.kind in ("temp", "output"):
                self._bufs[b.id] = torch.empty(b.rows, b.cols, dtype=b.dtype, device=dev)
            elif b.kind == "workspace":      # zero on entry to every launch: the kernel re-zeroes what it uses
                self._bufs[b.id] = torch.zeros(b.rows, b.cols, dtype=b.dtype, device=dev)

    def _addr(self, v) -> int:
        t = self._bufs[v.buf.id]
        return t.data_ptr() + (v.row0 * v.buf.cols + v.col0) * ELEM_BYTES[v.buf.dtype]

    @staticmethod
    def _version(t) -> int:
        try:
            return t._version
        except RuntimeError:              # inference tensors keep no version counter
            return 0

    def _descriptors(self, stream):
        """Bring the device's op descriptors up to date with the bound tensors.  Only the descriptors
        of ops that touch a tensor whose address changed are re-encoded (a caller that passes a fresh
        input tensor every call re-encodes the ops that read it, not the whole graph).  A parameter
        changed in place since the last call (torch's version counter) makes the library drop its
        packed tile copies of the weights, so tile GEMMs never run on a stale snapshot."""
        named = self.g.inputs + self.g.params + self.g.states
        ptrs = {b.id: self._bufs[b.id].data_ptr() for b in named}
        vers = tuple(self._version(self._bufs[b.id]) for b in self.g.params)
        old = self._desc_key
        if old is not None and old[0] == ptrs and old[1] == vers:
            return
        if old is not None and old[1] != vers and self.packed_weight_bytes:
            _lib.check(_lib.load().mk_program_refresh_weights(self._handle, stream), "mk_program_refresh_weights")
        if old is None:
            todo = range(len(self.g.ops))
        else:
            moved = {i for i, a in ptrs.items() if old[0].get(i) != a}
            todo = sorted({k for i in moved for k in self._ops_of_buf.get(i, ())})
        for k in todo:
            encode.fill(self._desc[k], self.g.ops[k], self._addr)
        _lib.check(_lib.load().mk_program_set_ops(self._handle, ctypes.addressof(self._desc), len(self.g.ops), stream),
                   "mk_program_set_ops")
        self._desc_key = (ptrs, vers)

    # ---- run
    def __call__(self, **bindings):
        if self._handle is None:
            self.compile()
        self._bind(bindings)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        self._descriptors(stream)
        lib = _lib.load()
        if self.trace:
            _lib.check(lib.mk_program_clear_trace(self._handle, stream))
        _lib.check(lib.mk_launch(self._handle, stream), "mk_launch")
        self.epoch = lib.mk_program_epoch(self._handle)
        if self.debug:
            self.check()
        outs = [self._bufs[v.buf.id].as_strided(v.shape, (v.buf.cols, 1), v.row0 * v.buf.cols + v.col0)
                for v in self.g.outputs]
        return outs[0] if len(outs) == 1 else tuple(outs)

    # ---- status, recovery, introspection
    @property
    def tcgen05_ops(self) -> int:
        """Tile-GEMM ops the library bound to its tcgen05 / bulk-tensor-copy body at the last launch
        (the rest run the mma.sync body)."""
        return int(_lib.load().mk_program_tcgen05_ops(self._handle)) if self._handle is not None else 0

    @property
    def tcgen05_attention_ops(self) -> int:
        """Prefill attention ops bound to the tcgen05 body at the last launch (head_dim 64)."""
        return int(_lib.load().mk_program_tcgen05_attention_ops(self._handle)) if self._handle is not None else 0

    @property
    def packed_weight_bytes(self) -> int:
        """Device memory held for tile-image copies of tile-GEMM weights (snapshots taken when a weight
        tensor is first bound; `refresh_weights()` after changing weights in place)."""
        return int(_lib.load().mk_program_packed_bytes(self._handle)) if self._handle is not None else 0

    def refresh_weights(self):
        """Call after changing bound weights in place: the packed tile copies of tile-GEMM weights are
        dropped and made again at the next launch."""
        if self._handle is None:
            return
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(_lib.load().mk_program_refresh_weights(self._handle, stream), "mk_program_refresh_weights")
        self._desc_key = None

    def check(self):
        """Synchronise and raise if the kernel reported an error (bounded wait gave up, bad table)."""
        st = (ctypes.c_int32 * _lib.ST_WORDS)()
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        rc = _lib.load().mk_program_status(self._handle, stream, st)
        if rc == -4:
            code, cta, warp, seq, where, a, b, c = list(st)[:8]
            names = {1: "dependency counter wait timed out", 2: "shared-memory barrier wait timed out",
                     3: "bad instruction", 4: "self-check: a shared-memory barrier is in a state its protocol rules out"}
            exc = _lib.MegakernelTimeout if code in (1, 2) else _lib.MegakernelError
            raise exc(f"megakernel: {names.get(code, code)} (cta {cta}, warp {warp}, inst {seq}, where {where}, "
                      f"a={a}, b={b}, c={c}); call prog.reset() before reusing the program")
        _lib.check(rc, "mk_program_status")

    def reset(self):
        """Zero the dependency counters, status and epoch (after an error or to resume from saved states)."""
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(_lib.load().mk_program_reset(self._handle, stream))
        for b in self.g.buffers:
            if b.kind == "workspace" and b.id in self._bufs:
                self._bufs[b.id].zero_()
        self.epoch = 0

    def set_timeout(self, seconds: float):
        _lib.check(_lib.load().mk_program_set_timeout(self._handle, int(seconds * 1e9)))

    def counters(self) -> np.ndarray:
        torch.cuda.synchronize(self.device)
        out = np.zeros(max(1, self.sched.num_counters), np.int32)
        _lib.check(_lib.load().mk_program_read_counters(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                                        self.sched.num_counters))
        return out[:self.sched.num_counters]

    def timeline(self):
        """Trace of the most recent launch (requires trace=True)."""
        from .trace import Timeline
        if not self.trace:
            raise RuntimeError("compile with trace=True to record a timeline")
        torch.cuda.synchronize(self.device)
        buf = np.zeros((self.sm_count, 3, self.trace_cap, 4), np.int64)
        _lib.check(_lib.load().mk_program_read_trace(self._handle, buf.ctypes.data, buf.size))
        return Timeline(self, buf)


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Greedy sampling: row-wise argmax of a (rows, cols) bf16 or fp32 CUDA tensor (ties to the lowest
    index), one launch on the current stream.  Stands where the reference's decode loop calls
    ``logits.argmax(-1)`` (``examples/llama/llama1b.py:105``)."""
    if logits.dim() != 2 or not logits.is_cuda or logits.stride(1) != 1 or logits.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("argmax: expected a 2-D CUDA bf16/fp32 tensor with unit inner stride")
    rows, cols = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(logits.device).cuda_stream)
    _lib.check(_lib.load().mk_argmax(logits.data_ptr(), 0 if logits.dtype == torch.bfloat16 else 1, rows, cols,
                                     logits.stride(0), out.data_ptr(), stream), "mk_argmax")
    return out


def compile(g: Graph, **kw) -> Program:
    return Program(g, **kw).compile()
