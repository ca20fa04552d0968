"""mk_launch_noalloc: the launch variant for hosts that may not allocate device memory.

Some users of the C ABI cannot call cudaMalloc when they launch -- a serving process that gave all
of HBM to its own pool at start-up, or a latency-critical loop that cannot afford the device-wide
synchronisation of an allocation.  mk_launch_noalloc keeps the kernel's dependency counters and
status words in a static device array inside the library instead.  This test drives it through the
C ABI with tables and tensors that the *test* places on the device (torch stands in for the host's
own pool) and checks, on two calls in a row, that it writes the same result as the ordinary
mk_program_create / mk_launch path.

Collected last on purpose (file name): a failure here never hides another test's result.
"""
import ctypes

import pytest
import torch

import megacute_b200 as mc
from megacute_b200 import _lib
from oracle.graph_oracle import evaluate, rel_l2
from tests.helpers import TOL

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _graph():
    g = mc.Graph()
    x = g.input("x", (1, 512))
    h = g.linear(g.rms_norm(x, g.param("nw", (1, 512)), eps=1e-5), g.param("w1", (2048, 512)), act="swiglu")
    y = g.linear(h, g.param("w2", (512, 1024)), residual=x)
    g.output(g.linear(y, g.param("w3", (768, 512)), act="gelu_tanh"))
    return g


def _inputs(dev):
    gen = torch.Generator().manual_seed(11)
    r = lambda shape, std, mean=0.0: (torch.randn(shape, generator=gen) * std + mean).to(BF)
    return {k: v.to(dev) for k, v in dict(x=r((1, 512), 1.0), nw=r((1, 512), 0.05, 1.0), w1=r((2048, 512), 0.04),
                                          w2=r((512, 1024), 0.03), w3=r((768, 512), 0.04)).items()}


def test_noalloc_launch_matches_program_launch(cuda):
    g = _graph()
    t = _inputs(cuda)
    prog = mc.compile(g)
    want = prog(**t).clone()                       # ordinary path: library-allocated counters
    prog.check()
    ref, _ = evaluate(g, {k: v.cpu() for k, v in t.items()})
    assert rel_l2(want.float().cpu(), ref[0]) < TOL

    # tables and descriptors in device memory owned by the caller (here: torch tensors)
    insts, waits, arrives = (a.to(cuda) for a in prog._tables)
    desc = torch.frombuffer(bytearray(bytes(prog._desc)), dtype=torch.uint8).to(cuda)
    out = prog(**t)                                # same buffer the descriptors point at
    torch.cuda.synchronize()
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = (ctypes.c_int32 * _lib.ST_WORDS)()
    s = prog.sched
    for call in range(2):                          # two calls in a row share the static scratch
        out.zero_()
        rc = lib.mk_launch_noalloc(cuda.index or 0, insts.data_ptr(), s.n, waits.data_ptr(), len(s.wait_cnt),
                                   arrives.data_ptr(), len(s.arr_cnt), desc.data_ptr(), len(prog.g.ops),
                                   s.num_counters, prog.sm_count, stream, status)
        _lib.check(rc, f"mk_launch_noalloc call {call}")
        assert list(status)[0] == 0
        got = out.float().cpu()
        assert rel_l2(got, want.float().cpu()) < TOL
        assert torch.equal(out, want)              # same kernel, same order of operations: identical bits


def test_noalloc_rejects_oversized_graph(cuda):
    lib = _lib.load()
    dummy = torch.zeros(64, dtype=torch.int32, device=cuda)
    rc = lib.mk_launch_noalloc(cuda.index or 0, dummy.data_ptr(), 1, None, 0, None, 0, dummy.data_ptr(), 1,
                               16384 + 1, 1, None, None)
    assert rc == -6 and b"MK_NOALLOC_MAX_COUNTERS" in lib.mk_strerror(rc)


def test_noalloc_runs_tile_gemm_and_decode_attention(cuda, monkeypatch):
    """A batch-16 decode step through mk_launch_noalloc: tile GEMMs (their mma.sync body, since the
    caller's descriptors carry no library-made tensor maps), split-K reductions, the fused decode
    attention with a two-way KV split (partial and arrival-count workspaces, zeroed by the caller as
    the header requires), norms and the increment.  Checked, on two calls in a row, against the
    ordinary launch of the same graph with its mma.sync body, the oracle, and the integer state."""
    from tests.helpers import small_decode
    monkeypatch.setenv("MEGACUTE_B200_KV_SPLITS", "2")
    monkeypatch.setenv("MEGACUTE_B200_NO_TCGEN05", "1")
    g, params, st0, ids = small_decode(B=16, E=256, H=4, KVH=2, F=512, n=2, max_seq=256, ctx=120, vocab=1000)
    prog = mc.compile(g)
    kinds = {o.kind for o in prog.g.ops}
    assert {"LinearSplit", "DecodeAttention", "Norm"} <= kinds
    assert all(o.splits == 2 for o in prog.g.ops if o.kind == "DecodeAttention")
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st0.items()}
    want = prog(**dp, **ds).float().cpu()
    prog.check()
    assert prog.tcgen05_ops == 0
    want_k = ds["k_cache"].clone()
    ref, ref_st = evaluate(g, {**params, **st0})
    assert rel_l2(want, ref[0]) < TOL

    insts, waits, arrives = (a.to(cuda) for a in prog._tables)
    desc = torch.frombuffer(bytearray(bytes(prog._desc)), dtype=torch.uint8).to(cuda)
    out = prog._bufs[prog.g.outputs[0].buf.id]
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = (ctypes.c_int32 * _lib.ST_WORDS)()
    s = prog.sched
    before = torch.cuda.current_device()
    for call in range(2):
        for k, v in st0.items():                   # same tensors (the descriptors hold their addresses), fresh contents
            ds[k].copy_(v)
        for b in prog.g.buffers:                   # workspaces are zero on entry: the caller's duty here
            if b.kind == "workspace":
                prog._bufs[b.id].zero_()
        out.zero_()
        rc = lib.mk_launch_noalloc(cuda.index or 0, insts.data_ptr(), s.n, waits.data_ptr(), len(s.wait_cnt),
                                   arrives.data_ptr(), len(s.arr_cnt), desc.data_ptr(), len(prog.g.ops),
                                   s.num_counters, prog.sm_count, stream, None)
        _lib.check(rc, f"mk_launch_noalloc call {call}")
        _lib.check(lib.mk_noalloc_status(cuda.index or 0, stream, status), "mk_noalloc_status")
        assert list(status)[0] == 0
        got = out.float().cpu()
        assert rel_l2(got, want) < 1e-3            # split-K partial sums arrive in any order: equal up to fp32 rounding
        assert rel_l2(got, ref[0]) < TOL
        assert int(ds["pos"]) == int(ref_st["pos"]) == 121
        assert rel_l2(ds["k_cache"].float(), want_k.float()) < 1e-3
        parts = {o.part.buf.id for o in prog.g.ops if o.kind == "DecodeAttention"}
        for b in prog.g.buffers:                   # ... and zero again on exit (split-K sums, arrival counts; the
            if b.kind == "workspace" and b.id not in parts:      # split-KV partial rows are overwritten, not zeroed)
                assert not prog._bufs[b.id].any()
    assert torch.cuda.current_device() == before   # the entry point leaves the caller's device alone


def test_grid_larger_than_the_device_is_an_argument_error(cuda):
    """All CTAs must be resident at once; a grid above the SM count is refused up front (it would
    otherwise end in a dependency timeout)."""
    g = _graph()
    caps = _lib.Caps()
    _lib.check(_lib.load().mk_query(cuda.index or 0, ctypes.byref(caps)))
    with pytest.raises(_lib.MegakernelError, match="grid"):
        mc.compile(g, sm_count=caps.sm_count + 1)
    lib = _lib.load()
    dummy = torch.zeros(64, dtype=torch.int32, device=cuda)
    rc = lib.mk_launch_noalloc(cuda.index or 0, dummy.data_ptr(), 1, None, 0, None, 0, dummy.data_ptr(), 1, 1,
                               caps.sm_count + 1, None, None)
    assert rc == -2
