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
