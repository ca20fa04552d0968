"""GPU parity tests: every op kind of the megakernel against the fp32 oracle, through the C ABI.

Floating point: bf16 outputs within rel-L2 <= 1e-2 of the fp32 evaluation (helpers.TOL).
Integer work (pos, cache rows written, counters): bit exact.
"""
import numpy as np
import pytest
import torch

import megacute_b200 as mc
from megacute_b200 import workloads as W
from oracle.graph_oracle import evaluate, rel_l2
from tests.helpers import TOL, small_decode, to_cpu

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def rnd(shape, std=1.0, seed=0, mean=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std + mean).to(BF)


def run_both(g, tensors, cuda, steps=1, **kw):
    """Run graph g on the GPU (steps launches) and in the oracle; return (gpu outs, oracle outs, gpu
    states, oracle states, prog)."""
    prog = mc.compile(g, **kw)
    dev = {k: v.to(cuda).contiguous() for k, v in tensors.items()}
    ref_t = {k: v.clone() for k, v in tensors.items()}
    outs = ref = None
    states = {b.name for b in g.states}
    for _ in range(steps):
        outs = prog(**dev)
        outs = outs if isinstance(outs, tuple) else (outs,)
        ref, st = evaluate(g, ref_t)
        for n in states:
            ref_t[n] = st[n]
    prog.check()
    return [o.float().cpu() for o in outs], ref, {n: dev[n].cpu() for n in states}, {n: ref_t[n] for n in states}, prog


def assert_close(outs, ref, tol=TOL):
    for o, r in zip(outs, ref):
        assert torch.isfinite(o).all()
        assert rel_l2(o, r) < tol, rel_l2(o, r)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols,rms,affine", [(1, 2048, True, True), (3, 512, True, False), (300, 1024, False, False),
                                                 (260, 256, False, True), (64, 2048, True, True)])
def test_norm(cuda, rows, cols, rms, affine):
    g = mc.Graph()
    x = g.input("x", (rows, cols))
    w = g.param("w", (1, cols)) if affine else None
    if rms:
        y = g.rms_norm(x, w, eps=1e-5)
    else:
        y = g.layer_norm(x, w, g.param("b", (1, cols)) if affine else None, eps=1e-5)
    g.output(g.unary(y, "identity"))         # keeps the norm unfolded and adds a dependent op
    t = {"x": rnd((rows, cols), 2.0, 1, 0.3)}
    if affine:
        t["w"] = rnd((1, cols), 0.1, 2, 1.0)
        if not rms:
            t["b"] = rnd((1, cols), 0.1, 3)
    outs, ref, *_ = run_both(g, t, cuda)
    assert_close(outs, ref)


@pytest.mark.parametrize("fn", ["relu", "silu", "gelu_tanh", "gelu", "exp", "neg", "sigmoid", "square", "identity"])
def test_unary(cuda, fn):
    g = mc.Graph()
    x = g.input("x", (70, 1032))
    g.output(g.unary(x, fn))
    outs, ref, *_ = run_both(g, {"x": rnd((70, 1032), 1.0, 4)}, cuda)
    assert_close(outs, ref)


@pytest.mark.parametrize("fn", ["add", "sub", "mul", "max", "min"])
def test_binary_and_broadcast(cuda, fn):
    g = mc.Graph()
    a = g.input("a", (96, 520))
    b = g.input("b", (96, 520))
    c = g.input("c", (3, 520))
    y = g.binary(a, b, fn)
    g.output(y, g.binary(y, c, fn, b_group=32))
    outs, ref, *_ = run_both(g, {"a": rnd((96, 520), 1, 5), "b": rnd((96, 520), 1, 6), "c": rnd((3, 520), 1, 7)}, cuda)
    assert_close(outs, ref)


def test_swiglu_modulate_rope(cuda):
    g = mc.Graph()
    S, H, D = 40, 6, 64
    x = g.input("x", (2 * S, H * D))
    u = g.input("u", (2 * S, H * D))
    sc = g.input("sc", (2, H * D))
    sh = g.input("sh", (2, H * D))
    cos = g.input("cos", (S, D))
    sin = g.input("sin", (S, D))
    a = g.swiglu(x, u)
    b = g.modulate(x, sc, sh, group=S)
    c = g.rope(x, cos, sin, heads=H, head_dim=D, seq=S)
    d = g.rope(x.cols_slice(128, 256), cos, sin, heads=4, head_dim=D, seq=S)      # a column slice of a wider buffer
    g.output(a, b, c, d)
    cs, sn = W.rope_tables(S, D)
    t = {"x": rnd((2 * S, H * D), 1, 8), "u": rnd((2 * S, H * D), 1, 9), "sc": rnd((2, H * D), 0.3, 10),
         "sh": rnd((2, H * D), 0.3, 11), "cos": cs, "sin": sn}
    outs, ref, *_ = run_both(g, t, cuda)
    assert_close(outs, ref)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,N,act,bias,res,norm", [
    (1, 2048, 512, None, False, False, False),
    (1, 2048, 3072, None, False, False, True),
    (1, 8192, 296, None, False, True, False),
    (1, 2048, 1024, "swiglu", False, False, True),
    (2, 4096, 640, "gelu_tanh", True, True, False),
    (4, 1024, 1000, "silu", True, False, True),
    (8, 2048, 1544, "relu", True, True, True),
    (3, 1064, 136, None, True, True, False),
    (5, 264, 256, "swiglu", False, False, False),
])
def test_streaming_linear(cuda, M, K, N, act, bias, res, norm):
    """Linears with <= 8 rows run on the weight-streaming path (GEMV)."""
    g = mc.Graph()
    x = g.input("x", (M, K))
    w = g.param("w", (N, K))
    n_out = N // 2 if act == "swiglu" else N
    h = g.rms_norm(x, g.param("nw", (1, K)), eps=1e-5) if norm else x
    y = g.linear(h, w, bias=g.param("b", (1, n_out)) if bias else None, act=act,
                 residual=g.input("r", (M, n_out)) if res else None)
    g.output(y)
    t = {"x": rnd((M, K), 1.0, 1), "w": rnd((N, K), 0.03, 2)}
    if norm:
        t["nw"] = rnd((1, K), 0.05, 3, 1.0)
    if bias:
        t["b"] = rnd((1, n_out), 0.5, 4)
    if res:
        t["r"] = rnd((M, n_out), 1.0, 5)
    outs, ref, _, _, prog = run_both(g, t, cuda)
    assert_close(outs, ref)
    assert [o.kind for o in prog.g.ops] == ["Linear"]                 # the norm was folded


def test_streaming_linear_chain_and_counters(cuda):
    """Dependent streaming linears; dependency counters end at arrivals * launches."""
    g = mc.Graph()
    x = g.input("x", (1, 512))
    w1 = g.param("w1", (1024, 512))
    w2 = g.param("w2", (512, 1024))
    w3 = g.param("w3", (2048, 512))
    h = g.linear(x, w1, act="silu")
    y = g.linear(h, w2, residual=x)
    g.output(g.linear(y, w3))
    t = {"x": rnd((1, 512), 1, 1), "w1": rnd((1024, 512), 0.04, 2), "w2": rnd((512, 1024), 0.03, 3),
         "w3": rnd((2048, 512), 0.04, 4)}
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=3)
    assert_close(outs, ref)
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 3)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,H,KVH,D,max_seq,ctx", [(1, 8, 2, 64, 256, 100), (3, 4, 4, 64, 128, 0), (2, 8, 1, 128, 256, 200),
                                                  (1, 32, 8, 64, 1152, 1024), (20, 8, 2, 64, 384, 300),
                                                  (40, 16, 8, 64, 256, 129), (160, 4, 1, 64, 128, 0), (50, 8, 4, 128, 256, 77),
                                                  (150, 32, 8, 64, 128, 64)])
@pytest.mark.parametrize("fused", [False, True])
def test_decode_attention(cuda, B, H, KVH, D, max_seq, ctx, fused):
    """rope_append + decode_attention, kept separate (q_out is also an output) or fused by the pass."""
    _decode_attention_case(cuda, B, H, KVH, D, max_seq, ctx, fused)


@pytest.mark.parametrize("B,H,KVH,max_seq,ctx,splits", [
    (9, 8, 2, 128, 37, 1), (9, 8, 2, 128, 37, 2), (12, 16, 2, 256, 45, 3), (16, 32, 8, 384, 300, 1), (16, 32, 8, 384, 300, 5),
    (3, 32, 8, 256, 17, 4), (70, 32, 8, 128, 0, 2), (24, 8, 8, 256, 200, 3), (150, 32, 8, 256, 129, 2)])
@pytest.mark.parametrize("fused", [False, True])
def test_decode_attention_many_sequences(cuda, monkeypatch, B, H, KVH, max_seq, ctx, splits, fused):
    """The many-sequence form: one instruction = a sequence's KV split over all kv heads, whole cache rows
    through bulk copies, one warp per kv head.  GQA groups of 1, 4 and 8, fewer kv heads than warps,
    contexts that are not a multiple of the 16-row tile, shorter than one tile, or empty; splits that get
    no keys; the last split of a sequence to arrive merges."""
    monkeypatch.setenv("MEGACUTE_B200_ATT_BULK", "1")
    monkeypatch.setenv("MEGACUTE_B200_KV_SPLITS", str(splits))
    prog = _decode_attention_case(cuda, B, H, KVH, 64, max_seq, ctx, fused)
    att = [o for o in prog.g.ops if o.kind == "DecodeAttention"]
    assert att and all(o.bulk and o.heads_per_inst == KVH and o.splits == min(splits, max_seq // 64) for o in att)


def _decode_attention_case(cuda, B, H, KVH, D, max_seq, ctx, fused):
    g = mc.Graph()
    qkv = g.input("qkv", (B, (H + 2 * KVH) * D))
    cos = g.input("cos", (max_seq, D))
    sin = g.input("sin", (max_seq, D))
    pos = g.state("pos", (1, 1), torch.int32)
    kc = g.state("k_cache", (B * max_seq, KVH * D))
    vc = g.state("v_cache", (B * max_seq, KVH * D))
    q = g.rope_append(qkv, cos, sin, pos, kc, vc, heads=H, kv_heads=KVH, head_dim=D, max_seq=max_seq)
    a = g.decode_attention(q, kc, vc, pos, heads=H, kv_heads=KVH, head_dim=D, max_seq=max_seq)
    g.increment(pos)
    if fused:
        g.output(a)
    else:
        g.output(a, q)
    cs, sn = W.rope_tables(max_seq, D)
    cache = lambda s: (torch.cat([rnd((B, ctx, KVH * D), 1, s), torch.zeros(B, max_seq - ctx, KVH * D, dtype=BF)], 1)
                       .reshape(B * max_seq, KVH * D).contiguous())
    t = {"qkv": rnd((B, (H + 2 * KVH) * D), 1, 1), "cos": cs, "sin": sn,
         "pos": torch.full((1, 1), ctx, dtype=torch.int32), "k_cache": cache(2), "v_cache": cache(3)}
    before = {n: t[n].clone() for n in ("k_cache", "v_cache")}
    outs, ref, st, rst, prog = run_both(g, t, cuda, steps=2)
    kinds = [o.kind for o in prog.g.ops]
    assert ("RopeAppend" not in kinds) == fused
    assert_close(outs, ref)
    assert int(st["pos"]) == ctx + 2 == int(rst["pos"])
    for n in ("k_cache", "v_cache"):
        got, want = st[n].view(B, max_seq, -1), rst[n].view(B, max_seq, -1)
        old = before[n].view(B, max_seq, -1)
        # exactly rows ctx and ctx+1 of every sequence changed (integer-exact append slots)
        changed = (got != old).any(-1)
        mask = torch.zeros(B, max_seq, dtype=torch.bool)
        mask[:, ctx:ctx + 2] = True
        assert not changed[~mask].any()
        assert rel_l2(got[:, ctx:ctx + 2].float(), want[:, ctx:ctx + 2].float()) < TOL
    for b in prog.g.buffers:
        if b.kind == "workspace" and b.dtype == torch.int32:
            assert int(prog.buffer(b).abs().sum()) == 0
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 2)
    return prog


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B", [1, 2, 8])
def test_small_llama_decode_steps(cuda, B):
    g, params, st, ids = small_decode(B=B, E=256, H=4, KVH=2, F=512, n=3, max_seq=256, ctx=70, vocab=1000)
    prog = mc.compile(g)
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st.items()}
    rs = {k: v.clone() for k, v in st.items()}
    emb = params["lm_head"]
    ids_g, ids_r = ids.clone(), ids.clone()
    for step in range(6):
        ds["x"].copy_(dp["lm_head"][ids_g.to(cuda)])
        logits = prog(**dp, **ds).float().cpu()
        rs["x"] = emb[ids_r].clone()
        ref, new = evaluate(g, {**params, **rs})
        for n in ("pos", "k_cache", "v_cache"):
            rs[n] = new[n]
        assert rel_l2(logits, ref[0]) < TOL, (step, rel_l2(logits, ref[0]))
        ids_g, ids_r = logits.argmax(-1), ref[0].argmax(-1)
        assert torch.equal(ids_g, ids_r)
        assert int(ds["pos"]) == int(rs["pos"]) == 71 + step
    prog.check()
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 6)


def test_timeout_is_reported_not_hung(cuda):
    """Host-made fault: a wait target no arrival can satisfy.  The launch must end with an error
    status within the (shortened) limit and the program must be reusable after reset()."""
    g = mc.Graph()
    x = g.input("x", (1, 512))
    h = g.linear(x, g.param("w1", (512, 512)))
    g.output(g.linear(h, g.param("w2", (512, 512))))
    t = {"x": rnd((1, 512), 1, 1).to(cuda), "w1": rnd((512, 512), 0.04, 2).to(cuda), "w2": rnd((512, 512), 0.04, 3).to(cuda)}
    prog = mc.compile(g)
    good = prog(**t).float().cpu().clone()
    prog.check()
    from megacute_b200 import _lib
    prog.set_timeout(0.05)
    s = prog.sched
    _lib.check(_lib.load().mk_program_poke_wait(prog._handle, 0, int(s.wait_cnt[0]), int(s.wait_tgt[0]) + 1000))
    prog(**t)
    with pytest.raises(_lib.MegakernelTimeout):
        prog.check()
    _lib.check(_lib.load().mk_program_poke_wait(prog._handle, 0, int(s.wait_cnt[0]), int(s.wait_tgt[0])))
    prog.reset()
    again = prog(**t).float().cpu()
    prog.check()
    assert torch.equal(again, good)


def test_timeline(cuda):
    g, params, st, ids = small_decode(B=1, n=2)
    prog = mc.compile(g, trace=True)
    with pytest.raises(RuntimeError):
        mc.compile(g).timeline()
    dp = {k: v.to(cuda) for k, v in {**params, **st}.items()}
    prog(**dp)
    tl = prog.timeline()
    assert len([r for r in tl.records if r[1] == 1]) == prog.sched.n
    assert tl.span_us() > 0 and "Linear" in tl.summary() and len(tl.chrome_events()) > 0


def test_timeline_of_tile_gemm_runs(cuda):
    """A CTA that gets several tile-GEMM instructions in a row runs them inside one call of the body, which then writes
    the trace records itself: every instruction must still have exactly one record, under its own sequence number,
    with ordered time stamps and phase marks."""
    import numpy as np
    M, K = 4096, 512
    g = mc.Graph()
    x = g.input("x", (M, K))
    y = g.linear(g.unary(x, "identity"), g.param("w1", (1024, K)), act="gelu_tanh")     # 32 x 4 (or 8) tiles: 2 or more per CTA
    g.output(g.linear(y, g.param("w2", (384, 1024))))                                    # narrow tiles behind them
    gen = torch.Generator().manual_seed(5)
    t = {"x": torch.randn(M, K, generator=gen).to(torch.bfloat16), "w1": (torch.randn(1024, K, generator=gen) * 0.04).to(torch.bfloat16),
         "w2": (torch.randn(384, 1024, generator=gen) * 0.03).to(torch.bfloat16)}
    prog = mc.compile(g, trace=True)
    dp = {k: v.to(cuda) for k, v in t.items()}
    for _ in range(2):
        prog(**dp)
    prog.check()
    tl = prog.timeline()
    comp = tl.table[tl.table["role"] == 1]
    assert len(comp) == prog.sched.n and np.array_equal(np.sort(comp["seq"]), np.arange(prog.sched.n))
    assert bool((comp["t0"] <= comp["t1"]).all()) and bool((comp["t1"] < comp["t2"]).all())
    per_op = np.bincount(np.asarray(prog.sched.op_of)[comp["seq"]], minlength=len(prog.g.ops))
    assert np.array_equal(per_op, np.bincount(np.asarray(prog.sched.op_of), minlength=len(prog.g.ops)))
    # a CTA runs its instructions in list order: sequence numbers rise with the slot
    for sm in np.unique(comp["sm"])[:8]:
        rows = comp[comp["sm"] == sm]
        assert bool((np.diff(rows["seq"]) > 0).all()) and bool((np.diff(rows["t2"]) > 0).all())
    ph = tl.table[tl.table["role"] == 2]
    gemm = np.array([prog.g.ops[int(k)].kind in ("Linear", "LinearSplit") for k in np.asarray(prog.sched.op_of)[ph["seq"]]])
    by_seq = {int(r["seq"]): r for r in comp}
    for r in ph[gemm][:256]:
        c = by_seq[int(r["seq"])]
        assert c["t1"] <= r["t0"] <= r["t1"] <= r["t2"] <= c["t2"], (r, c)


# ---------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(1, 128256), (64, 128256), (3, 1000), (2, 8)])
def test_argmax_rows(cuda, dtype, rows, cols):
    g = torch.Generator(device=cuda).manual_seed(rows * 131 + cols)
    x = torch.randn(rows, cols, generator=g, device=cuda, dtype=torch.float32).to(dtype)
    # plant a unique maximum per row, and a tie whose lower index must win in row 0
    want = torch.randint(0, cols, (rows,), generator=g, device=cuda)
    x[torch.arange(rows, device=cuda), want] = 100.0
    if cols > 8:
        lo = int(want[0])
        hi = min(cols - 1, lo + 5)
        x[0, hi] = 100.0
    got = mc.argmax(x)
    assert got.dtype == torch.int64 and torch.equal(got, want)
    # a view with a leading dimension larger than its width
    wide = torch.zeros(rows, cols + 16, device=cuda, dtype=dtype)
    wide[:, :cols] = x
    assert torch.equal(mc.argmax(wide[:, :cols]), want)
