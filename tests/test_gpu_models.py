"""GPU parity tests of the tile GEMM, prefill attention and the benchmarked model graphs."""
import numpy as np
import pytest
import torch

import megacute_b200 as mc
from megacute_b200 import workloads as W
from megacute_b200.builders import dit_stack, llama_decode, llama_stack, mlp_block
from oracle.graph_oracle import evaluate, rel_l2
from tests.helpers import TOL, small_decode
from tests.test_gpu_ops import assert_close, rnd, run_both

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("M,K,N,act,bias,res", [
    (128, 64, 128, None, False, False),
    (256, 2048, 512, None, True, True),
    (200, 512, 328, "gelu_tanh", True, False),
    (9, 2048, 3072, None, False, False),
    (64, 8192, 2048, None, False, True),
    (130, 256, 1024, "swiglu", False, False),
    (64, 2048, 16384, "swiglu", False, False),
    (300, 1024, 136, "relu", True, True),
])
def test_tile_linear(cuda, M, K, N, act, bias, res):
    g = mc.Graph()
    x = g.input("x", (M, K))
    w = g.param("w", (N, K))
    n_out = N // 2 if act == "swiglu" else N
    y = g.linear(x, w, bias=g.param("b", (1, n_out)) if bias else None, act=act,
                 residual=g.input("r", (M, n_out)) if res else None)
    g.output(y)
    t = {"x": rnd((M, K), 1.0, 1), "w": rnd((N, K), 0.03, 2)}
    if bias:
        t["b"] = rnd((1, n_out), 0.5, 4)
    if res:
        t["r"] = rnd((M, n_out), 1.0, 5)
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)      # twice: split-K workspaces are re-zeroed
    assert_close(outs, ref)
    # every one of these shapes has whole 64-element k-tiles per instruction and aligned operands:
    # the library must have bound the tile GEMM ops to its tcgen05 body, not the mma.sync one
    n_gemm = sum(o.kind in ("Linear", "LinearSplit") for o in prog.g.ops)
    assert prog.tcgen05_ops == n_gemm >= 1


def test_tile_linear_both_bodies_agree(cuda, monkeypatch):
    """The mma.sync body (MEGACUTE_B200_NO_TCGEN05) and the tcgen05 body give the same result up to
    the order of fp32 accumulation."""
    g = mc.Graph()
    y = g.linear(g.input("x", (96, 1024)), g.param("w", (640, 1024)), act="gelu_tanh")
    g.output(y)
    t = {"x": rnd((96, 1024), 1.0, 1), "w": rnd((640, 1024), 0.03, 2)}
    outs_tc, ref, _, _, prog_tc = run_both(g, t, cuda)
    monkeypatch.setenv("MEGACUTE_B200_NO_TCGEN05", "1")
    outs_mma, _, _, _, prog_mma = run_both(g, t, cuda)
    assert prog_tc.tcgen05_ops == 1 and prog_mma.tcgen05_ops == 0
    assert_close(outs_tc, ref)
    assert_close(outs_mma, ref)
    assert rel_l2(outs_tc[0], outs_mma[0]) < 2e-3


def test_tile_linear_weight_sources_and_rebind(cuda, monkeypatch):
    """Packed weight tiles (default) and bulk tensor copies over the caller's matrix
    (MEGACUTE_B200_NO_WEIGHT_PACK) give the same result; binding another weight tensor re-packs."""
    g = mc.Graph()
    g.output(g.linear(g.input("x", (64, 2048)), g.param("w", (1536, 2048)), residual=g.input("r", (64, 1536))))
    t = {"x": rnd((64, 2048), 1.0, 1), "w": rnd((1536, 2048), 0.03, 2), "r": rnd((64, 1536), 1.0, 3)}
    outs_p, ref, _, _, prog_p = run_both(g, t, cuda)
    assert prog_p.tcgen05_ops >= 1 and prog_p.packed_weight_bytes == 1536 * 2048 * 2
    assert_close(outs_p, ref)
    # the same program with another weight tensor: the snapshot follows the rebind
    t2 = dict(t, w=rnd((1536, 2048), 0.03, 7))
    dev2 = {k: v.to(cuda).contiguous() for k, v in t2.items()}
    out2 = prog_p(**dev2)
    prog_p.check()
    ref2, _ = evaluate(g, t2)
    assert rel_l2(out2.float().cpu(), ref2[0]) < TOL
    assert prog_p.packed_weight_bytes == 1536 * 2048 * 2            # the first copy was freed
    # weights changed in place: the snapshot is stale until refresh_weights()
    dev2["w"].mul_(0.5)
    t3 = dict(t2, w=(t2["w"].float() * 0.5).to(BF))
    prog_p.refresh_weights()
    out3 = prog_p(**dev2)
    prog_p.check()
    ref3, _ = evaluate(g, t3)
    assert rel_l2(out3.float().cpu(), ref3[0]) < TOL
    # another input tensor, same weights: bound again, not packed again
    dev2["x"] = dev2["x"].clone()
    out4 = prog_p(**dev2)
    prog_p.check()
    assert torch.equal(out4, out3) and prog_p.packed_weight_bytes == 1536 * 2048 * 2
    monkeypatch.setenv("MEGACUTE_B200_NO_WEIGHT_PACK", "1")
    outs_t, _, _, _, prog_t = run_both(g, t, cuda)
    assert prog_t.tcgen05_ops >= 1 and prog_t.packed_weight_bytes == 0
    assert_close(outs_t, ref)
    assert rel_l2(outs_t[0], outs_p[0]) < 1e-3


def test_tile_linear_timeout_is_reported_not_hung(cuda):
    """Host-made fault in a launch of tcgen05 tile linears: a wait target no arrival can satisfy.
    The launch ends with an error status (bounded waits; weight tiles already requested are waited
    for, tensor memory is given back) and the program works again after reset()."""
    g = mc.Graph()
    h = g.linear(g.input("x", (96, 512)), g.param("w1", (1024, 512)), act="relu")
    g.output(g.linear(h, g.param("w2", (512, 1024))))
    t = {"x": rnd((96, 512), 1, 1).to(cuda), "w1": rnd((1024, 512), 0.04, 2).to(cuda), "w2": rnd((512, 1024), 0.04, 3).to(cuda)}
    prog = mc.compile(g)
    good = prog(**t).float().cpu().clone()
    prog.check()
    assert prog.tcgen05_ops >= 2
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
    # (split-K partial sums are reduce-added in whatever order the CTAs arrive: equal up to fp32 rounding)
    assert rel_l2(again, good) < 1e-3


def test_streaming_and_tile_linears_alternate(cuda):
    """Streaming linears (<= 8 rows: two-stage weight ring) and tcgen05 tile linears (eight single-tile
    weight slots in the same shared memory) alternate in one launch, several instructions of each
    per CTA: the producer warp must drain one kind of slot before it fills the other."""
    g = mc.Graph()
    a = g.input("a", (4, 1024))
    b = g.input("b", (96, 1024))
    for i in range(3):
        a = g.linear(a, g.param(f"ws{i}", (40 * 148, 1024)), act="gelu_tanh")      # 40 outputs per CTA and op
        a = g.linear(a, g.param(f"wd{i}", (1024, 40 * 148)))
        b = g.linear(b, g.param(f"wt{i}", (2 * 148 * 128, 1024)), act="relu")       # two tiles per CTA and op
        b = g.linear(b, g.param(f"wu{i}", (1024, 2 * 148 * 128)))
    g.output(a)
    g.output(b)
    t = {"a": rnd((4, 1024), 1.0, 1), "b": rnd((96, 1024), 1.0, 2)}
    for i in range(3):
        t[f"ws{i}"] = rnd((40 * 148, 1024), 0.03, 10 + i)
        t[f"wd{i}"] = rnd((1024, 40 * 148), 0.03, 20 + i)
        t[f"wt{i}"] = rnd((2 * 148 * 128, 1024), 0.03, 30 + i)
        t[f"wu{i}"] = rnd((1024, 2 * 148 * 128), 0.01, 40 + i)
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)
    kinds = {o.kind for o in prog.g.ops}
    assert prog.tcgen05_ops >= 6 and prog.packed_weight_bytes > 0
    assert_close(outs, ref)


def test_split_k_in_place_residual(cuda):
    """A residual linear with few tiles reduce-adds its K splits straight into the residual stream."""
    g = mc.Graph()
    x = g.input("x", (64, 4096))
    r = g.input("r", (64, 1024))
    s = g.unary(r, "identity")                       # a runtime-owned residual stream
    y = g.linear(x, g.param("w", (1024, 4096)), residual=s)
    g.output(g.unary(y, "identity"))
    t = {"x": rnd((64, 4096), 1, 1), "r": rnd((64, 1024), 1, 2), "w": rnd((1024, 4096), 0.02, 3)}
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)
    kinds = [o.kind for o in prog.g.ops]
    assert "LinearSplit" in kinds and "SplitFinalize" not in kinds
    assert_close(outs, ref)


def test_mlp_block_config(cuda):
    """The single MLP block of the benchmark configurations: y = linear(linear(rms_norm(x, nw), w1, swiglu), w2, residual=x), M = 256."""
    g = mlp_block(256)
    t = {k: v.cpu() for k, v in W.mlp_block_inputs(256, device="cpu").items()}
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)
    assert_close(outs, ref)


@pytest.mark.parametrize("B,Sq,Sk,H,KVH,D,causal", [
    (2, 128, 128, 4, 4, 64, False), (2, 256, 256, 4, 2, 64, True), (1, 200, 200, 2, 1, 64, True),
    (3, 96, 160, 2, 2, 64, False), (1, 256, 256, 2, 1, 128, True), (2, 130, 130, 2, 2, 128, False),
    (1, 1024, 1024, 8, 2, 64, True), (2, 300, 300, 4, 1, 64, True), (1, 64, 700, 2, 2, 64, False), (5, 128, 128, 3, 3, 64, True),
])
@pytest.mark.parametrize("body", ["mma.sync", "tcgen05"])
def test_prefill_attention(cuda, monkeypatch, B, Sq, Sk, H, KVH, D, causal, body):
    if body == "tcgen05" and D != 64:
        pytest.skip("the tcgen05 body takes head_dim 64")
    monkeypatch.setenv("MEGACUTE_B200_ATTN_TCGEN05", "1" if body == "tcgen05" else "0")     # (the default is the tcgen05 body)
    g = mc.Graph()
    q = g.input("q", (B * Sq, H * D))
    kv = g.input("kv", (B * Sk, 2 * KVH * D))          # k and v are column slices of one buffer
    g.output(g.attention(q, kv.cols_slice(0, KVH * D), kv.cols_slice(KVH * D, KVH * D), batch=B, heads=H,
                         head_dim=D, causal=causal, kv_heads=KVH))
    t = {"q": rnd((B * Sq, H * D), 1, 1), "kv": rnd((B * Sk, 2 * KVH * D), 1, 2)}
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)
    assert_close(outs, ref)
    # the counter says which body ran: tcgen05 (S and O in tensor memory) when asked for, else mma.sync
    assert prog.tcgen05_attention_ops == (1 if body == "tcgen05" else 0)


def test_prefill_attention_both_bodies_agree(cuda, monkeypatch):
    """The tcgen05 body and the mma.sync body (MEGACUTE_B200_NO_TCGEN05) of the prefill attention on the same
    inputs: scores with a wide range (so that the lazy rescale of the running maximum triggers), causal,
    GQA, a ragged last query tile."""
    B, S, H, KVH, D = 2, 333, 4, 2, 64
    g = mc.Graph()
    q = g.input("q", (B * S, H * D))
    kv = g.input("kv", (B * S, 2 * KVH * D))
    g.output(g.attention(q, kv.cols_slice(0, KVH * D), kv.cols_slice(KVH * D, KVH * D), batch=B, heads=H, head_dim=D,
                         causal=True, kv_heads=KVH))
    t = {"q": rnd((B * S, H * D), 3.0, 1), "kv": rnd((B * S, 2 * KVH * D), 3.0, 2)}       # logits of +-70: maxima jump
    monkeypatch.setenv("MEGACUTE_B200_ATTN_TCGEN05", "1")
    outs_tc, ref, _, _, prog_tc = run_both(g, t, cuda)
    monkeypatch.setenv("MEGACUTE_B200_ATTN_TCGEN05", "0")
    outs_mma, _, _, _, prog_mma = run_both(g, t, cuda)
    assert prog_tc.tcgen05_attention_ops == 1 and prog_mma.tcgen05_attention_ops == 0
    assert_close(outs_tc, ref)
    assert_close(outs_mma, ref)
    assert rel_l2(outs_tc[0], outs_mma[0]) < 5e-3


@pytest.mark.parametrize("attn_tc", ["0", "1"])
def test_small_prefill_stack(cuda, monkeypatch, attn_tc):
    monkeypatch.setenv("MEGACUTE_B200_ATTN_TCGEN05", attn_tc)
    B, S, E, H, KVH, F, n, V = 2, 192, 256, 4, 2, 512, 2, 1000
    g = llama_stack(B, S, E, H, KVH, F, n, eps=1e-5, vocab=V)
    w = W.llama_weights(E, H, KVH, F, n, V, 0, "cpu")
    cos, sin = W.rope_tables(S, E // H)
    ids = torch.randint(0, V, (B * S,), generator=torch.Generator().manual_seed(1))
    t = dict(x=w["lm_head"][ids].contiguous(), cos=cos, sin=sin, **w)
    outs, ref, _, _, prog = run_both(g, t, cuda)
    assert_close(outs, ref)
    assert torch.equal(outs[0].argmax(-1), ref[0].argmax(-1))
    assert prog.tcgen05_attention_ops == (n if attn_tc == "1" else 0)


def test_small_dit_stack(cuda):
    B, S, E, H, F, n = 3, 64, 256, 4, 1024, 2
    g = dit_stack(B, S, E, H, F, n)
    t = W.dit_inputs(B, S, E, F, n, 0, "cpu")
    outs, ref, *_ = run_both(g, t, cuda)
    assert_close(outs, ref)


@pytest.mark.parametrize("B,att_heads,bulk", [(16, None, "0"), (64, None, "0"), (64, "2", "0"), (16, None, "1"), (64, None, None)])
def test_batched_decode_small(cuda, monkeypatch, B, att_heads, bulk):
    """More than 8 sequences: unfolded norms, tile GEMMs with split-K, and the decode attention in its
    many-sequence form (the default from 32 sequences on: all kv heads of a sequence per instruction) or,
    with that switched off, in the per-head form -- one kv head per instruction, or (forced here;
    chosen when there are more pairs than SMs) several."""
    if att_heads:
        monkeypatch.setenv("MEGACUTE_B200_ATT_HEADS", att_heads)
    if bulk:
        monkeypatch.setenv("MEGACUTE_B200_ATT_BULK", bulk)
    g, params, st, ids = small_decode(B=B, E=256, H=4, KVH=2, F=512, n=2, max_seq=256, ctx=120, vocab=1000)
    prog = mc.compile(g)
    hp = {o.heads_per_inst for o in prog.g.ops if o.kind == "DecodeAttention"}
    assert hp == ({2} if att_heads or bulk != "0" else {1})
    assert {bool(o.bulk) for o in prog.g.ops if o.kind == "DecodeAttention"} == {bulk != "0"}
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st.items()}
    rs = {k: v.clone() for k, v in st.items()}
    for step in range(3):
        logits = prog(**dp, **ds).float().cpu()
        ref, new = evaluate(g, {**params, **rs})
        assert rel_l2(logits, ref[0]) < TOL, (step, rel_l2(logits, ref[0]))
        for n_ in ("pos", "k_cache", "v_cache"):
            rs[n_] = new[n_]
        nxt = ref[0].argmax(-1)
        rs["x"] = params["lm_head"][nxt].clone()
        ds["x"].copy_(rs["x"].to(cuda))
    prog.check()
    assert int(ds["pos"]) == 123
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 3)


@pytest.mark.parametrize("bulk", ["0", "1"])
def test_batched_decode_workspace_inputs_with_kv_splits(cuda, monkeypatch, bulk):
    """Split-K QKV projection feeding the fused decode attention straight from its fp32 workspace, with
    the KV range split over several instructions: the pair's (many-sequence form: the sequence's) last
    instruction to arrive zeroes the workspace columns, so three consecutive steps (which accumulate
    into the same workspace) stay right."""
    monkeypatch.setenv("MEGACUTE_B200_KV_SPLITS", "3")
    monkeypatch.setenv("MEGACUTE_B200_ATT_BULK", bulk)
    g, params, st, ids = small_decode(B=16, E=2048, H=32, KVH=8, F=512, n=1, max_seq=512, ctx=300, vocab=512)
    prog = mc.compile(g)
    att = [o for o in prog.g.ops if o.kind == "DecodeAttention"]
    assert att and all(o.zero_inputs and o.splits == 3 for o in att)
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st.items()}
    rs = {k: v.clone() for k, v in st.items()}
    for step in range(3):
        logits = prog(**dp, **ds).float().cpu()
        ref, new = evaluate(g, {**params, **rs})
        assert rel_l2(logits, ref[0]) < TOL, (step, rel_l2(logits, ref[0]))
        for n_ in ("pos", "k_cache", "v_cache"):
            rs[n_] = new[n_]
        rs["x"] = params["lm_head"][ref[0].argmax(-1)].clone()
        ds["x"].copy_(rs["x"].to(cuda))
    prog.check()
    # (split-K sums arrive in any order, so an appended key may differ from the oracle's by a bf16 ulp)
    assert rel_l2(ds["k_cache"].float().cpu(), rs["k_cache"].float()) < 1e-3 and int(ds["pos"]) == 303


def test_llama_1b_decode_32_greedy_steps(cuda):
    """The headline decode configuration at full size: 32 greedy steps, tokens identical to the fp32 evaluation
    (run on the same GPU in fp32 torch so that it finishes in seconds), logits within tolerance,
    pos and the appended cache rows exact."""
    c = W.LLAMA_1B
    B, ctx, max_seq = 1, 1024, 1152
    g = llama_decode(B, c["E"], c["H"], c["KVH"], c["F"], c["n"], max_seq, c["vocab"], c["eps"])
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], 0, cuda)
    st, ids = W.llama_decode_state(B, c["E"], c["H"], c["KVH"], c["n"], max_seq, ctx, c["vocab"], 1, cuda)
    cos, sin = W.rope_tables(max_seq, 64, c["theta"], cuda)
    params = dict(cos=cos, sin=sin, **w)
    rs = {k: v.clone() for k, v in st.items()}
    k0 = st["k_cache"].clone()
    prog = mc.compile(g)
    # Random-init weights give a flat next-token distribution: the two best logits often differ by
    # less than one bf16 step of the (bf16) logits tensor, where no bf16 implementation can be
    # expected to order them like fp32 does.  The oracle's token is fed to both sides every step;
    # the GPU token must equal it unless the fp32 margin between the two candidates is below two
    # bf16 steps (2^-7 relative) of the winning logit.
    worst, exact = 0.0, 0
    for step in range(32):
        st["x"].copy_(w["lm_head"][ids])
        logits = prog(**params, **st).float()
        rs["x"] = w["lm_head"][ids].clone()
        ref, new = evaluate(g, {**params, **rs}, device=cuda)
        for n_ in ("pos", "k_cache", "v_cache"):
            rs[n_] = new[n_]
        worst = max(worst, rel_l2(logits, ref[0]))
        tok_g, tok_r = logits.argmax(-1), ref[0].argmax(-1)
        top = ref[0][0, tok_r[0]]
        margin = float(top - ref[0][0, tok_g[0]])
        assert margin <= float(top.abs()) * 2 ** -7 * 2, f"step {step}: token {int(tok_g)} vs {int(tok_r)}, margin {margin}"
        exact += int(torch.equal(tok_g, tok_r))
        ids = tok_r
    prog.check()
    print(f"greedy tokens identical on {exact}/32 steps; worst rel-L2 {worst:.2e}")
    assert exact >= 31
    assert worst < TOL, worst
    assert int(st["pos"]) == ctx + 32 == int(rs["pos"])
    changed = (st["k_cache"] != k0).any(-1).view(c["n"], max_seq)
    want = torch.zeros_like(changed)
    want[:, ctx:ctx + 32] = True
    assert torch.equal(changed, want)                               # exactly the 32 appended rows per layer
    assert rel_l2(st["k_cache"].float(), rs["k_cache"].float()) < TOL
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 32)


def test_weight_changed_in_place_is_noticed(cuda):
    """Tile-GEMM weights are read from packed snapshots.  A parameter updated in place through torch
    (optimizer step, LoRA merge) moves its version counter; the next call packs again, without
    refresh_weights() and without the tensor's address changing."""
    g = mc.Graph()
    g.output(g.linear(g.input("x", (64, 1024)), g.param("w", (512, 1024))))
    t = {"x": rnd((64, 1024), 1.0, 1), "w": rnd((512, 1024), 0.03, 2)}
    dev = {k: v.to(cuda).contiguous() for k, v in t.items()}
    prog = mc.compile(g)
    a = prog(**dev).float().cpu()
    prog.check()
    assert prog.tcgen05_ops == 1 and prog.packed_weight_bytes == 512 * 1024 * 2
    ref, _ = evaluate(g, t)
    assert rel_l2(a, ref[0]) < TOL
    addr = dev["w"].data_ptr()
    dev["w"].mul_(-0.5)                                  # in place: same address, new version
    assert dev["w"].data_ptr() == addr
    b = prog(**dev).float().cpu()
    prog.check()
    ref2, _ = evaluate(g, dict(t, w=dev["w"].cpu()))
    assert rel_l2(b, ref2[0]) < TOL and rel_l2(b, a) > 1.0
    assert prog.packed_weight_bytes == 512 * 1024 * 2


def test_bind_checks_instruction_arguments(cuda):
    """mk_program_set_ops checks every instruction against the extents its descriptor states: a
    descriptor whose extent has shrunk under the instruction table is refused with MK_E_ARG (and the
    instruction named) before anything reaches the device."""
    import ctypes
    from megacute_b200 import _lib
    g = mc.Graph()
    g.output(g.linear(g.input("x", (200, 256)), g.param("w", (384, 256)), act="relu"))
    dev = {"x": rnd((200, 256), 1.0, 1).to(cuda), "w": rnd((384, 256), 0.05, 2).to(cuda)}
    prog = mc.compile(g)
    good = prog(**dev).clone()
    prog.check()
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    bad = (_lib.OpDesc * len(prog.g.ops))()
    ctypes.memmove(bad, prog._desc, ctypes.sizeof(bad))
    k = next(i for i, o in enumerate(prog.g.ops) if o.kind == "Linear")
    bad[k].i[0] = 100                                    # M = 100: the instruction of m tile 1 now starts past the rows
    rc = lib.mk_program_set_ops(prog._handle, ctypes.addressof(bad), len(prog.g.ops), stream)
    assert rc == -2 and b"m tile" in lib.mk_last_cuda_error()
    again = prog(**dev)                                  # the refused table changed nothing
    prog.check()
    assert torch.equal(again, good)


def test_program_on_another_device_than_the_current_one():
    """A Program is bound to its device; the caller's current device is left alone by every call."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    other = torch.device("cuda", 1)
    g = mc.Graph()
    g.output(g.linear(g.input("x", (64, 512)), g.param("w", (256, 512)), act="gelu_tanh"))
    t = {"x": rnd((64, 512), 1.0, 1), "w": rnd((256, 512), 0.05, 2)}
    torch.cuda.set_device(0)
    prog = mc.compile(g, device=1)
    with torch.cuda.device(other):
        stream_args = {k: v.to(other) for k, v in t.items()}
    out = prog(**stream_args)
    prog.check()
    assert torch.cuda.current_device() == 0 and out.device == other
    ref, _ = evaluate(g, t)
    assert rel_l2(out.float().cpu(), ref[0]) < TOL


@pytest.mark.parametrize("B,vocab", [(1, 5000), (5, 1000), (40, 20000)])
def test_fused_step_feeds_itself(cuda, B, vocab):
    """The decode step as one launch: embedding gather as its first instructions, greedy argmax (column
    chunks merged by the last to arrive) as its last, token ids staying on the device.  Over 32 steps the
    ids the launch leaves equal mk_argmax of the logits it returns, bit for bit, and the logits stay
    within tolerance of the oracle fed the same ids."""
    E, H, KVH, F, n, L, ctx = 256, 4, 2, 512, 2, 256, 60
    g = llama_decode(B, E, H, KVH, F, n, L, vocab, 1e-5, fused_step=True)
    w = W.llama_weights(E, H, KVH, F, n, vocab, 0, "cpu")
    st, ids = W.llama_decode_state(B, E, H, KVH, n, L, ctx, vocab, 1, "cpu")
    del st["x"]
    st["ids"] = ids.to(torch.int32).reshape(B, 1)
    cos, sin = W.rope_tables(L, E // H)
    params = dict(cos=cos, sin=sin, **w)
    prog = mc.compile(g)
    am = [o for o in prog.g.ops if o.kind == "Argmax"]
    assert [o.kind for o in prog.g.ops][0] == "Gather" and len(am) == 1 and (am[0].chunks > 1) == (vocab >= 2048)
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st.items()}
    rs = {k: v.clone() for k, v in st.items()}
    for step in range(32):
        rs["ids"] = ds["ids"].cpu().clone()                  # the oracle follows the tokens the device chose
        logits = prog(**dp, **ds)
        assert torch.equal(ds["ids"].flatten().long(), mc.argmax(logits))
        ref, new = evaluate(g, {**params, **rs})
        assert rel_l2(logits.float().cpu(), ref[0]) < TOL, step
        for name in ("pos", "k_cache", "v_cache"):
            rs[name] = new[name]
    prog.check()
    assert int(ds["pos"]) == ctx + 32
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 32)
    for b in prog.g.buffers:
        if b.kind == "workspace" and b.dtype == torch.int32:
            assert int(prog.buffer(b).abs().sum()) == 0


@pytest.mark.parametrize("M,K,N,act,bias,res", [
    (256, 2048, 512, None, True, True),
    (200, 512, 768, "gelu_tanh", True, False),
    (300, 1024, 1024, "swiglu", False, False),
    (130, 256, 256, "relu", True, True),
    (520, 4096, 256, None, False, True),
    (1100, 512, 1280, None, False, False),
])
def test_tile_linear_wide_tiles(cuda, monkeypatch, M, K, N, act, bias, res):
    """128 x 256 output tiles (one activation k-tile feeds two weight tiles, two accumulator halves in tensor
    memory): plain, swiglu and split-K epilogues, ragged last row tile, several tiles per CTA."""
    monkeypatch.setenv("MEGACUTE_B200_WIDE_TILES", "1")
    g = mc.Graph()
    x = g.input("x", (M, K))
    w = g.param("w", (N, K))
    n_out = N // 2 if act == "swiglu" else N
    h = g.unary(x, "identity")                      # a runtime-owned (fp16) activation, as inside a model
    y = g.linear(h, w, bias=g.param("b", (1, n_out)) if bias else None, act=act,
                 residual=g.input("r", (M, n_out)) if res else None)
    g.output(y)
    t = {"x": rnd((M, K), 1.0, 1), "w": rnd((N, K), 0.03, 2)}
    if bias:
        t["b"] = rnd((1, n_out), 0.5, 4)
    if res:
        t["r"] = rnd((M, n_out), 1.0, 5)
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)
    lin = [o for o in prog.g.ops if o.kind in ("Linear", "LinearSplit")]
    assert lin and all(o.bn == 256 for o in lin) and prog.tcgen05_ops == len(lin)
    assert_close(outs, ref)
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 2)


def test_wide_tiles_many_per_cta_and_slot_kinds(cuda, monkeypatch):
    """Several 128 x 256 tiles per CTA (the weight slots' positions and parities carry over from one instruction to the
    next, and the producer warp fills the next instruction's first slots during this one's epilogue), followed by
    linears that use the ring's memory differently: a narrow-tile one (16 KB slots) and a streaming one (64 KB stages),
    and then wide tiles again -- every change of kind drains the slots of the previous one."""
    monkeypatch.setenv("MEGACUTE_B200_WIDE_TILES", "1")
    M, K = 8192, 512
    g = mc.Graph()
    x = g.input("x", (M, K))
    x2 = g.input("x2", (4, K))
    h = g.unary(x, "identity")
    y1 = g.linear(h, g.param("w1", (1024, K)), act="gelu_tanh")              # wide: 64 x 4 tiles
    y2 = g.linear(h, g.param("w2", (384, K)))                                 # narrow tiles: 384 is no multiple of 256
    s1 = g.linear(x2, g.param("w3", (2048, K)))                               # streaming (4 rows)
    y3 = g.linear(y1, g.param("w4", (512, 1024)), residual=g.input("r", (M, 512)))   # wide again: 64 x 2 tiles, K = 1024
    g.output(y2)
    g.output(s1)
    g.output(y3)
    t = {"x": rnd((M, K), 1.0, 1), "x2": rnd((4, K), 1.0, 2), "w1": rnd((1024, K), 0.04, 3), "w2": rnd((384, K), 0.04, 4),
         "w3": rnd((2048, K), 0.04, 5), "w4": rnd((512, 1024), 0.03, 6), "r": rnd((M, 512), 1.0, 7)}
    outs, ref, _, _, prog = run_both(g, t, cuda, steps=2)
    lin = [o for o in prog.g.ops if o.kind in ("Linear", "LinearSplit")]
    assert sorted(o.bn or 128 for o in lin) == [128, 128, 256, 256] and prog.tcgen05_ops == 3
    assert_close(outs, ref)
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 2)


def _ragged_decode(B, ragged_pos, window, n=2, E=256, H=4, KVH=2, F=512, L=256, V=1024):
    g = llama_decode(B, E, H, KVH, F, n, L, V, 1e-5, ragged=ragged_pos is not None, window=window)
    w = W.llama_weights(E, H, KVH, F, n, V, 0, "cpu")
    st, ids = W.llama_decode_state(B, E, H, KVH, n, L, max(ragged_pos) if ragged_pos else 150, V, 1, "cpu")
    cos, sin = W.rope_tables(L, E // H)
    if ragged_pos is not None:
        st["pos"] = torch.tensor(ragged_pos, dtype=torch.int32).reshape(B, 1)
    st["x"] = w["lm_head"][ids].clone()
    return g, dict(cos=cos, sin=sin, **w), st


@pytest.mark.parametrize("B,bulk", [(1, None), (3, None), (12, None), (33, "0"), (33, "1")])
def test_decode_ragged_positions(cuda, monkeypatch, B, bulk):
    """One position per sequence (pos is a (B, 1) column): every sequence ropes, appends and attends at its own length --
    streaming linears (B <= 8), tile GEMMs, and both forms of the decode attention.  Three steps against the oracle;
    positions, the cache rows written and the dependency counters exact."""
    if bulk:
        monkeypatch.setenv("MEGACUTE_B200_ATT_BULK", bulk)
    gen = torch.Generator().manual_seed(B)
    ps = [int(v) for v in torch.randint(5, 200, (B,), generator=gen)]
    ps[0] = 0                                            # a sequence at its very first token
    g, params, st = _ragged_decode(B, ps, None)
    prog = mc.compile(g)
    assert {bool(o.bulk) for o in prog.g.ops if o.kind == "DecodeAttention"} == {bulk == "1" or (bulk is None and B >= 32)}
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st.items()}
    rs = {k: v.clone() for k, v in st.items()}
    for step in range(3):
        logits = prog(**dp, **ds).float().cpu()
        ref, new = evaluate(g, {**params, **rs})
        assert rel_l2(logits, ref[0]) < TOL, (step, rel_l2(logits, ref[0]))
        for n_ in ("pos", "k_cache", "v_cache"):
            rs[n_] = new[n_]
        rs["x"] = params["lm_head"][ref[0].argmax(-1)].clone()
        ds["x"].copy_(rs["x"].to(cuda))
    prog.check()
    assert ds["pos"].flatten().tolist() == [p + 3 for p in ps]
    kc, rk = ds["k_cache"].cpu().float(), rs["k_cache"].float()
    changed = (kc != st["k_cache"].float()).any(-1).reshape(2, B, 256)
    want = torch.zeros_like(changed)
    for b, p in enumerate(ps):
        want[:, b, p:p + 3] = True
    assert torch.equal(changed, want) and rel_l2(kc, rk) < TOL
    assert np.array_equal(prog.counters(), prog.sched.counter_target * 3)


@pytest.mark.parametrize("B,window,ragged", [(1, 32, False), (2, 100, False), (5, 17, True), (12, 64, True), (2, 1000, False)])
def test_decode_sliding_window(cuda, B, window, ragged):
    """Sliding-window attention: a sequence attends its last `window` tokens (the new one included), whatever the split
    count; with one position for the batch and with one per sequence; a window beyond the context changes nothing."""
    ps = [150 - 13 * b for b in range(B)] if ragged else None
    g, params, st = _ragged_decode(B, ps, window)
    prog = mc.compile(g)
    dp = {k: v.to(cuda) for k, v in params.items()}
    ds = {k: v.to(cuda) for k, v in st.items()}
    rs = {k: v.clone() for k, v in st.items()}
    for step in range(2):
        logits = prog(**dp, **ds).float().cpu()
        ref, new = evaluate(g, {**params, **rs})
        assert rel_l2(logits, ref[0]) < TOL, (step, rel_l2(logits, ref[0]))
        for n_ in ("pos", "k_cache", "v_cache"):
            rs[n_] = new[n_]
        rs["x"] = params["lm_head"][ref[0].argmax(-1)].clone()
        ds["x"].copy_(rs["x"].to(cuda))
    prog.check()
    if window < 100:                                     # the window matters: the full-context result differs
        full, _ = evaluate(llama_decode(B, 256, 4, 2, 512, 2, 256, 1024, 1e-5, ragged=ragged), {**params, **st})
        win, _ = evaluate(g, {**params, **st})
        assert rel_l2(win[0], full[0]) > 1e-3
