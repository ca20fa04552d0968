"""CPU tests of the host side: graph API, passes, scheduler invariants, encoding."""
import numpy as np
import pytest
import torch

import megacute_b200 as mc
from megacute_b200 import config as C
from megacute_b200.builders import dit_stack, llama_decode, llama_stack, mlp_block
from megacute_b200.passes import fold_norms, fuse_rope_attention, run_all, split_k, split_kv
from megacute_b200.schedule import schedule
from megacute_b200.verify import VerifyError, check_hazards, check_tables
from oracle.graph_oracle import evaluate, rel_l2
from tests.helpers import small_decode

BF = torch.bfloat16


def test_api_surface_and_errors():
    g = mc.Graph()
    x = g.input("x", (16, 64))
    w = g.param("w", (128, 64))
    with pytest.raises(TypeError):
        g.input("bad", (4, 8), torch.float16)
    with pytest.raises(ValueError):
        g.input("odd", (4, 7))                      # row stride not 16-byte aligned
    with pytest.raises(ValueError):
        x.cols_slice(60, 8)                          # out of bounds
    with pytest.raises(ValueError):
        g.unary(x, "relu", out=g.param("ro", (16, 64)))   # writes a param
    with pytest.raises(AssertionError):
        g.linear(x, g.param("w2", (128, 32)))        # K mismatch
    y = g.linear(x, w, act="swiglu")
    assert y.shape == (16, 64)
    g.output(y)
    assert y.buf.kind == "output" and "Linear" in repr(g)
    assert mc.schedule is not None and mc.View is not None and mc.Buffer is not None


def test_swiglu_weight_layout():
    gate = torch.arange(128 * 8, dtype=torch.float32).reshape(128, 8)
    up = -gate
    w = mc.swiglu_weight(gate, up)
    assert w.shape == (256, 8)
    assert torch.equal(w[0:64], gate[0:64]) and torch.equal(w[64:128], up[0:64])
    assert torch.equal(w[128:192], gate[64:128]) and torch.equal(w[192:256], up[64:128])


@pytest.mark.parametrize("B", [1, 3, 16])
def test_passes_preserve_semantics_decode(B):
    g, params, st, _ = small_decode(B=B)
    ref_out, ref_st = evaluate(g, {**params, **st})
    for sm in (8, 148):
        g2 = run_all(g, sm)
        out, st2 = evaluate(g2, {**params, **st})
        assert rel_l2(out[0], ref_out[0]) < 1e-5
        assert int(st2["pos"]) == int(ref_st["pos"]) == int(st["pos"]) + 1
        assert torch.equal(st2["k_cache"], ref_st["k_cache"]) and torch.equal(st2["v_cache"], ref_st["v_cache"])
    kinds = [o.kind for o in run_all(g, 148).ops]
    assert "RopeAppend" not in kinds                                  # fused into DecodeAttention
    if B <= C.GEMV_MAX_ROWS:
        assert "Norm" not in kinds                                    # folded into the linears


def test_fold_and_fuse_conditions():
    g, *_ = small_decode(B=1, max_seq=1024)            # long enough for the KV split to pay
    f = fold_norms(g)
    assert sum(o.kind == "Norm" for o in f.ops) == 0
    assert all(o.rms_eps is not None for o in f.ops if o.kind == "Linear" and o.norm_w is not None)
    fused = fuse_rope_attention(f)
    att = [o for o in fused.ops if o.kind == "DecodeAttention"]
    assert all(o.k_new is not None and o.cos is not None for o in att)
    s = split_kv(fused, 148)
    att = [o for o in s.ops if o.kind == "DecodeAttention"]
    assert all(o.splits > 1 and o.part is not None and o.count is not None for o in att)
    # a norm whose output is a graph output must stay
    g2 = mc.Graph()
    x = g2.input("x", (1, 64))
    n = g2.rms_norm(x, g2.param("nw", (1, 64)))
    g2.output(g2.linear(n, g2.param("w", (64, 64))), n)
    assert any(o.kind == "Norm" for o in fold_norms(g2).ops)


def test_split_k_mlp_block():
    g = mlp_block(256)
    g2 = split_k(fold_norms(g), 148)
    kinds = [o.kind for o in g2.ops]
    assert kinds == ["Norm", "Linear", "LinearSplit", "SplitFinalize"]
    x = torch.randn(256, 2048).to(BF)
    t = dict(x=x, nw=torch.ones(1, 2048).to(BF), w1=(torch.randn(11264, 2048) * 0.02).to(BF),
             w2=(torch.randn(2048, 5632) * 0.02).to(BF))
    a, _ = evaluate(g, t)
    b, _ = evaluate(g2, t)
    assert rel_l2(b[0], a[0]) < 1e-5


def _check_schedule(s, g):
    n = s.n
    # every dependency points backwards; counters reach exactly their target per launch
    arrivals = np.bincount(s.arr_cnt, minlength=s.num_counters)
    assert np.array_equal(arrivals, s.counter_target)
    first_arrive = np.full(s.num_counters, n, np.int64)
    last_arrive = np.full(s.num_counters, -1, np.int64)
    for i in range(n):
        for c in s.arr_cnt[s.arr_ptr[i]:s.arr_ptr[i + 1]]:
            first_arrive[c] = min(first_arrive[c], i)
            last_arrive[c] = max(last_arrive[c], i)
    for i in range(n):
        for c, t in zip(s.wait_cnt[s.wait_ptr[i]:s.wait_ptr[i + 1]], s.wait_tgt[s.wait_ptr[i]:s.wait_ptr[i + 1]]):
            assert last_arrive[c] < i and t == s.counter_target[c]
    ins, waits, arrives = s.encode()
    assert ins.shape == (n, C.IW) and ins.dtype == torch.int32
    assert int(ins[:, C.W_OP].min()) >= 1 and int(ins[:, C.W_OP].max()) == len(g.ops)
    assert int(ins[:, C.W_NARRIVE].sum()) == len(s.arr_cnt) and int(ins[:, C.W_NWAIT].sum()) == len(s.wait_cnt)


def _simulate(s, g, order_seed):
    """Execute the stream in a random counter-legal order with `grid` in-order CTAs: some CTA can
    always make progress and every instruction runs (no deadlock).  That every conflicting pair of
    accesses is ORDERED is not decided by sampling executions but exactly, by `_ordered` below."""
    rng = np.random.default_rng(order_seed)
    grid = s.sm_count
    counters = np.zeros(s.num_counters, np.int64)
    nxt = list(range(min(grid, s.n)))                # next instruction of each CTA
    done_order = []
    live = set(range(len(nxt)))
    while live:
        ready = [c for c in live if all(counters[cn] >= t for cn, t in
                                        zip(s.wait_cnt[s.wait_ptr[nxt[c]]:s.wait_ptr[nxt[c] + 1]],
                                            s.wait_tgt[s.wait_ptr[nxt[c]]:s.wait_ptr[nxt[c] + 1]]))]
        assert ready, "deadlock: no CTA can make progress"
        c = ready[rng.integers(len(ready))]
        i = nxt[c]
        done_order.append(i)
        counters[s.arr_cnt[s.arr_ptr[i]:s.arr_ptr[i + 1]]] += 1
        nxt[c] += grid
        if nxt[c] >= s.n:
            live.discard(c)
    assert sorted(done_order) == list(range(s.n))       # every instruction ran: no deadlock in this order


def _ordered(s, g):
    """Tables of a schedule are complete: arguments and operand windows in range, and every hazard
    ordered in the happens-before closure of the wait / arrival tables."""
    check_tables(g, s)
    assert check_hazards(s, g) > 0


def test_finalize_fused_into_decode_attention():
    """Batched decode: the split-K QKV projection's SplitFinalize (a plain fp32 copy) is dropped, the
    fused attention reads the workspace and zeroes it; every hazard on the workspace stays ordered."""
    g, *_ = small_decode(B=16, n=2, E=2048, H=32, KVH=8, F=1024, vocab=512, max_seq=128, ctx=10)
    g2 = run_all(g, 148)
    att = [o for o in g2.ops if o.kind == "DecodeAttention"]
    assert att and all(o.zero_inputs and o.q.buf.kind == "workspace" and o.q.buf is o.k_new.buf is o.v_new.buf for o in att)
    fins = [o for o in g2.ops if o.kind == "SplitFinalize"]
    assert not any(o.out.buf is a.q.buf for o in fins for a in att)
    for a in att:                                                     # a split-K QKV projection accumulates there
        assert any(o.kind == "LinearSplit" and o.ws.buf is a.q.buf for o in g2.ops)
    s = schedule(g2, 148)
    _check_schedule(s, g2)
    _simulate(s, g2, 0)
    _ordered(s, g2)
    g1, *_ = small_decode(B=1)
    assert not any(o.zero_inputs for o in run_all(g1, 148).ops if o.kind == "DecodeAttention")


def test_many_sequence_attention_choice_and_schedule(monkeypatch):
    """From 32 sequences on (8 with long caches) the decode attention runs in its many-sequence form:
    one instruction per (sequence, KV split) over all kv heads, split count from the context length;
    the schedule of such a graph orders every hazard, partial-row and arrival-count workspaces included."""
    from megacute_b200.passes import bulk_kv_splits
    assert bulk_kv_splits(64, 8, 1152, 148) == 2 and bulk_kv_splits(64, 8, 32896, 148) > 4
    for B, splits in ((40, None), (16, "3")):
        if splits:
            monkeypatch.setenv("MEGACUTE_B200_KV_SPLITS", splits)
            monkeypatch.setenv("MEGACUTE_B200_ATT_BULK", "1")
        g, *_ = small_decode(B=B, n=2, E=512, H=8, KVH=8, F=512, vocab=512, max_seq=256, ctx=10)
        g2 = run_all(g, 148)
        att = [o for o in g2.ops if o.kind == "DecodeAttention"]
        assert att and all(o.bulk and o.heads_per_inst == 8 for o in att)
        if splits:
            assert all(o.splits == 3 and o.part.rows == B * 8 * 3 for o in att)
        s = schedule(g2, 148)
        assert s.node_ranges[g2.ops.index(att[0])][1] - s.node_ranges[g2.ops.index(att[0])][0] == B * att[0].splits
        _check_schedule(s, g2)
        _simulate(s, g2, 0)
        _ordered(s, g2)
    monkeypatch.delenv("MEGACUTE_B200_ATT_BULK")
    monkeypatch.delenv("MEGACUTE_B200_KV_SPLITS")
    for B, L, want in ((2, 256, False), (16, 256, False), (16, 8192, True), (32, 256, True)):
        gb, *_ = small_decode(B=B, n=1, max_seq=L)
        assert all(bool(o.bulk) == want for o in run_all(gb, 148).ops if o.kind == "DecodeAttention"), (B, L)


def test_kv_heads_per_instruction_choice_and_schedule(monkeypatch):
    """The per-head form with more (sequence, kv head) pairs than SMs: several kv heads per attention
    instruction; the schedule of such a graph still orders every hazard."""
    from megacute_b200.passes import kv_heads_per_instruction
    monkeypatch.setenv("MEGACUTE_B200_ATT_BULK", "0")
    assert kv_heads_per_instruction(512, 8, 1280, 148) == 4            # batch 64 of the 1B shape: one wave of 128
    assert kv_heads_per_instruction(128, 8, 1280, 148) == 1            # fewer pairs than SMs: nothing to amortise over
    g, *_ = small_decode(B=40, n=1, E=512, H=8, KVH=8, F=512, vocab=512, max_seq=128, ctx=10)
    g2 = run_all(g, 148)
    att = [o for o in g2.ops if o.kind == "DecodeAttention"]
    assert att and all(o.heads_per_inst > 1 and o.splits == 1 for o in att)
    s = schedule(g2, 148)
    _check_schedule(s, g2)
    _simulate(s, g2, 0)
    _ordered(s, g2)


def test_schedule_invariants_decode():
    for B, sm in ((1, 148), (16, 148), (2, 8)):
        g, *_ = small_decode(B=B)
        g2 = run_all(g, sm)
        s = schedule(g2, sm)
        _check_schedule(s, g2)
        _ordered(s, g2)


def test_schedule_orders_every_hazard():
    g, *_ = small_decode(B=1, n=2, E=128, H=2, KVH=1, F=256, vocab=256, max_seq=128, ctx=10)
    g2 = run_all(g, 6)
    s = schedule(g2, 6)
    _simulate(s, g2, 0)
    _ordered(s, g2)
    m = run_all(mlp_block(256, 256, 512), 6)
    sm_ = schedule(m, 6)
    _simulate(sm_, m, 0)
    _ordered(sm_, m)
    for build in (lambda: llama_stack(2, 256, 256, 4, 2, 512, 2, vocab=512), lambda: dit_stack(2, 64, 128, 2, 256, 2)):
        gg = run_all(build(), 16)
        _ordered(schedule(gg, 16), gg)


def test_verifier_catches_a_dropped_wait_and_a_bad_argument():
    """The checks fail when the tables are wrong: remove one wait (an unordered hazard appears), move
    a tile index outside its op, shrink an operand below the window the kernel addresses."""
    import copy
    g, *_ = small_decode(B=1, n=1, E=128, H=2, KVH=1, F=256, vocab=256, max_seq=128, ctx=10)
    g2 = run_all(g, 6)
    s = schedule(g2, 6)
    _ordered(s, g2)
    # drop the only wait of the first instruction that has exactly one
    one = [i for i in range(s.n) if s.wait_ptr[i + 1] - s.wait_ptr[i] == 1 and i >= 6]
    assert one
    hit = 0
    for i in one[:8]:
        bad = copy.copy(s)
        keep = np.ones(len(s.wait_cnt), bool)
        keep[s.wait_ptr[i]] = False
        bad.wait_cnt, bad.wait_tgt = s.wait_cnt[keep], s.wait_tgt[keep]
        bad.wait_ptr = s.wait_ptr.copy()
        bad.wait_ptr[i + 1:] -= 1
        try:
            check_hazards(bad, g2)
        except VerifyError:
            hit += 1
    assert hit > 0                                   # (a wait may be redundant through another chain; not all of them are)
    bad = copy.copy(s)
    bad.args = s.args.copy()
    k = next(k for k, o in enumerate(g2.ops) if o.kind == "DecodeAttention")
    bad.args[s.node_ranges[k][0], 1] = 7            # kv head 7 of 1
    with pytest.raises(VerifyError):
        check_tables(g2, bad)
    op = g2.ops[k]
    g3 = copy.copy(g2)
    g3.ops = list(g2.ops)
    g3.ops[k] = copy.copy(op)
    g3.ops[k].k_cache = op.k_cache.rows_slice(0, op.k_cache.rows - 1)     # one row short of batch * max_seq
    with pytest.raises(VerifyError):
        check_tables(g3, s)


def test_timeline_reports_on_synthetic_records():
    """Timeline is pure host code over the trace buffer: feed it records and check every report."""
    from megacute_b200.trace import Timeline

    class FakeProg:
        pass
    g, *_ = small_decode(B=1, n=1, E=128, H=2, KVH=1, F=256, vocab=256, max_seq=128, ctx=10)
    prog = FakeProg()
    prog.g = run_all(g, 4)
    prog.sched = schedule(prog.g, 4)
    prog.node_of = [(k, 0) for k in range(len(prog.g.ops))]
    prog.nodes = [[o] for o in prog.g.ops]
    cap = -(-prog.sched.n // 4)
    buf = np.zeros((4, 3, cap, 4), np.int64)
    t = 1000
    for i in range(prog.sched.n):
        sm, slot = i % 4, i // 4
        buf[sm, 1, slot] = (i, t, t + 100 * (i % 3), t + 500)
        if i % 5 == 0:
            buf[sm, 0, slot] = (i, t - 50, t - 50, t + 20)
        t += 37
    tl = Timeline(prog, buf)
    comp = [r for r in tl.records if r[1] == 1]
    assert len(comp) == prog.sched.n and all(isinstance(x, int) for x in comp[0])
    assert tl.t_base == 950 and abs(tl.span_us() - (t - 37 + 500 - 950) / 1e3) < 1e-9
    tab = tl.node_table()
    assert int(tab["insts"].sum()) == prog.sched.n and (tab["end"] >= tab["start"]).all()
    text = tl.summary()
    assert "Linear" in text and f"{prog.sched.n} instructions traced" in text
    ev = tl.chrome_events()
    waits = sum(1 for i in range(prog.sched.n) if i % 3)
    assert len(ev) == prog.sched.n + waits + sum(1 for i in range(prog.sched.n) if i % 5 == 0)
    assert {e["tid"] for e in ev} == {"producer", "compute"} and all(e["dur"] >= 0 for e in ev)


def test_schedule_sizes_baseline_configs():
    g = llama_decode(1, 2048, 32, 8, 8192, 16, 1152, 128256, 1e-5)
    s = schedule(run_all(g, 148), 148)
    assert s.n < 13000 and int(np.diff(s.wait_ptr).max()) <= 16
    _check_schedule(s, run_all(g, 148))
    _ordered(s, run_all(g, 148))
    # batch 64 at full size (split-K tile GEMMs, workspace-fed attention, several kv heads per instruction)
    g64 = run_all(llama_decode(64, 2048, 32, 8, 8192, 16, 1152, 128256, 1e-5), 148)
    _ordered(schedule(g64, 148), g64)


def test_builders_prefill_and_dit_schedule():
    g = llama_stack(2, 256, 256, 4, 2, 512, 2, vocab=512)
    s = schedule(run_all(g, 16), 16)
    _check_schedule(s, run_all(g, 16))
    d = dit_stack(2, 64, 128, 2, 256, 2)
    s = schedule(run_all(d, 16), 16)
    _check_schedule(s, run_all(d, 16))


def test_fused_step_graph_and_oracle():
    """gather / argmax (the two ends of a decode step inside the launch): oracle semantics, the pass that
    cuts the argmax into column chunks, and a schedule that orders the ids hazard (gather reads the ids
    the argmax overwrites)."""
    from megacute_b200 import workloads as W
    B, vocab = 3, 4096
    g = llama_decode(B, 256, 4, 2, 512, 2, 256, vocab, 1e-5, fused_step=True)
    assert [b.name for b in g.states] == ["ids", "pos", "k_cache", "v_cache"]
    w = W.llama_weights(256, 4, 2, 512, 2, vocab, 0, "cpu")
    st, ids = W.llama_decode_state(B, 256, 4, 2, 2, 256, 40, vocab, 1, "cpu")
    cos, sin = W.rope_tables(256, 64)
    x = st.pop("x")
    st["ids"] = ids.to(torch.int32).reshape(B, 1)
    out, new = evaluate(g, dict(cos=cos, sin=sin, **w, **st))
    plain = llama_decode(B, 256, 4, 2, 512, 2, 256, vocab, 1e-5)
    out0, _ = evaluate(plain, dict(cos=cos, sin=sin, **w, **st, x=w["lm_head"][ids].clone()))
    assert torch.equal(out[0], out0[0])                               # gather == the embedding lookup done outside
    assert torch.equal(new["ids"].flatten().long(), out[0].argmax(-1)) and new["ids"].dtype == torch.int32
    g2 = run_all(g, 148)
    am = [o for o in g2.ops if o.kind == "Argmax"]
    assert len(am) == 1 and am[0].chunks == 4 and am[0].part.shape == (B, 8)
    out2, new2 = evaluate(g2, dict(cos=cos, sin=sin, **w, **st))
    assert torch.equal(new2["ids"], new["ids"])
    s = schedule(g2, 148)
    _check_schedule(s, g2)
    _simulate(s, g2, 0)
    _ordered(s, g2)
    with pytest.raises(AssertionError):
        mc.Graph().gather(g.params[0].full, g.states[2].full)        # ids must be an int32 column


def test_ragged_positions_and_window_semantics():
    """The oracle's reading of the two decode extensions: a ragged batch equals its sequences run one by one at their own
    positions, and passes keep it; a windowed decode attention equals a plain softmax over the window's cache rows."""
    import torch
    import megacute_b200 as mc
    from megacute_b200 import workloads as W
    from megacute_b200.builders import llama_decode
    from megacute_b200.passes import run_all
    from oracle.graph_oracle import evaluate, rel_l2
    B, E, H, KVH, F, n, L, V = 3, 256, 4, 2, 512, 2, 256, 512
    w = W.llama_weights(E, H, KVH, F, n, V, 0, "cpu")
    st, ids = W.llama_decode_state(B, E, H, KVH, n, L, 60, V, 1, "cpu")
    cos, sin = W.rope_tables(L, E // H)
    ps = [17, 60, 33]
    st["pos"] = torch.tensor(ps, dtype=torch.int32).reshape(B, 1)
    st["x"] = w["lm_head"][ids].clone()
    g = llama_decode(B, E, H, KVH, F, n, L, V, ragged=True)
    out, new = evaluate(g, dict(cos=cos, sin=sin, **w, **st))
    out2, _ = evaluate(run_all(g, 148), dict(cos=cos, sin=sin, **w, **{k: v.clone() for k, v in st.items()}))
    assert rel_l2(out2[0], out[0]) < 1e-6
    assert new["pos"].flatten().tolist() == [p + 1 for p in ps]
    g1 = llama_decode(1, E, H, KVH, F, n, L, V)
    for b in range(B):
        pick = lambda c: c.reshape(n, B, L, -1)[:, b].reshape(n * L, -1).clone()
        st1 = {"x": st["x"][b:b + 1].clone(), "pos": torch.tensor([[ps[b]]], dtype=torch.int32),
               "k_cache": pick(st["k_cache"]), "v_cache": pick(st["v_cache"])}
        o1, _ = evaluate(g1, dict(cos=cos, sin=sin, **w, **st1))
        assert rel_l2(out[0][b:b + 1], o1[0]) < 1e-5
    # the window, on the attention op alone
    D, window = E // H, 20
    ga = mc.Graph()
    q = ga.input("q", (B, H * D))
    kc, vc = ga.state("k_cache", (B * L, KVH * D)), ga.state("v_cache", (B * L, KVH * D))
    pos = ga.state("pos", (B, 1), torch.int32)
    ga.output(ga.decode_attention(q, kc, vc, pos, heads=H, kv_heads=KVH, head_dim=D, max_seq=L, window=window))
    t = {"q": torch.randn(B, H * D).bfloat16(), "k_cache": torch.randn(B * L, KVH * D).bfloat16(), "v_cache": torch.randn(B * L, KVH * D).bfloat16(),
         "pos": st["pos"].clone()}
    got, _ = evaluate(ga, t)
    for b in range(B):
        lo = max(0, ps[b] + 1 - window)
        k = t["k_cache"].float().reshape(B, L, KVH, D)[b, lo:ps[b] + 1]
        v = t["v_cache"].float().reshape(B, L, KVH, D)[b, lo:ps[b] + 1]
        qq = t["q"].float()[b].reshape(KVH, H // KVH, D)
        sc = torch.einsum("kgd,skd->kgs", qq, k) * D ** -0.5
        want = torch.einsum("kgs,skd->kgd", torch.softmax(sc, -1), v).reshape(1, H * D)
        assert rel_l2(got[0][b:b + 1], want) < 1e-5
