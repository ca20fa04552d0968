"""CPU tests of the N > 1 path: two gloo ranks shard a decode batch, each evaluates its own sequences,
and the pieces equal the unsharded evaluation (sequences never interact, so no data-path collective
is needed); the timing reductions return the slowest rank's time on every rank."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from megacute_b200 import workloads as W
from megacute_b200.builders import llama_decode
from megacute_b200.sharding import job_throughput, max_over_ranks, shard_range
from oracle.graph_oracle import evaluate

CFG = dict(E=256, H=4, KVH=2, F=512, n=2, vocab=512, eps=1e-5)
TOTAL, CTX, MAX_SEQ = 6, 20, 128


def test_shard_range_partitions_exactly():
    for total in (0, 1, 7, 64, 513):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s1 == s0 + c0
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _inputs(B, seed_state):
    w = W.llama_weights(CFG["E"], CFG["H"], CFG["KVH"], CFG["F"], CFG["n"], CFG["vocab"], 0, "cpu")
    st, ids = W.llama_decode_state(B, CFG["E"], CFG["H"], CFG["KVH"], CFG["n"], MAX_SEQ, CTX, CFG["vocab"], seed_state, "cpu")
    cos, sin = W.rope_tables(MAX_SEQ, CFG["E"] // CFG["H"])
    return w, st, ids, cos, sin


def _decode(B, w, st, ids, cos, sin):
    g = llama_decode(B, CFG["E"], CFG["H"], CFG["KVH"], CFG["F"], CFG["n"], MAX_SEQ, CFG["vocab"], CFG["eps"])
    st = dict(st, x=w["lm_head"][ids].clone())
    out, new = evaluate(g, dict(cos=cos, sin=sin, **w, **st))
    return out[0], new


def _slice_state(st, start, count):
    out = {}
    for name, t in st.items():
        if name == "pos":
            out[name] = t.clone()
        elif name == "x":
            out[name] = t[start:start + count].clone()
        else:                                   # caches: (layers * B * max_seq, KVH * D), layer-major then sequence
            out[name] = _cache_rows(t, start, count).clone()
    return out


def _cache_rows(t, start, count):
    n = CFG["n"]
    return t.view(n, TOTAL, MAX_SEQ, -1)[:, start:start + count].reshape(n * count * MAX_SEQ, -1)


def _rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        w, st, ids, cos, sin = _inputs(TOTAL, 1)
        start, count = shard_range(TOTAL, world, rank)
        logits, new = _decode(count, w, _slice_state(st, start, count), ids[start:start + count], cos, sin)
        slowest = max_over_ranks(10.0 + rank)                 # rank 1 is the slow one
        tput = job_throughput(count, 10.0 + rank)
        ret[rank] = (start, count, logits, {k: v for k, v in new.items() if k != "pos"}, int(new["pos"]), slowest, tput)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_equal_the_unsharded_batch():
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_rank, args=(world, port, ret), nprocs=world, join=True)
    w, st, ids, cos, sin = _inputs(TOTAL, 1)
    want, want_state = _decode(TOTAL, w, st, ids, cos, sin)
    covered = 0
    for r in range(world):
        start, count, logits, new, pos, slowest, tput = ret[r]
        assert (start, count) == shard_range(TOTAL, world, r)
        assert torch.equal(logits, want[start:start + count])            # same arithmetic, same order: bit-exact
        for name in ("k_cache", "v_cache"):
            assert torch.equal(new[name], _cache_rows(want_state[name], start, count)), name
        assert pos == CTX + 1
        assert slowest == 11.0                                             # MAX over ranks, on every rank
        assert tput == pytest.approx(TOTAL * 1e3 / 11.0)
        covered += count
    assert covered == TOTAL
