"""Graph builders for the benchmarked workloads, written against the public Graph API.

They produce the same op sequences as the reference's example builders
(``examples/llama/model.py:20-80`` llama_stack / llama_decode, ``examples/dit/model.py:20-50``
dit_stack, and the MLP block of ``README.md:14-20``); tests check that the reference's own builder
files, imported unchanged, yield identical graphs.  Per-layer parameters are stacked along rows:
layer ``i`` of a parameter with ``r`` rows per layer is rows ``[i*r, (i+1)*r)``.
"""

from __future__ import annotations

import torch

from .graph import Graph


def llama_param_shapes(E: int, H: int, KVH: int, F: int) -> dict:
    D = E // H
    return {"attn_norm": (1, E), "wqkv": ((H + 2 * KVH) * D, E), "wo": (E, E), "mlp_norm": (1, E),
            "wgu": (2 * F, E), "wd": (E, F)}


def _stacked(g: Graph, shapes: dict, n: int):
    whole = {k: g.param(k, (n * r, c)) for k, (r, c) in shapes.items()}
    return lambda i: {k: whole[k].rows_slice(i * r, r) for k, (r, _) in shapes.items()}


def mlp_block(M: int, E: int = 2048, F: int = 5632, eps: float = 1e-5) -> Graph:
    """y = linear(linear(rms_norm(x, nw), w1, act="swiglu"), w2, residual=x)."""
    g = Graph()
    x = g.input("x", (M, E))
    nw = g.param("nw", (1, E))
    w1 = g.param("w1", (2 * F, E))
    w2 = g.param("w2", (E, F))
    h = g.linear(g.rms_norm(x, nw, eps), w1, act="swiglu")
    g.output(g.linear(h, w2, residual=x))
    return g


def llama_stack(B: int, S: int, E: int, H: int, KVH: int, F: int, n: int, eps: float = 1e-6,
                vocab: int | None = None) -> Graph:
    """Prefill: n pre-norm decoder blocks over B prompts of S tokens; x is (B*S, E), cos/sin (S, D).
    With ``vocab`` the graph also applies the final norm and the lm_head to the last token of each
    prompt and returns (B, vocab) logits instead of the residual stream."""
    D = E // H
    g = Graph()
    x = g.input("x", (B * S, E))
    cos, sin = g.input("cos", (S, D)), g.input("sin", (S, D))
    layer = _stacked(g, llama_param_shapes(E, H, KVH, F), n)
    for i in range(n):
        g.layer = i
        p = layer(i)
        qkv = g.linear(g.rms_norm(x, p["attn_norm"], eps), p["wqkv"])
        q = g.rope(qkv.cols_slice(0, E), cos, sin, heads=H, head_dim=D, seq=S)
        k = g.rope(qkv.cols_slice(E, KVH * D), cos, sin, heads=KVH, head_dim=D, seq=S)
        v = qkv.cols_slice(E + KVH * D, KVH * D)
        a = g.attention(q, k, v, batch=B, heads=H, head_dim=D, causal=True, kv_heads=KVH)
        x = g.linear(a, p["wo"], residual=x)
        x = g.linear(g.linear(g.rms_norm(x, p["mlp_norm"], eps), p["wgu"], act="swiglu"), p["wd"], residual=x)
    g.layer = None
    if vocab:
        fw, head = g.param("final_norm", (1, E)), g.param("lm_head", (vocab, E))
        last = g.temp((B, E), name="last_tokens")
        for b in range(B):
            g.unary(x.rows_slice(b * S + S - 1, 1), "identity", out=last.rows_slice(b, 1))
        x = g.linear(g.rms_norm(last, fw, eps), head)
    g.output(x)
    return g


def llama_decode(B: int, E: int, H: int, KVH: int, F: int, n: int, max_seq: int, vocab: int | None = None,
                 eps: float = 1e-6, fused_step: bool = False, ragged: bool = False, window: int | None = None) -> Graph:
    """One decode step for B sequences.  States: x (B, E) embedded tokens, pos (1, 1) int32,
    k_cache / v_cache (n*B*max_seq, KVH*D) with layer i at rows [i*B*max_seq, ...) and sequence b of
    it at [b*max_seq, ...).  Output: (B, vocab) logits, or the hidden state without ``vocab``.

    ``fused_step`` (needs ``vocab``; tied embeddings) puts the two ends of the step inside the launch:
    the state is ``ids`` (B, 1) int32 instead of x -- the launch gathers the embedding rows itself and
    overwrites ids with the greedy tokens, so a decode loop is one launch per step with nothing
    around it (the reference's step is index_select + copy_ + launch + argmax,
    examples/llama/llama1b.py:103-105).

    ``ragged``: pos is (B, 1), one position per sequence, so sequences of different lengths decode in
    one batch; ``window``: sliding-window attention over each sequence's last ``window`` tokens.  (The
    reference has neither: README.md:225-228.)"""
    D = E // H
    g = Graph()
    if fused_step:
        assert vocab, "fused_step samples from the logits: it needs the lm_head"
        ids = g.state("ids", (B, 1), torch.int32)
        head = g.param("lm_head", (vocab, E))
        x = g.gather(head, ids)
    else:
        x = g.state("x", (B, E))
    cos, sin = g.input("cos", (max_seq, D)), g.input("sin", (max_seq, D))
    pos = g.state("pos", (B if ragged else 1, 1), torch.int32)
    kc = g.state("k_cache", (n * B * max_seq, KVH * D))
    vc = g.state("v_cache", (n * B * max_seq, KVH * D))
    layer = _stacked(g, llama_param_shapes(E, H, KVH, F), n)
    R = B * max_seq
    for i in range(n):
        g.layer = i
        p = layer(i)
        kci, vci = kc.rows_slice(i * R, R), vc.rows_slice(i * R, R)
        qkv = g.linear(g.rms_norm(x, p["attn_norm"], eps), p["wqkv"])
        q = g.rope_append(qkv, cos, sin, pos, kci, vci, heads=H, kv_heads=KVH, head_dim=D, max_seq=max_seq)
        a = g.decode_attention(q, kci, vci, pos, heads=H, kv_heads=KVH, head_dim=D, max_seq=max_seq, window=window)
        x = g.linear(a, p["wo"], residual=x)
        x = g.linear(g.linear(g.rms_norm(x, p["mlp_norm"], eps), p["wgu"], act="swiglu"), p["wd"], residual=x)
    g.layer = None
    if vocab:
        x = g.linear(g.rms_norm(x, g.param("final_norm", (1, E)), eps), head if fused_step else g.param("lm_head", (vocab, E)))
    if fused_step:
        g.argmax(x, ids)
    g.increment(pos)
    g.output(x)
    return g


def dit_param_shapes(E: int, F: int) -> dict:
    return {"w_ada": (6 * E, E), "b_ada": (1, 6 * E), "wqkv": (3 * E, E), "bqkv": (1, 3 * E), "wo": (E, E),
            "bo": (1, E), "w1": (F, E), "b1": (1, F), "w2": (E, F), "b2": (1, E)}


def dit_stack(B: int, S: int, E: int, H: int, F: int, n: int, eps: float = 1e-6) -> Graph:
    """n DiT blocks with adaLN-Zero conditioning; x (B*S, E), c (B, E).  Per block:
    mod = linear(silu(c)) -> shift/scale/gate for attention and MLP; gated residuals."""
    D = E // H
    g = Graph()
    x = g.input("x", (B * S, E))
    c = g.input("c", (B, E))
    sc = g.unary(c, "silu")
    layer = _stacked(g, dit_param_shapes(E, F), n)
    for i in range(n):
        g.layer = i
        p = layer(i)
        mod = g.linear(sc, p["w_ada"], bias=p["b_ada"])
        sh1, sc1, gt1, sh2, sc2, gt2 = (mod.cols_slice(j * E, E) for j in range(6))
        h = g.modulate(g.layer_norm(x, eps=eps), sc1, sh1, group=S)
        qkv = g.linear(h, p["wqkv"], bias=p["bqkv"])
        a = g.attention(qkv.cols_slice(0, E), qkv.cols_slice(E, E), qkv.cols_slice(2 * E, E), batch=B, heads=H,
                        head_dim=D, causal=False)
        o = g.linear(a, p["wo"], bias=p["bo"])
        x = g.add(x, g.binary(o, gt1, "mul", b_group=S))
        h = g.modulate(g.layer_norm(x, eps=eps), sc2, sh2, group=S)
        m = g.linear(g.linear(h, p["w1"], bias=p["b1"], act="gelu_tanh"), p["w2"], bias=p["b2"])
        x = g.add(x, g.binary(m, gt2, "mul", b_group=S))
    g.layer = None
    g.output(x)
    return g
