"""The checkpoint runner's offline parts: Hugging Face weight re-layout, Llama-3 RoPE scaling, generate loop.

No checkpoint is available offline, so the tests build a small random state dict with Hugging Face's
tensor names and compare against a plain fp32 implementation of the Llama forward pass written here in
Hugging Face's conventions (separate q / k / v / gate / up projections, rotate-half RoPE over the first
and second half of each head, repeat_kv for GQA)."""
import math

import pytest
import torch

from megacute_b200.builders import llama_decode
from megacute_b200.checkpoint import LlamaGenerator, llama_shapes, params_from_hf, rope_inverse_frequencies, rope_tables_from_config
from oracle.graph_oracle import evaluate, rel_l2
from tests.helpers import TOL

BF = torch.bfloat16
CFG = dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256, num_hidden_layers=2,
           vocab_size=512, rms_norm_eps=1e-5, rope_theta=500000.0,
           rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=64))


def hf_state_dict(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    E, H, KVH, F, V = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "intermediate_size", "vocab_size"))
    D = E // H
    r = lambda *s, std=0.05, mean=0.0: (torch.randn(*s, generator=g) * std + mean).to(BF)
    sd = {"model.embed_tokens.weight": r(V, E, std=0.5), "model.norm.weight": r(E, std=0.05, mean=1.0)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        sd.update({p + "input_layernorm.weight": r(E, mean=1.0), p + "post_attention_layernorm.weight": r(E, mean=1.0),
                   p + "self_attn.q_proj.weight": r(H * D, E), p + "self_attn.k_proj.weight": r(KVH * D, E),
                   p + "self_attn.v_proj.weight": r(KVH * D, E), p + "self_attn.o_proj.weight": r(E, H * D),
                   p + "mlp.gate_proj.weight": r(F, E), p + "mlp.up_proj.weight": r(F, E), p + "mlp.down_proj.weight": r(E, F)})
    return sd


def hf_forward(cfg, sd, tokens, cos, sin):
    """Logits (len(tokens), vocab) of a causal Llama forward pass, fp32, Hugging Face conventions."""
    E, H, KVH = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D, eps, T = E // H, cfg["rms_norm_eps"], len(tokens)
    f = {k: v.float() for k, v in sd.items()}
    rms = lambda x, w: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
    rot = lambda x: torch.cat([-x[..., D // 2:], x[..., :D // 2]], -1)
    c, s = cos[:T].float()[:, None], sin[:T].float()[:, None]
    x = f["model.embed_tokens.weight"][torch.tensor(tokens)]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rms(x, f[p + "input_layernorm.weight"])
        q = (h @ f[p + "self_attn.q_proj.weight"].T).view(T, H, D)
        k = (h @ f[p + "self_attn.k_proj.weight"].T).view(T, KVH, D)
        v = (h @ f[p + "self_attn.v_proj.weight"].T).view(T, KVH, D)
        q, k = q * c + rot(q) * s, k * c + rot(k) * s
        k, v = k.repeat_interleave(H // KVH, 1), v.repeat_interleave(H // KVH, 1)
        att = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        att = att.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf")).softmax(-1)
        o = torch.einsum("hqk,khd->qhd", att, v).reshape(T, H * D)
        x = x + o @ f[p + "self_attn.o_proj.weight"].T
        h = rms(x, f[p + "post_attention_layernorm.weight"])
        x = x + (torch.nn.functional.silu(h @ f[p + "mlp.gate_proj.weight"].T) * (h @ f[p + "mlp.up_proj.weight"].T)) @ f[p + "mlp.down_proj.weight"].T
    return rms(x, f["model.norm.weight"]) @ f.get("lm_head.weight", f["model.embed_tokens.weight"]).T


def test_llama3_rope_scaling_closed_form():
    inv = rope_inverse_frequencies(CFG)
    D = CFG["hidden_size"] // CFG["num_attention_heads"]
    sc = CFG["rope_scaling"]
    base = 1.0 / CFG["rope_theta"] ** (torch.arange(0, D, 2, dtype=torch.float64) / D)
    for b, got in zip(base.tolist(), inv.tolist()):
        wl = 2 * math.pi / b
        orig = sc["original_max_position_embeddings"]
        if wl > orig / sc["low_freq_factor"]:
            want = b / sc["factor"]
        elif wl < orig / sc["high_freq_factor"]:
            want = b
        else:
            t = (orig / wl - sc["low_freq_factor"]) / (sc["high_freq_factor"] - sc["low_freq_factor"])
            want = (1 - t) * b / sc["factor"] + t * b
        assert abs(got - want) <= 1e-15 + 1e-12 * abs(want)
    kinds = {("long" if 2 * math.pi / b > 64 else "short" if 2 * math.pi / b < 16 else "band") for b in base.tolist()}
    assert kinds == {"long", "short", "band"}                       # the test config exercises all three branches
    plain = rope_inverse_frequencies({**CFG, "rope_scaling": None})
    assert torch.equal(plain, base)
    cos, sin = rope_tables_from_config(CFG, 256)
    assert cos.shape == sin.shape == (256, D) and cos.dtype == BF
    assert torch.equal(cos[:, :D // 2], cos[:, D // 2:]) and float(cos[0, 0]) == 1.0 and float(sin[0, 0]) == 0.0
    # the published Llama-3.2-1B numbers: factor 32, low 1, high 4, 8192 positions, theta 5e5, head_dim 64
    real = dict(hidden_size=2048, num_attention_heads=32, rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))
    r = rope_inverse_frequencies(real)
    assert abs(float(r[0]) - 1.0) < 1e-12 and abs(float(r[-1]) - 500000.0 ** (-62 / 64) / 32.0) < 1e-18


def test_hf_relayout_matches_a_plain_llama_forward():
    """Decode steps of llama_decode on the re-laid weights (oracle, fp32) reproduce, token by token, the
    last-position logits of a full causal forward pass written in Hugging Face's conventions."""
    sd = hf_state_dict(CFG)
    s = llama_shapes(CFG)
    p = params_from_hf(CFG, sd)
    assert p["wqkv"].shape == (2 * (4 + 2 * 2) * 64, 256) and p["wgu"].shape == (2 * 512, 256) and p["attn_norm"].shape == (2, 256)
    assert p["lm_head"].data_ptr() == sd["model.embed_tokens.weight"].data_ptr() or torch.equal(p["lm_head"], sd["model.embed_tokens.weight"])
    L = 128
    cos, sin = rope_tables_from_config(CFG, L)
    g = llama_decode(1, s["E"], s["H"], s["KVH"], s["F"], s["n"], L, s["vocab"], s["eps"], fused_step=True)
    tokens = [3, 401, 77, 12, 500, 9]
    want = hf_forward(CFG, sd, tokens, cos, sin)
    kvd = s["KVH"] * (s["E"] // s["H"])
    st = dict(ids=torch.zeros(1, 1, dtype=torch.int32), pos=torch.zeros(1, 1, dtype=torch.int32),
              k_cache=torch.zeros(s["n"] * L, kvd, dtype=BF), v_cache=torch.zeros(s["n"] * L, kvd, dtype=BF))
    for t, tok in enumerate(tokens):
        st["ids"].fill_(tok)
        out, st = evaluate(g, dict(cos=cos, sin=sin, **p, **st))
        # (the cache holds bf16 keys and values: a few 1e-3 against the all-fp32 forward pass)
        assert rel_l2(out[0][0], want[t]) < 5e-3, t
        assert int(st["ids"]) == int(out[0].argmax(-1)) and int(st["pos"]) == t + 1
    untied = dict(sd, **{"lm_head.weight": sd["model.embed_tokens.weight"].flip(0).contiguous()})
    assert torch.equal(params_from_hf(CFG, untied)["lm_head"], untied["lm_head.weight"])


@pytest.mark.gpu
def test_generator_matches_plain_forward(cuda):
    """LlamaGenerator (one self-feeding launch per token) on a synthetic Hugging Face state dict: the
    logits of every step against the plain forward pass over the tokens generated so far, and each chosen
    token is the argmax of the returned logits."""
    import megacute_b200 as mc
    sd = hf_state_dict(CFG, seed=3)
    gen = LlamaGenerator(CFG, sd, batch=2, max_seq=128, device=cuda)
    prompt = [5, 17, 300, 42]
    cos, sin = rope_tables_from_config(CFG, 128)
    for tok in prompt[:-1]:
        gen.state["ids"].fill_(tok)
        gen.step()
    gen.state["ids"].fill_(prompt[-1])
    seq = list(prompt)
    for _ in range(12):
        logits = gen.step()
        assert torch.equal(gen.state["ids"].flatten().long(), mc.argmax(logits))
        want = hf_forward(CFG, sd, seq, cos, sin)[-1]
        got = logits.float().cpu()
        assert rel_l2(got[0], want) < TOL and torch.equal(got[0], got[1])
        seq.append(int(gen.state["ids"][0]))
    assert int(gen.state["pos"]) == len(prompt) - 1 + 12
    gen2 = LlamaGenerator(CFG, sd, batch=2, max_seq=128, device=cuda)
    out = gen2.generate(prompt, 12)
    assert out.shape == (2, 12) and out[0].tolist() == seq[len(prompt):] and torch.equal(out[0], out[1])
    with pytest.raises(ValueError):
        gen2.generate(prompt, 500)
