"""Seeded synthetic inputs for the benchmarked workloads.

The reference publishes its numbers on the real Llama-3.2-1B checkpoint
(``examples/llama/llama1b.py``); no checkpoint or dataset is available offline, so every workload
here takes that model's shapes with random-init values: weights bf16 ~ N(0, 0.02), norm gains
1 + N(0, 0.02), KV caches bf16 ~ N(0, 1) up to the context length and zero beyond, token ids
uniform over the vocabulary.
"""

from __future__ import annotations

import torch

from .builders import dit_param_shapes, llama_param_shapes
from .graph import swiglu_weight

BF = torch.bfloat16
LLAMA_1B = dict(E=2048, H=32, KVH=8, F=8192, n=16, vocab=128256, eps=1e-5, theta=500000.0)


def _gen(device, seed):
    return torch.Generator(device=device).manual_seed(seed)


def randn(shape, std, gen, device, mean=0.0):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std + mean).to(BF)


def rope_tables(max_seq: int, D: int, theta: float = 500000.0, device="cpu"):
    """Rotate-half cos/sin tables (max_seq, D): fp64 math stored as bf16, no frequency scaling."""
    inv = 1.0 / theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D)
    ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * inv[None]
    ang = torch.cat([ang, ang], -1)
    return ang.cos().to(BF).contiguous().to(device), ang.sin().to(BF).contiguous().to(device)


def llama_weights(E, H, KVH, F, n, vocab=None, seed=0, device="cuda"):
    g = _gen(device, seed)
    out = {}
    for name, (r, c) in llama_param_shapes(E, H, KVH, F).items():
        if name.endswith("norm"):
            out[name] = randn((n * r, c), 0.02, g, device, mean=1.0)
        elif name == "wgu":
            per = [swiglu_weight(randn((F, E), 0.02, g, device), randn((F, E), 0.02, g, device)) for _ in range(n)]
            out[name] = torch.cat(per).contiguous()
        else:
            out[name] = randn((n * r, c), 0.02, g, device)
    if vocab:
        out["final_norm"] = randn((1, E), 0.02, g, device, mean=1.0)
        out["lm_head"] = randn((vocab, E), 0.02, g, device)       # tied: also the embedding table
    return out


def llama_decode_state(B, E, H, KVH, n, max_seq, ctx, vocab=None, seed=1, device="cuda"):
    """States of a decode step with caches prefilled to ``ctx`` tokens: x (filled by the caller
    from the embedding), pos, k_cache, v_cache; plus the first token ids."""
    g = _gen(device, seed)
    D = E // H
    kvd = KVH * D
    st = {"x": torch.zeros(B, E, dtype=BF, device=device),
          "pos": torch.full((1, 1), ctx, dtype=torch.int32, device=device)}
    for name in ("k_cache", "v_cache"):
        c = torch.zeros(n * B, max_seq, kvd, dtype=BF, device=device)
        if ctx:
            step = max(1, (1 << 28) // max(1, ctx * kvd))        # bound the fp32 temporary
            for r0 in range(0, n * B, step):
                r1 = min(n * B, r0 + step)
                c[r0:r1, :ctx] = torch.randn((r1 - r0, ctx, kvd), generator=g, device=device,
                                             dtype=torch.float32).to(BF)
        st[name] = c.reshape(n * B * max_seq, kvd)
    ids = torch.randint(0, vocab or E, (B,), generator=g, device=device)
    return st, ids


def mlp_block_inputs(M=256, E=2048, F=5632, seed=0, device="cuda"):
    g = _gen(device, seed)
    return {"x": randn((M, E), 1.0, g, device), "nw": randn((1, E), 0.02, g, device, mean=1.0),
            "w1": swiglu_weight(randn((F, E), 0.02, g, device), randn((F, E), 0.02, g, device)).contiguous(),
            "w2": randn((E, F), 0.02, g, device)}


def dit_inputs(B, S, E, F, n, seed=0, device="cuda"):
    g = _gen(device, seed)
    out = {"x": randn((B * S, E), 1.0, g, device), "c": randn((B, E), 1.0, g, device)}
    for name, (r, c) in dit_param_shapes(E, F).items():
        out[name] = randn((n * r, c), 0.02, g, device)
    return out
