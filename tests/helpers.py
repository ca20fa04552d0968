"""Shared helpers of the test-suite: small seeded workloads and comparison with the oracle."""
import torch

from megacute_b200 import workloads as W
from megacute_b200.builders import llama_decode
from oracle.graph_oracle import evaluate, rel_l2  # noqa: F401

BF = torch.bfloat16
TOL = 1e-2          # rel-L2 bound of bf16 outputs against the fp32 oracle


def small_decode(B=1, E=256, H=4, KVH=2, F=512, n=2, max_seq=256, ctx=100, vocab=1000, seed=0, device="cpu",
                 eps=1e-5):
    g = llama_decode(B, E, H, KVH, F, n, max_seq, vocab, eps)
    w = W.llama_weights(E, H, KVH, F, n, vocab, seed, device)
    st, ids = W.llama_decode_state(B, E, H, KVH, n, max_seq, ctx, vocab, seed + 1, device)
    cos, sin = W.rope_tables(max_seq, E // H, device=device)
    st["x"] = w["lm_head"][ids].clone()
    return g, dict(cos=cos, sin=sin, **w), st, ids


def to_cpu(d):
    return {k: v.detach().cpu() for k, v in d.items()}
