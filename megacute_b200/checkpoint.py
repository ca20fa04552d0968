"""Running a Hugging Face Llama checkpoint through the decode megakernel: the pieces that need no network.

The reference ships this as a script (``examples/llama/llama1b.py``): download the checkpoint, re-lay
its weights for ``llama_decode`` (:42-57), build Llama-3 RoPE tables (:59-71), feed the prompt one
token per decode step and generate greedily (:103-121), optionally compare the tokens with
``transformers`` (``--check``, :124-131).  Downloading and ``--check`` need the hub; everything else is
here as functions that take an already loaded config dict and state dict:

    cfg, sd = <config.json as dict>, <name -> tensor, Hugging Face Llama names>
    gen = LlamaGenerator(cfg, sd, batch=1, max_seq=1024)        # compiles one self-feeding decode launch
    tokens = gen.generate(prompt_ids, 128)                      # greedy; one launch per token

``python -m megacute_b200.checkpoint --model DIR`` does the same from a local directory holding
``config.json`` and ``*.safetensors`` (no download is attempted).
"""

from __future__ import annotations

import json
import math
import pathlib

import torch

from .builders import llama_decode
from .graph import swiglu_weight

BF = torch.bfloat16


def llama_shapes(cfg: dict) -> dict:
    """The builder arguments of ``llama_decode`` from a Hugging Face Llama config."""
    return dict(E=cfg["hidden_size"], H=cfg["num_attention_heads"], KVH=cfg.get("num_key_value_heads", cfg["num_attention_heads"]),
                F=cfg["intermediate_size"], n=cfg["num_hidden_layers"], vocab=cfg["vocab_size"], eps=cfg.get("rms_norm_eps", 1e-6))


def params_from_hf(cfg: dict, sd: dict, device=None) -> dict:
    """Hugging Face Llama tensors -> the stacked parameters of ``llama_decode``.

    Per layer: q, k and v projections stacked into one (H + 2 KVH) D x E matrix (the rows the fused
    QKV linear produces in that order), gate and up interleaved in 64-row blocks for the swiglu linear
    (``swiglu_weight``), norm gains as one row each; layer i of every parameter is rows
    [i r, (i + 1) r).  A checkpoint without ``lm_head.weight`` ties the head to the embedding table.
    (reference: examples/llama/llama1b.py:42-57)"""
    n = cfg["num_hidden_layers"]

    def layer(i, name):
        return sd[f"model.layers.{i}.{name}.weight"]

    def stack(make):
        t = torch.cat([make(i) for i in range(n)]).to(BF).contiguous()
        return t.to(device) if device is not None else t

    out = {
        "attn_norm": stack(lambda i: layer(i, "input_layernorm").reshape(1, -1)),
        "wqkv": stack(lambda i: torch.cat([layer(i, "self_attn.q_proj"), layer(i, "self_attn.k_proj"), layer(i, "self_attn.v_proj")])),
        "wo": stack(lambda i: layer(i, "self_attn.o_proj")),
        "mlp_norm": stack(lambda i: layer(i, "post_attention_layernorm").reshape(1, -1)),
        "wgu": stack(lambda i: swiglu_weight(layer(i, "mlp.gate_proj"), layer(i, "mlp.up_proj"))),
        "wd": stack(lambda i: layer(i, "mlp.down_proj")),
    }
    head = sd.get("lm_head.weight", sd["model.embed_tokens.weight"])
    for name, t in (("final_norm", sd["model.norm.weight"].reshape(1, -1)), ("lm_head", head)):
        t = t.to(BF).contiguous()
        out[name] = t.to(device) if device is not None else t
    return out


def rope_inverse_frequencies(cfg: dict) -> torch.Tensor:
    """Inverse frequencies of the D / 2 rotary pairs, fp64, with the Llama-3 scaling when the config asks
    for it (``rope_scaling.rope_type == "llama3"``): wavelengths longer than ``orig / low_freq_factor``
    are stretched by ``factor``, those shorter than ``orig / high_freq_factor`` are kept, and the band
    between is blended linearly in ``orig / wavelength``.  (reference: examples/llama/llama1b.py:59-68)"""
    D = cfg["hidden_size"] // cfg["num_attention_heads"]
    inv = 1.0 / float(cfg.get("rope_theta", 10000.0)) ** (torch.arange(0, D, 2, dtype=torch.float64) / D)
    sc = cfg.get("rope_scaling") or {}
    if sc.get("rope_type", sc.get("type")) != "llama3":
        return inv
    factor, lo, hi = float(sc["factor"]), float(sc["low_freq_factor"]), float(sc["high_freq_factor"])
    orig = float(sc["original_max_position_embeddings"])
    wavelength = 2 * math.pi / inv
    blend = ((orig / wavelength - lo) / (hi - lo)).clamp(0.0, 1.0)          # 0: fully stretched, 1: untouched
    return (1.0 - blend) * inv / factor + blend * inv


def rope_tables_from_config(cfg: dict, max_seq: int, device=None):
    """cos / sin tables (max_seq, D) in the rotate-half convention, bf16, from fp64 angles."""
    inv = rope_inverse_frequencies(cfg)
    ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * inv[None]
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().to(BF).contiguous(), ang.sin().to(BF).contiguous()
    return (cos.to(device), sin.to(device)) if device is not None else (cos, sin)


class LlamaGenerator:
    """Greedy generation with one megakernel launch per token.

    The decode graph is built with ``fused_step=True``: the token ids live on the device, the launch
    gathers their embedding rows and overwrites them with the argmax of its logits, so the loop below
    is nothing but launches (the reference's loop wraps its launch in index_select / copy_ / argmax,
    examples/llama/llama1b.py:103-121).  The prompt goes through the same program one token per step."""

    def __init__(self, cfg: dict, sd: dict, batch: int = 1, max_seq: int = 1024, device=None, **compile_kw):
        import megacute_b200 as mc
        self.cfg, self.batch, self.max_seq = cfg, batch, max_seq
        s = llama_shapes(cfg)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        assert max_seq % 128 == 0, "max_seq must be a multiple of 128 (decode attention tiles)"
        self.graph = llama_decode(batch, s["E"], s["H"], s["KVH"], s["F"], s["n"], max_seq, s["vocab"], s["eps"], fused_step=True)
        self.prog = mc.compile(self.graph, **compile_kw)
        self.params = params_from_hf(cfg, sd, self.device)
        cos, sin = rope_tables_from_config(cfg, max_seq, self.device)
        kvd = s["KVH"] * (s["E"] // s["H"])
        self.state = dict(ids=torch.zeros(batch, 1, dtype=torch.int32, device=self.device),
                          pos=torch.zeros(1, 1, dtype=torch.int32, device=self.device),
                          k_cache=torch.zeros(s["n"] * batch * max_seq, kvd, dtype=BF, device=self.device),
                          v_cache=torch.zeros(s["n"] * batch * max_seq, kvd, dtype=BF, device=self.device))
        self.inputs = dict(cos=cos, sin=sin)

    def step(self):
        """One decode step: consumes ``state['ids']`` at ``state['pos']``, leaves the greedy tokens in ``ids``.
        Returns the logits (a program-owned buffer, overwritten by the next step)."""
        return self.prog(**self.inputs, **self.params, **self.state)

    def generate(self, prompt: list[int], n_tokens: int) -> torch.Tensor:
        """Feed ``prompt`` (the same for every sequence of the batch) token by token, then generate
        ``n_tokens`` greedily.  Returns (batch, n_tokens) int32 on the device; no host synchronisation
        inside the loop."""
        if not prompt:
            raise ValueError("empty prompt")
        if int(self.state["pos"]) + len(prompt) + n_tokens > self.max_seq:
            raise ValueError("prompt + generated tokens exceed max_seq")
        for tok in prompt[:-1]:                         # the tokens the model is told, not asked
            self.state["ids"].fill_(int(tok))
            self.step()
        self.state["ids"].fill_(int(prompt[-1]))
        out = torch.empty(self.batch, n_tokens, dtype=torch.int32, device=self.device)
        for i in range(n_tokens):
            self.step()
            out[:, i] = self.state["ids"][:, 0]         # device-side copy of the tokens this step chose
        self.prog.check()
        return out


def load_local(path) -> tuple[dict, dict]:
    """config.json and every *.safetensors of a local checkpoint directory (nothing is downloaded)."""
    from safetensors.torch import load_file
    path = pathlib.Path(path)
    cfg = json.loads((path / "config.json").read_text())
    sd: dict = {}
    for f in sorted(path.glob("*.safetensors")):
        sd.update(load_file(str(f)))
    if not sd:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    return cfg, sd


def main(argv=None):
    import argparse
    import time
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="local directory with config.json and *.safetensors")
    ap.add_argument("--prompt-ids", default="128000,791,2380,7016,315,30945,80011,527", help="comma-separated token ids")
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--max-seq", type=int, default=1024)
    a = ap.parse_args(argv)
    cfg, sd = load_local(a.model)
    gen = LlamaGenerator(cfg, sd, a.batch, a.max_seq)
    prompt = [int(x) for x in a.prompt_ids.split(",")]
    torch.cuda.synchronize()
    t0 = time.time()
    out = gen.generate(prompt, a.tokens)
    torch.cuda.synchronize()
    dt = time.time() - t0
    print(f"{len(prompt) - 1 + a.tokens} steps x batch {a.batch}: {dt / (len(prompt) - 1 + a.tokens) * 1e3:.3f} ms/step")
    print(out[0].tolist())


if __name__ == "__main__":
    main()
