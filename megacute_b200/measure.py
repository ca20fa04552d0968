"""Kernel-time measurements of the tensor-bound benchmark configurations (the decode step has its own
driver, ``bench.py``):

    python -m megacute_b200.measure [mlp_block] [dit] [prefill] [decode_b64_small] [prefill_small] [decode_b64_ragged]

* ``mlp_block``: RMS norm -> gate/up + swiglu -> down + residual, 256 rows, 2048 -> 2 x 5632 -> 2048
* ``dit``: 28 DiT blocks, 32 images x 256 tokens, width 1024, 16 heads, MLP 4096
* ``prefill``: Llama-3.2-1B shape, 4 sequences x 4096 tokens, 16 layers + lm_head
* ``decode_b64_small``, ``prefill_small``: cut-down cases of the same kernels for profiler captures
  (batch-64 decode at context 4096 with 4 layers and a 32768-row lm_head, 2.2 GB of cache; prefill
  with 2 layers): a few GB on the device, a handful of launches

* ``decode_b64_ragged``: the full 16-layer batch-64 decode step with one position per sequence, spread
  evenly over 256 .. 4096 tokens (a ragged batch: not possible in the reference)

Synthetic bf16 inputs and weights of those shapes; each configuration is compiled once, warmed up
twice, then timed over a few launches with CUDA events on the launching stream.  Prints one line
per configuration: time per launch and TFLOP/s against the configuration's algorithmic flops.
"""

from __future__ import annotations

import sys
import time

import torch

import megacute_b200 as mc
from megacute_b200 import workloads as W
from megacute_b200.builders import dit_stack, llama_stack, mlp_block


def _time(prog, args, launches):
    for _ in range(2):
        prog(**args)
    prog.check()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        prog(**args)
    e1.record()
    torch.cuda.synchronize()
    prog.check()
    return e0.elapsed_time(e1) / launches


def measure_mlp_block(dev):
    g = mlp_block(256)
    prog = mc.compile(g)
    ms = _time(prog, W.mlp_block_inputs(device=dev), 20)
    flop = 2 * 256 * 2048 * 11264 + 2 * 256 * 5632 * 2048
    return ms, flop, prog


def measure_dit(dev):
    g = dit_stack(32, 256, 1024, 16, 4096, 28)
    prog = mc.compile(g)
    ms = _time(prog, W.dit_inputs(32, 256, 1024, 4096, 28, 0, dev), 3)
    return ms, 6.02e12, prog


def measure_prefill(dev):
    c = W.LLAMA_1B
    g = llama_stack(4, 4096, c["E"], c["H"], c["KVH"], c["F"], c["n"], vocab=c["vocab"])
    prog = mc.compile(g)
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], 0, dev)
    x = torch.randn(4 * 4096, c["E"], device=dev, dtype=torch.bfloat16)
    cos, sin = W.rope_tables(4096, c["E"] // c["H"], c["theta"], dev)
    names = {b.name for b in prog.g.inputs + prog.g.params + prog.g.states}
    args = {k: v for k, v in dict(x=x, cos=cos, sin=sin, **w).items() if k in names}
    ms = _time(prog, args, 2)
    return ms, 3.63e13, prog


def measure_prefill_small(dev):
    c = W.LLAMA_1B
    n = 2
    g = llama_stack(4, 4096, c["E"], c["H"], c["KVH"], c["F"], n, vocab=c["vocab"])
    prog = mc.compile(g)
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], n, c["vocab"], 0, dev)
    x = torch.randn(4 * 4096, c["E"], device=dev, dtype=torch.bfloat16)
    cos, sin = W.rope_tables(4096, c["E"] // c["H"], c["theta"], dev)
    names = {b.name for b in prog.g.inputs + prog.g.params + prog.g.states}
    args = {k: v for k, v in dict(x=x, cos=cos, sin=sin, **w).items() if k in names}
    ms = _time(prog, args, 2)
    T, E, F, D, KVH = 4 * 4096, c["E"], c["F"], c["E"] // c["H"], c["KVH"]
    layer = 2 * T * E * (E + 2 * KVH * D) + 2 * T * E * E + 6 * T * E * F + 4 * 4 * c["H"] * D * 4096 * 4096 // 2
    return ms, n * layer + 2 * 4 * E * c["vocab"], prog


def measure_decode_b64_small(dev):
    from megacute_b200.builders import llama_decode
    c = W.LLAMA_1B
    B, ctx, n, vocab = 64, 4096, 4, 32768
    max_seq = ctx + 128
    g = llama_decode(B, c["E"], c["H"], c["KVH"], c["F"], n, max_seq, vocab, c["eps"])
    prog = mc.compile(g)
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], n, vocab, 0, dev)
    st, _ = W.llama_decode_state(B, c["E"], c["H"], c["KVH"], n, max_seq, ctx, vocab, 1, dev)
    cos, sin = W.rope_tables(max_seq, c["E"] // c["H"], c["theta"], dev)
    ms = _time(prog, dict(cos=cos, sin=sin, **w, **st), 2)
    kv_bytes = n * B * (ctx + 3) * 2 * c["KVH"] * (c["E"] // c["H"]) * 2          # the cache rows the third launch reads
    print(f"decode_b64_small: cache bytes read per launch {kv_bytes}")
    E, F, D, KVH = c["E"], c["F"], c["E"] // c["H"], c["KVH"]
    return ms, 2 * B * (n * (E * (E + 2 * KVH * D) + E * E + 3 * E * F) + E * vocab), prog


def measure_decode_b64_ragged(dev):
    from megacute_b200.builders import llama_decode
    c = W.LLAMA_1B
    B, n, vocab, max_seq = 64, c["n"], c["vocab"], 4096 + 128
    g = llama_decode(B, c["E"], c["H"], c["KVH"], c["F"], n, max_seq, vocab, c["eps"], ragged=True)
    prog = mc.compile(g)
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], n, vocab, 0, dev)
    st, _ = W.llama_decode_state(B, c["E"], c["H"], c["KVH"], n, max_seq, 4096, vocab, 1, dev)
    pos = torch.linspace(256, 4096, B).round().to(torch.int32).reshape(B, 1)
    st["pos"] = pos.to(dev)
    cos, sin = W.rope_tables(max_seq, c["E"] // c["H"], c["theta"], dev)
    args = dict(cos=cos, sin=sin, **w, **st)
    launches = 6
    ms = _time(prog, args, launches)
    kv = int((pos.sum() + B * (2 + (launches - 1) / 2)) * n * 2 * c["KVH"] * (c["E"] // c["H"]) * 2)      # mean over the timed launches
    print(f"decode_b64_ragged: positions {int(pos.min())} .. {int(pos.max())}, cache bytes per launch {kv}, "
          f"{(kv + 2471493632) / ms / 1e6:.0f} GB/s of weights + cache")
    E, F, D, KVH = c["E"], c["F"], c["E"] // c["H"], c["KVH"]
    return ms, 2 * B * (n * (E * (E + 2 * KVH * D) + E * E + 3 * E * F) + E * vocab), prog


CONFIGS = {"mlp_block": measure_mlp_block, "dit": measure_dit, "prefill": measure_prefill,
           "decode_b64_small": measure_decode_b64_small, "prefill_small": measure_prefill_small,
           "decode_b64_ragged": measure_decode_b64_ragged}
DEFAULT = ["mlp_block", "dit", "prefill"]


def main(argv):
    names = argv or DEFAULT
    unknown = [n for n in names if n not in CONFIGS]
    if unknown:
        raise SystemExit(f"unknown configuration(s) {unknown}; choose from {list(CONFIGS)}")
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device (B200) is required: there is no CPU path")
    dev = torch.device("cuda", 0)
    for n in names:
        t0 = time.time()
        ms, flop, prog = CONFIGS[n](dev)
        print(f"{n}: {ms * 1e3:.1f} us per launch, {flop / ms / 1e9:.0f} TFLOP/s, {prog.tcgen05_ops} tile-GEMM ops on tcgen05, "
              f"{prog.packed_weight_bytes / 1e6:.0f} MB of packed weights, compiled and measured in {time.time() - t0:.1f} s")
        del prog
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main(sys.argv[1:])
