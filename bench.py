"""Benchmark of the hot path: one Llama-3.2-1B-shaped decode step = one persistent megakernel launch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--ctx C] [--impl reference]
                    [--no-sweep] [--no-secondary] [--no-cpu-baseline]

Headline workload (the reference's batch-1 decode benchmark): 16 layers, hidden 2048, 32 q / 8 kv heads,
head_dim 64, SwiGLU 8192, vocab 128256 tied, bf16 random-init weights, batch 1, KV caches prefilled to
context 1024, greedy decode.  A step is what the reference times in examples/llama/llama1b.py:103-121
(embedding gather, one megakernel launch, argmax), here with the gather and the argmax inside the launch.  With N > 1 every rank runs its own replica on
its own sequences (batch-sharded, weights replicated, no collective on the hot path).

Prints ONE JSON line (rank 0):
  value / ms_per_step   median over `repeats` blocks of exactly K steps (device time, CUDA events, slowest
                        rank), everything resident in HBM; `ms_per_step_min` is the best block
  kernel_ms             the megakernel launches alone: the same number, a step being one launch
  e2e                   the same loop driven from pinned host memory (token ids copied in and out every step)
  roofline              algorithmic bytes of a step / kernel_ms against the measured HBM copy bandwidth
  sweep                 the metric's other points: batch 1 and batch 64 at context 256 ... 32768 (one GPU), or,
                        with N > 1, batch 64 per GPU at context 1024 and 4096 (64 N sequences in all)
  secondary             the tensor-bound configurations (MLP block, prefill 4 x 4096, DiT): kernel time, TFLOP/s
  cpu_baseline          the fp32 torch oracle of the headline graph on the host cores (3 steps)
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WEIGHT_BYTES = 2 * (16 * (3072 * 2048 + 2048 * 2048 + 16384 * 2048 + 2048 * 8192) + 128256 * 2048)   # 2 471 493 632
KV_BYTES_PER_TOKEN = 16 * 2 * 512 * 2                                                               # 32 768
# the reference's published ms/step on one B200 (its README table for batch 64; batch 1 read off its latency plot)
PUBLISHED_MS = {(1, 256): 0.956, (1, 1024): 0.961, (1, 4096): 0.974, (1, 16384): 1.040, (1, 32768): 1.125,
                (64, 256): 1.06, (64, 1024): 1.31, (64, 4096): 2.21, (64, 16384): 5.92, (64, 32768): 10.97}
SWEEP_1GPU = [(1, 256), (1, 4096), (1, 16384), (1, 32768), (64, 256), (64, 1024), (64, 4096), (64, 16384), (64, 32768)]
SWEEP_NGPU = [(64, 1024), (64, 4096)]
MIN_TIMED_SECONDS = 0.5


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def csrc_digest() -> str:
    """Hash of the kernel sources: a DRAM-traffic figure from an ncu capture is only quoted while the
    kernel it was captured on is the kernel that runs."""
    h = hashlib.sha256()
    for p in sorted((ROOT / "megacute_b200" / "csrc").iterdir()):
        if p.suffix in (".cu", ".cuh"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()[:16]


def measured_traffic(B: int, ctx: int):
    """dram__bytes_read.sum + dram__bytes_write.sum of one megakernel launch of this workload, from
    profiles/traffic.json (written next to the ncu summary it comes from) -- or None when there is no
    capture of this workload, or the kernel sources have changed since it was taken."""
    p = ROOT / "profiles" / "traffic.json"
    if not p.exists():
        return None
    d = json.loads(p.read_text())
    if d.get("csrc_digest") != csrc_digest():
        return None
    return d.get("dram_bytes_per_launch", {}).get(f"b{B}_ctx{ctx}")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: self.rows.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_workload(B, ctx, device, seed=0, weights=None):
    """The decode step as one self-feeding launch: state `ids` (B, 1) int32 holds the current tokens; the
    launch gathers their embedding rows, runs the 16 layers and the lm_head, and overwrites ids with the
    greedy tokens (builders.llama_decode(fused_step=True))."""
    import megacute_b200 as mc
    from megacute_b200 import workloads as W
    from megacute_b200.builders import llama_decode
    c = W.LLAMA_1B
    max_seq = -(-(ctx + 128) // 128) * 128
    g = llama_decode(B, c["E"], c["H"], c["KVH"], c["F"], c["n"], max_seq, c["vocab"], c["eps"], fused_step=True)
    w = weights if weights is not None else W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], seed, device)
    st, ids = W.llama_decode_state(B, c["E"], c["H"], c["KVH"], c["n"], max_seq, ctx, c["vocab"], seed + 1, device)
    del st["x"]
    st["ids"] = ids.to(torch.int32).reshape(B, 1).contiguous()
    cos, sin = W.rope_tables(max_seq, c["E"] // c["H"], c["theta"], device)
    return mc, g, dict(cos=cos, sin=sin, **w), st, ids, max_seq


def cpu_oracle_ms(B, ctx, steps, seed=0):
    """Time the fp32 torch oracle of the same graph on the host cores: ms per decode step."""
    from oracle.graph_oracle import evaluate
    _, g, params, st, ids, _ = build_workload(B, ctx, "cpu", seed)
    times = []
    for _ in range(steps + 1):
        t0 = time.perf_counter()
        out, new = evaluate(g, {**params, **st})          # gather + layers + lm_head + argmax, states updated
        times.append((time.perf_counter() - t0) * 1e3)
        st = dict(new)
    return statistics.median(times[1:]) if steps > 1 else times[-1]


class Timing:
    """Device timing of a multi-rank job: blocks bracketed by barrier + synchronize, CUDA events on the
    launching stream, the slowest rank's time."""

    def __init__(self, dev, world):
        self.dev, self.world = dev, world

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def block(self, fn, n):
        from megacute_b200.sharding import max_over_ranks
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        fn(n)
        e1.record()
        self.barrier()
        return max_over_ranks(e0.elapsed_time(e1) / n, self.dev)        # ms per step, slowest rank

    def repeated(self, fn, n, before=lambda: None):
        """Blocks of exactly n steps until MIN_TIMED_SECONDS of device time have been timed (the count
        follows from the first block's time, which is the same number on every rank)."""
        before()
        first = self.block(fn, n)
        reps = max(1, min(200, math.ceil(MIN_TIMED_SECONDS * 1e3 / max(first * n, 1e-3))))
        times = [first]
        for _ in range(reps - 1):
            before()
            times.append(self.block(fn, n))
        return times


def measure_decode(mc, timing, B, ctx, dev, weights, steps, warmup, seed, with_e2e=False):
    """Compile and time the decode step of (B sequences on this GPU, context ctx).  Returns a dict of
    medians over the repeated blocks (ms per step)."""
    _, g, params, st, ids, max_seq = build_workload(B, ctx, dev, seed, weights)
    prog = mc.compile(g)
    args = dict(params, **st)
    room = max_seq - ctx - 1                 # steps before pos must go back to ctx

    def reset_state():
        st["pos"].fill_(ctx)

    def run_steps(n):                        # a step IS one launch: gather, layers, lm_head and argmax run inside it
        for i in range(n):
            if i % room == room - 1:
                reset_state()
            prog(**args)

    h_in = torch.empty(B, 1, dtype=torch.int32).pin_memory()
    h_out = torch.empty(B, 1, dtype=torch.int32).pin_memory()

    def run_e2e(n):
        h_in.copy_(st["ids"].cpu())
        for i in range(n):
            if i % room == room - 1:
                reset_state()
            st["ids"].copy_(h_in, non_blocking=True)             # host -> device: this step's token ids
            prog(**args)
            h_out.copy_(st["ids"], non_blocking=True)            # device -> host: the sampled tokens
            torch.cuda.current_stream().synchronize()
            h_in.copy_(h_out)

    run_steps(max(3, warmup))
    prog.check()
    t_step = timing.repeated(run_steps, steps, reset_state)
    out = {"ms_per_step": statistics.median(t_step), "ms_per_step_min": min(t_step), "repeats": len(t_step),
           "kernel_ms": statistics.median(t_step), "kernel_ms_min": min(t_step)}
    if with_e2e:
        t_e2e = timing.repeated(run_e2e, steps, reset_state)
        out["e2e_ms"] = statistics.median(t_e2e)
    prog.check()
    avg_ctx = ctx + (min(steps, room) - 1) / 2
    out["algorithmic_bytes"] = WEIGHT_BYTES + B * avg_ctx * KV_BYTES_PER_TOKEN
    del prog, st, args
    torch.cuda.empty_cache()
    return out


def roofline_of(m, pk):
    achieved = m["algorithmic_bytes"] / (m["kernel_ms"] * 1e-3) / 1e9
    return achieved, achieved / pk["hbm_gbs"]


def secondary_configs(pk):
    """Kernel time of the tensor-bound configurations (MLP block, prefill, DiT) on this GPU."""
    from megacute_b200 import measure
    rows = []
    for name in ("mlp_block", "prefill", "dit"):
        t0 = time.time()
        ms, flop, prog = measure.CONFIGS[name](torch.device("cuda", torch.cuda.current_device()))
        tf = flop / ms / 1e9
        rows.append({"config": name, "kernel_us": ms * 1e3, "tflops": tf, "frac_of_bf16_peak": tf / pk["bf16_tflops"],
                     "frac_of_bf16_sustained": tf / pk["bf16_tflops_sustained"], "tcgen05_ops": prog.tcgen05_ops,
                     "wall_s": round(time.time() - t0, 1)})
        del prog
        torch.cuda.empty_cache()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--impl", default="megacute_b200", choices=["megacute_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    a = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    headline = (a.batch, a.ctx) == (1, 1024)
    config = {"workload": f"llama-3.2-1b-shape decode step, batch {a.batch} per GPU, context {a.ctx}"
                          + (" (configs[1])" if headline else " (a point of configs[2])" if a.batch == 64 else ""),
              "batch_per_gpu": a.batch, "ctx": a.ctx,
              "layers": 16, "hidden": 2048, "vocab": 128256, "parallelism": f"replica x{world} (batch-sharded)",
              "l2": "weights (2.47 GB) exceed L2 (126 MB): every step re-reads them from HBM",
              "step": "one megakernel launch: embedding gather, 16 layers, lm_head, greedy argmax (token ids stay on the device)"}
    base = {"metric": "decode ms/step, 1B Llama-shape", "unit": "ms/step", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": config}

    if a.impl == "reference":
        # The reference has no CPU implementation and its CuTe-DSL kernel cannot run in this image
        # (needs nvidia-cutlass-dsl 4.8.0): the reference arm times the CPU oracle port of the
        # same graph on all host threads.
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)       # torchrun pins OMP_NUM_THREADS=1 for its workers
        steps = max(1, min(a.steps, 3))
        ms = cpu_oracle_ms(a.batch, a.ctx, steps)
        cores = torch.get_num_threads()
        line = dict(base, impl="reference", value=ms, ms_per_step=ms, steps=steps, warmup=1, dtype="f32",
                    cpu_baseline={"value": ms, "unit": "ms/step", "cores": cores, "kind": "port",
                                  "sample": f"{steps} full decode steps of the same config, fp32 torch oracle, "
                                            f"{cores} threads of {os.cpu_count()} host cores"},
                    e2e={"value": ms, "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        print(json.dumps(line))
        return

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from megacute_b200 import workloads as W
    from megacute_b200.sharding import shard_range
    import megacute_b200 as mc
    first_seq, n_seq = shard_range(a.batch * world, world, rank)       # weak scaling: batch_per_gpu sequences each
    assert n_seq == a.batch
    c = W.LLAMA_1B
    weights = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], rank, dev)   # replicated per GPU
    timing = Timing(dev, world)
    pk = peaks()

    with ClockSampler(local) as cs:                  # clocks and throttle reasons over the headline's timed regions
        m = measure_decode(mc, timing, a.batch, a.ctx, dev, weights, a.steps, a.warmup, rank, with_e2e=True)
    clocks = cs.summary()

    sweep = []
    if not a.no_sweep:
        for B, ctx in (SWEEP_1GPU if world == 1 else SWEEP_NGPU):
            if (B, ctx) == (a.batch, a.ctx):
                continue
            steps = a.steps if B * ctx < 64 * 16384 else max(4, min(a.steps, 20))
            r = measure_decode(mc, timing, B, ctx, dev, weights, steps, min(a.warmup, 4), rank)
            ach, frac = roofline_of(r, pk)
            pub = PUBLISHED_MS.get((B, ctx))
            sweep.append({"batch_per_gpu": B, "sequences": B * world, "ctx": ctx, "steps": steps, "repeats": r["repeats"],
                          "ms_per_step": r["ms_per_step"], "ms_per_step_min": r["ms_per_step_min"], "kernel_ms": r["kernel_ms"],
                          "tokens_per_s": world * B * 1e3 / r["ms_per_step"],
                          "roofline": {"achieved": ach, "frac": frac, "unit": "GB/s"},
                          "reference_published_ms": pub, "reference_over_ours": (pub / r["ms_per_step"]) if pub else None})
    del weights
    torch.cuda.empty_cache()
    secondary = secondary_configs(pk) if (world == 1 and not a.no_secondary) else []

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    achieved, frac = roofline_of(m, pk)
    pub = PUBLISHED_MS.get((a.batch, a.ctx))
    line = dict(base, value=m["ms_per_step"], ms_per_step=m["ms_per_step"], ms_per_step_min=m["ms_per_step_min"],
                repeats=m["repeats"], tokens_per_s=world * a.batch * 1e3 / m["ms_per_step"],
                e2e={"value": m["e2e_ms"], "unit": "ms/step", "h2d_bytes_per_step": a.batch * 4,
                     "d2h_bytes_per_step": a.batch * 4},
                # our kernels inside one timed block of `steps` steps: one megakernel launch per step (embedding
                # gather and greedy argmax are its first and last instructions), nothing else on the stream
                gpu_launches=a.steps,
                kernel_ms=m["kernel_ms"], kernel_ms_min=m["kernel_ms_min"], clocks=clocks,
                reference_published_ms=pub,
                roofline={"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": frac,
                          "peak_kind": pk["kind"], "traffic": measured_traffic(a.batch, a.ctx),
                          "algorithmic_bytes": m["algorithmic_bytes"], "kernel": "mk::megakernel<false>"},
                sweep=sweep, secondary=secondary)
    if not a.no_cpu_baseline and world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        cpu_ms = cpu_oracle_ms(a.batch, a.ctx, 3)
        line["cpu_baseline"] = {"value": cpu_ms, "unit": "ms/step", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "3 full decode steps of the same config, fp32 torch oracle on host cores"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
