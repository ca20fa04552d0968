"""Benchmark of the hot path: one Llama-3.2-1B-shaped decode step = one persistent megakernel launch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--ctx C] [--impl reference]

Workload (the reference's batch-1 decode benchmark): 16 layers, hidden 2048, 32 q / 8 kv heads, head_dim 64,
SwiGLU 8192, vocab 128256 tied, bf16 random-init weights, batch 1, KV caches prefilled to context
1024, greedy decode.  A step is what the reference times in examples/llama/llama1b.py:103-121:
embedding gather + copy into x, one megakernel launch, argmax.  With N > 1 every rank runs its own
replica on its own sequences (batch-sharded, weights replicated, no collective on the hot path).

Prints ONE JSON line (rank 0).  `value` is ms per decode step with everything resident in HBM,
`e2e` the same loop driven from host memory (token ids copied in and out every step).
"""

from __future__ import annotations

import argparse
import json
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

# DRAM bytes of one megakernel launch of the default workload (batch 1, ctx 1024), from one ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum of the megakernel launch)
MEASURED_TRAFFIC_B1_CTX1024 = 2_506_453_000 + 6_217_216
WEIGHT_BYTES = 2 * (16 * (3072 * 2048 + 2048 * 2048 + 16384 * 2048 + 2048 * 8192) + 128256 * 2048)   # 2 471 493 632
KV_BYTES_PER_TOKEN = 16 * 2 * 512 * 2                                                               # 32 768


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def build_workload(B, ctx, device, seed=0):
    import megacute_b200 as mc
    from megacute_b200 import workloads as W
    from megacute_b200.builders import llama_decode
    c = W.LLAMA_1B
    max_seq = -(-(ctx + 128) // 128) * 128
    g = llama_decode(B, c["E"], c["H"], c["KVH"], c["F"], c["n"], max_seq, c["vocab"], c["eps"])
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], seed, device)
    st, ids = W.llama_decode_state(B, c["E"], c["H"], c["KVH"], c["n"], max_seq, ctx, c["vocab"], seed + 1, device)
    cos, sin = W.rope_tables(max_seq, c["E"] // c["H"], c["theta"], device)
    return mc, g, dict(cos=cos, sin=sin, **w), st, ids, max_seq


def cpu_oracle_ms(B, ctx, steps, seed=0):
    """Time the fp32 torch oracle of the same graph on the host cores: ms per decode step."""
    from oracle.graph_oracle import evaluate
    _, g, params, st, ids, _ = build_workload(B, ctx, "cpu", seed)
    emb = params["lm_head"]
    times = []
    for _ in range(steps + 1):
        st["x"] = emb[ids].clone()
        t0 = time.perf_counter()
        out, new = evaluate(g, {**params, **st})
        times.append((time.perf_counter() - t0) * 1e3)
        for n in ("pos", "k_cache", "v_cache"):
            st[n] = new[n]
        ids = out[0].argmax(-1)
    return statistics.median(times[1:]) if steps > 1 else times[-1]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--impl", default="megacute_b200", choices=["megacute_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    a = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    config = {"workload": "llama-3.2-1b-shape decode step (configs[1])", "batch_per_gpu": a.batch, "ctx": a.ctx,
              "layers": 16, "hidden": 2048, "vocab": 128256, "parallelism": f"replica x{world} (batch-sharded)",
              "l2": "weights (2.47 GB) exceed L2 (126 MB): every step re-reads them from HBM"}
    base = {"metric": "decode ms/step, 1B Llama-shape", "unit": "ms/step", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": config}

    if a.impl == "reference":
        # The reference has no CPU implementation and its CuTe-DSL kernel cannot run in this image
        # (needs nvidia-cutlass-dsl 4.8.0): the reference arm times the CPU oracle port of the
        # same graph on all host threads.
        if rank != 0:
            return
        steps = max(1, min(a.steps, 3))
        ms = cpu_oracle_ms(a.batch, a.ctx, steps)
        cores = torch.get_num_threads()
        line = dict(base, impl="reference", value=ms, ms_per_step=ms, steps=steps, warmup=1, dtype="f32",
                    cpu_baseline={"value": ms, "unit": "ms/step", "cores": cores, "kind": "port",
                                  "sample": f"{steps} full decode steps of the same config, fp32 torch oracle"},
                    e2e={"value": ms, "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        print(json.dumps(line))
        return

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from megacute_b200.sharding import max_over_ranks, shard_range
    first_seq, n_seq = shard_range(a.batch * world, world, rank)       # weak scaling: batch_per_gpu sequences each
    assert n_seq == a.batch
    mc, g, params, st, ids, max_seq = build_workload(n_seq, a.ctx, dev, seed=rank)
    prog = mc.compile(g)
    emb = params["lm_head"]
    args = dict(params, **st)

    def step(ids):
        torch.index_select(emb, 0, ids, out=st["x"])       # embedding rows of this step's tokens, straight into x
        return mc.argmax(prog(**args))

    def reset_state():
        st["pos"].fill_(a.ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        fn(n)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / n, dev)        # device time, slowest rank

    cur = [ids]

    def run_steps(n):
        for i in range(n):
            if i % 100 == 99:
                reset_state()              # keep pos inside the cache (max_seq = ctx + 128)
            cur[0] = step(cur[0])

    def run_kernel_only(n):
        for i in range(n):
            if i % 100 == 99:
                reset_state()
            prog(**args)

    h_in = torch.empty(a.batch, dtype=torch.int64).pin_memory()
    h_out = torch.empty(a.batch, dtype=torch.int64).pin_memory()
    d_ids = torch.empty(a.batch, dtype=torch.int64, device=dev)

    def run_e2e(n):
        h_in.copy_(cur[0].cpu())
        for i in range(n):
            if i % 100 == 99:
                reset_state()
            d_ids.copy_(h_in, non_blocking=True)                 # host -> device: this step's token ids
            nxt = step(d_ids)
            h_out.copy_(nxt, non_blocking=True)                  # device -> host: the sampled tokens
            torch.cuda.current_stream().synchronize()
            h_in.copy_(h_out)

    run_steps(max(3, a.warmup))
    prog.check()
    reset_state()
    with ClockSampler(local) as cs:                  # clocks and throttle reasons over all three timed regions
        ms = timed(run_steps, a.steps)
        reset_state()
        kernel_ms = timed(run_kernel_only, a.steps)
        reset_state()
        e2e_ms = timed(run_e2e, a.steps)
    clocks = cs.summary()
    prog.check()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = peaks()
    avg_ctx = a.ctx + (a.steps - 1) / 2
    algo_bytes = WEIGHT_BYTES + a.batch * avg_ctx * KV_BYTES_PER_TOKEN
    achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
    line = dict(base, value=ms, ms_per_step=ms, tokens_per_s=world * a.batch * 1e3 / ms,
                e2e={"value": e2e_ms, "unit": "ms/step", "h2d_bytes_per_step": a.batch * 8,
                     "d2h_bytes_per_step": a.batch * 8},
                gpu_launches=2 * a.steps,        # per step: the megakernel and mk_argmax's kernel (+ torch's index_select)
                kernel_ms=kernel_ms, clocks=clocks,
                roofline={"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                          "peak_kind": peak_kind,
                          "traffic": MEASURED_TRAFFIC_B1_CTX1024 if (a.batch, a.ctx) == (1, 1024) else None, "algorithmic_bytes": algo_bytes,
                          "kernel": "mk::megakernel<false>"})
    if not a.no_cpu_baseline and world == 1:
        cpu_ms = cpu_oracle_ms(a.batch, a.ctx, 3)
        line["cpu_baseline"] = {"value": cpu_ms, "unit": "ms/step", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "3 full decode steps of the same config, fp32 torch oracle on host cores"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
