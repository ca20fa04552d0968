"""Generate the fixtures in this folder from the reference's own host code.

Run where a checkout of the reference is available (read-only is enough); MEGACUTE_REFERENCE names
its root:

    MEGACUTE_REFERENCE=<reference checkout> python tests/golden/gen_golden.py

What is recorded (the reference ships no tests or golden vectors of its own, and its device code
cannot run without a Blackwell GPU and nvidia-cutlass-dsl 4.8.0, so these are what the reference
*can* pin):
  graphs.json        structure of the graphs its example builders produce (examples/llama/model.py,
                     examples/dit/model.py): buffers, ops, operand windows, scalar attributes
  swiglu_weight.pt   megacute.swiglu_weight on a small seeded input
  oracle_small.pt    seeded inputs of two small graphs built by the REFERENCE's builders and the
                     fp32 oracle's outputs on them (ties the oracle's duck-typed reading of the
                     reference's op dataclasses to this repository's graphs)
  ref_passes.pt      for graphs built by the reference's builders: the oracle's result on the graph as
                     built, and on the graph rewritten by the REFERENCE's own passes
                     (megacute/runtime.py:44-199: fold_norms, split_k, fuse_rope_attention, split_kv).
                     Both must agree, which pins the oracle's reading of LinearSplit, SplitFinalize,
                     folded rms_eps over a derived weight and the fused DecodeAttention against the
                     reference's own rewrites
"""
import importlib.util
import json
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
import os

REF = pathlib.Path(os.environ.get("MEGACUTE_REFERENCE") or pathlib.Path(__file__).resolve().parents[3] / "reference")


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def dump_graph(g):
    """Structure of a graph, independent of which package built it."""
    ids = {b.id: n for n, b in enumerate(g.buffers)}
    view = lambda v: None if v is None else [ids[v.buf.id], v.row0, v.col0, v.rows, v.cols]
    ops = []
    for op in g.ops:
        d = {"kind": op.kind if isinstance(op.kind, str) else type(op).__name__, "layer": getattr(op, "layer", None)}
        fields = vars(op) if not hasattr(op, "__dataclass_fields__") else {k: getattr(op, k) for k in op.__dataclass_fields__}
        for k, v in sorted(fields.items()):
            if k in ("kind", "layer"):
                continue
            if hasattr(v, "buf"):
                d[k] = view(v)
            elif v is None or isinstance(v, (int, float, str, bool)):
                d[k] = v
        ops.append(d)
    return {"buffers": [[b.name, b.rows, b.cols, str(b.dtype), b.kind] for b in g.buffers],
            "ops": ops, "outputs": [view(v) for v in g.outputs]}


CONFIGS = {
    "llama_decode": dict(B=2, E=256, H=4, KVH=2, F=512, n=2, max_seq=256, vocab=1000, eps=1e-5),
    "llama_stack": dict(B=2, S=128, E=256, H=4, KVH=2, F=512, n=2, eps=1e-5),
    "dit_stack": dict(B=2, S=64, E=128, H=2, F=256, n=2),
}


PASS_CASES = {
    # name: (builder, kwargs, context length of the caches)
    "decode_b1_splitkv": ("llama_decode", dict(B=1, E=256, H=4, KVH=2, F=512, n=2, max_seq=1024, vocab=1000, eps=1e-5), 700),
    "decode_b2_fold": ("llama_decode", dict(B=2, E=256, H=4, KVH=2, F=512, n=2, max_seq=256, vocab=1000, eps=1e-5), 40),
    "decode_b16_splitk": ("llama_decode", dict(B=16, E=256, H=4, KVH=2, F=512, n=2, max_seq=256, vocab=1000, eps=1e-5), 90),
    "decode_b40_head_parallel": ("llama_decode", dict(B=40, E=512, H=8, KVH=8, F=512, n=1, max_seq=128, vocab=512, eps=1e-5), 30),
    "mlp_block": ("mlp_block", dict(M=136, E=256, F=512), 0),
    "dit_stack": ("dit_stack", dict(B=2, S=64, E=128, H=2, F=256, n=2), 0),
}


def pass_case_inputs(name):
    """Seeded inputs of a PASS_CASES entry (shared with tests/test_oracle.py)."""
    from megacute_b200 import workloads as W
    kind, c, ctx = PASS_CASES[name]
    if kind == "llama_decode":
        w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], 0, "cpu")
        st, ids = W.llama_decode_state(c["B"], c["E"], c["H"], c["KVH"], c["n"], c["max_seq"], ctx, c["vocab"], 1, "cpu")
        cos, sin = W.rope_tables(c["max_seq"], c["E"] // c["H"])
        st["x"] = w["lm_head"][ids].clone()
        return dict(cos=cos, sin=sin, **w, **st)
    if kind == "mlp_block":
        return W.mlp_block_inputs(c["M"], c["E"], c["F"], 0, "cpu")
    return W.dit_inputs(c["B"], c["S"], c["E"], c["F"], c["n"], 0, "cpu")


def ref_mlp_block(ref, M, E, F, eps=1e-5):
    """The single-block graph of the reference's README (README.md:14-20), on its own Graph class."""
    g = ref.Graph()
    x = g.input("x", (M, E))
    nw, w1, w2 = g.param("nw", (1, E)), g.param("w1", (2 * F, E)), g.param("w2", (E, F))
    g.output(g.linear(g.linear(g.rms_norm(x, nw, eps), w1, act="swiglu"), w2, residual=x))
    return g


def gen_ref_passes(ref, llama, dit):
    import importlib
    from oracle.graph_oracle import evaluate
    rt = importlib.import_module("megacute.runtime")
    out = {}
    for name, (kind, c, ctx) in PASS_CASES.items():
        g = {"llama_decode": llama.llama_decode, "dit_stack": dit.dit_stack,
             "mlp_block": lambda **kw: ref_mlp_block(ref, **kw)}[kind](**c)
        g2 = rt.split_kv(rt.fuse_rope_attention(rt.split_k(rt.fold_norms(g), 148)), 148)      # runtime.py:235
        t = pass_case_inputs(name)
        a, sa = evaluate(g, t)
        b, sb = evaluate(g2, t)
        rec = {"rewritten": b[0], "plain_vs_rewritten": float((a[0] - b[0]).norm() / a[0].norm()), "ops": [type(o).__name__ for o in g2.ops],
               "flags": sorted({k for o in g2.ops for k in ("rms_eps", "head_parallel", "k_new")
                                if getattr(o, k, None) not in (None, False)} |
                               ({"splits"} if any(getattr(o, "splits", 1) > 1 and type(o).__name__ == "DecodeAttention" for o in g2.ops) else set()) |
                               ({"derived"} if any(b_.kind == "derived" for b_ in g2.buffers) else set()))}
        if kind == "llama_decode":
            L = c["max_seq"]
            rows = [i * L + ctx for i in range(c["n"] * c["B"])]
            assert int(sa["pos"]) == int(sb["pos"]) == ctx + 1
            rec.update(pos_rewritten=sb["pos"], k_rows_rewritten=sb["k_cache"][rows].clone(),
                       v_rows_rewritten=sb["v_cache"][rows].clone(),
                       k_rows_equal=bool(torch.equal(sa["k_cache"][rows], sb["k_cache"][rows])))
        out[name] = rec
    torch.save(out, HERE / "ref_passes.pt")
    return out


def main():
    import megacute as ref                       # the reference package (PYTHONPATH)
    assert "reference" in str(pathlib.Path(ref.__file__).resolve()), ref.__file__
    llama = load(REF / "examples/llama/model.py", "ref_llama_model")
    dit = load(REF / "examples/dit/model.py", "ref_dit_model")
    graphs = {"llama_decode": llama.llama_decode(**CONFIGS["llama_decode"]),
              "llama_stack": llama.llama_stack(**CONFIGS["llama_stack"]),
              "dit_stack": dit.dit_stack(**CONFIGS["dit_stack"])}
    (HERE / "graphs.json").write_text(json.dumps({"configs": CONFIGS, "graphs": {k: dump_graph(g) for k, g in graphs.items()}}))

    gen = torch.Generator().manual_seed(3)
    gate, up = torch.randn(128, 16, generator=gen), torch.randn(128, 16, generator=gen)
    torch.save({"gate": gate, "up": up, "w": ref.swiglu_weight(gate, up)}, HERE / "swiglu_weight.pt")

    from oracle.graph_oracle import evaluate
    from megacute_b200 import workloads as W
    out = {}
    c = CONFIGS["llama_decode"]
    w = W.llama_weights(c["E"], c["H"], c["KVH"], c["F"], c["n"], c["vocab"], 0, "cpu")
    st, ids = W.llama_decode_state(c["B"], c["E"], c["H"], c["KVH"], c["n"], c["max_seq"], 40, c["vocab"], 1, "cpu")
    cos, sin = W.rope_tables(c["max_seq"], c["E"] // c["H"])
    st["x"] = w["lm_head"][ids].clone()
    o, s2 = evaluate(graphs["llama_decode"], dict(cos=cos, sin=sin, **w, **st))
    out["llama_decode"] = {"ids": ids, "logits": o[0], "pos": s2["pos"], "k_row": s2["k_cache"][40].clone()}
    c = CONFIGS["dit_stack"]
    t = W.dit_inputs(c["B"], c["S"], c["E"], c["F"], c["n"], 0, "cpu")
    o, _ = evaluate(graphs["dit_stack"], t)
    out["dit_stack"] = {"out": o[0]}
    torch.save(out, HERE / "oracle_small.pt")
    for name, rec in gen_ref_passes(ref, llama, dit).items():
        print(f"ref passes {name}: rel-L2 plain vs rewritten {rec['plain_vs_rewritten']:.2e}; flags {rec['flags']}; ops {sorted(set(rec['ops']))}")
    print("wrote", [p.name for p in HERE.iterdir()])


if __name__ == "__main__":
    main()
