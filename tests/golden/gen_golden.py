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
    print("wrote", [p.name for p in HERE.iterdir()])


if __name__ == "__main__":
    main()
