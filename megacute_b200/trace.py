"""In-kernel tracing: decode the per-SM globaltimer records of one launch.

    prog = mc.compile(g, trace=True); prog(**inputs)
    tl = prog.timeline(); print(tl.summary()); tl.save_chrome("trace.json")

Same surface as the reference's ``megacute/trace.py:22-91`` (records, span_us, summary,
chrome_events, save_chrome).  This kernel has three record kinds per SM:
  role 0 "producer": (seq, start of weight streaming, -, all copies of the instruction issued)
  role 1 "compute":  (seq, instruction fetched, dependencies met, arrivals published)
  role 2 "phases":   (seq, three op-internal marks) for the ops that wait for their own
                     dependencies: streaming linear (x staged, first stage landed, last group
                     done) and decode attention (tiles done, partial written, merged)
Times are globaltimer nanoseconds rebased to the earliest record.

The records are kept as one structured numpy table (``Timeline.table``) and every report is a
column operation on it; ``records`` is the same data as the reference's list of tuples.
"""

from __future__ import annotations

import json

import numpy as np

ROLES = ("producer", "compute", "phases")
_REC = np.dtype([("sm", np.int32), ("role", np.int32), ("seq", np.int64), ("t0", np.int64), ("t1", np.int64),
                 ("t2", np.int64)])


class Timeline:
    def __init__(self, prog, buf: np.ndarray):
        self.prog = prog
        self.op_of = np.asarray(prog.sched.op_of)
        sm, role, ev = np.nonzero(buf[..., 1])               # a record whose t0 is 0 was never written
        tab = np.empty(len(sm), _REC)
        tab["sm"], tab["role"] = sm, role
        for k, name in enumerate(("seq", "t0", "t1", "t2")):
            tab[name] = buf[sm, role, ev, k]
        self.table = tab
        self.t_base = int(tab["t0"].min()) if len(tab) else 0

    @property
    def records(self):
        """[(sm, role, seq, t0, t1, t2)] with plain ints, in (sm, role, slot) order."""
        return [tuple(int(x) for x in r) for r in self.table.tolist()]

    def _us(self, t):
        return (np.asarray(t, np.float64) - self.t_base) * 1e-3

    def span_us(self) -> float:
        return float(self._us(self.table["t2"].max())) if len(self.table) else 0.0

    def _label(self, seq) -> str:
        k = int(self.op_of[int(seq)])
        return f"{k}:{self.prog.g.ops[k].kind}"

    def node_table(self) -> np.ndarray:
        """One row per node that ran: node, instructions, first fetch, last publish, mean wait for
        dependencies and mean busy time per instruction (us), from the compute-role records."""
        c = self.table[self.table["role"] == 1]
        node = np.array([self.prog.node_of[int(k)][0] for k in self.op_of[c["seq"]]], np.int64)
        ids, inv, n = np.unique(node, return_inverse=True, return_counts=True)
        out = np.zeros(len(ids), [("node", np.int64), ("insts", np.int64), ("start", np.float64), ("end", np.float64),
                                  ("dep", np.float64), ("busy", np.float64)])
        out["node"], out["insts"] = ids, n
        first = np.full(len(ids), np.inf)
        last = np.full(len(ids), -np.inf)
        np.minimum.at(first, inv, self._us(c["t0"]))
        np.maximum.at(last, inv, self._us(c["t2"]))
        out["start"], out["end"] = first, last
        out["dep"] = np.bincount(inv, (c["t1"] - c["t0"]) * 1e-3, len(ids)) / n
        out["busy"] = np.bincount(inv, (c["t2"] - c["t1"]) * 1e-3, len(ids)) / n
        return out

    def summary(self) -> str:
        """Per node: instructions, first start, last end, mean dependency wait, mean busy time (us)."""
        tab = self.table
        head = (f"launch span {self.span_us():.1f} us over {len(np.unique(tab['sm']))} SMs; "
                f"{int((tab['role'] == 1).sum())} instructions traced")
        cols = f"{'node':<24}{'insts':>7}{'start':>9}{'end':>9}{'dep-wait/inst':>15}{'busy/inst':>12}"
        rows = [f"{int(r['node']):>3} {self.prog.nodes[int(r['node'])][0].kind:<20}{int(r['insts']):>7}{r['start']:>9.1f}"
                f"{r['end']:>9.1f}{r['dep']:>15.2f}{r['busy']:>12.2f}" for r in self.node_table()]
        return "\n".join([head, cols, *rows])

    def chrome_events(self):
        """Complete ("X") events, one process per SM and one thread per role: the producer's streaming
        span, and per instruction its dependency wait (when it had one) and its busy span."""
        tab = self.table
        out = []

        def emit(rows, prefix, tid, a, b):
            ts, dur = self._us(rows[a]), np.maximum(0.0, (rows[b] - rows[a]) * 1e-3)
            for r, t, d in zip(rows, ts.tolist(), dur.tolist()):
                out.append({"name": prefix + self._label(r["seq"]), "ph": "X", "pid": int(r["sm"]), "tid": tid, "ts": t,
                            "dur": d, "args": {"inst": int(r["seq"])}})

        emit(tab[tab["role"] == 0], "stream ", ROLES[0], "t0", "t2")
        comp = tab[tab["role"] == 1]
        emit(comp[comp["t1"] > comp["t0"]], "wait ", ROLES[1], "t0", "t1")
        emit(comp, "", ROLES[1], "t1", "t2")
        return out

    def save_chrome(self, path):
        doc = {"traceEvents": self.chrome_events(), "displayTimeUnit": "ns"}
        with open(path, "w") as f:
            json.dump(doc, f)
        return path
