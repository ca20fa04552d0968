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
"""

from __future__ import annotations

import json
from collections import defaultdict

import numpy as np

ROLES = ("producer", "compute")


class Timeline:
    def __init__(self, prog, buf: np.ndarray):
        self.prog = prog
        sms, roles, cap, _ = buf.shape
        idx = np.argwhere(buf[..., 1] != 0)
        self.records = [(int(sm), int(role), *(int(x) for x in buf[sm, role, ev])) for sm, role, ev in idx]
        self.t_base = min((r[3] for r in self.records), default=0)
        self.op_of = prog.sched.op_of

    def span_us(self) -> float:
        if not self.records:
            return 0.0
        return (max(r[5] for r in self.records) - self.t_base) / 1e3

    def _label(self, seq):
        k = int(self.op_of[seq])
        return f"{k}:{self.prog.g.ops[k].kind}"

    def summary(self) -> str:
        """Per node: instructions, first start, last end, mean dependency wait, mean busy time (us)."""
        agg = defaultdict(lambda: {"n": 0, "dep": 0.0, "busy": 0.0, "first": 1e30, "last": 0.0})
        for sm, role, seq, t0, t1, t2 in self.records:
            if role != 1:
                continue
            a = agg[self.prog.node_of[int(self.op_of[seq])][0]]
            a["n"] += 1
            a["dep"] += (t1 - t0) / 1e3
            a["busy"] += (t2 - t1) / 1e3
            a["first"] = min(a["first"], (t0 - self.t_base) / 1e3)
            a["last"] = max(a["last"], (t2 - self.t_base) / 1e3)
        lines = [f"launch span {self.span_us():.1f} us over {len({r[0] for r in self.records})} SMs; "
                 f"{sum(1 for r in self.records if r[1] == 1)} instructions traced",
                 f"{'node':<24}{'insts':>7}{'start':>9}{'end':>9}{'dep-wait/inst':>15}{'busy/inst':>12}"]
        for n in sorted(agg):
            a = agg[n]
            kind = self.prog.nodes[n][0].kind
            lines.append(f"{n:>3} {kind:<20}{a['n']:>7}{a['first']:>9.1f}{a['last']:>9.1f}"
                         f"{a['dep'] / a['n']:>15.2f}{a['busy'] / a['n']:>12.2f}")
        return "\n".join(lines)

    def chrome_events(self):
        ev = []
        us = lambda t: (t - self.t_base) / 1e3
        for sm, role, seq, t0, t1, t2 in self.records:
            name = self._label(seq)
            if role == 0:
                ev.append({"name": "stream " + name, "ph": "X", "pid": sm, "tid": ROLES[0], "ts": us(t0),
                           "dur": max(0.0, (t2 - t0) / 1e3), "args": {"inst": seq}})
            else:
                if t1 > t0:
                    ev.append({"name": "wait " + name, "ph": "X", "pid": sm, "tid": ROLES[1], "ts": us(t0),
                               "dur": (t1 - t0) / 1e3, "args": {"inst": seq}})
                ev.append({"name": name, "ph": "X", "pid": sm, "tid": ROLES[1], "ts": us(t1),
                           "dur": max(0.0, (t2 - t1) / 1e3), "args": {"inst": seq}})
        return ev

    def save_chrome(self, path):
        with open(path, "w") as f:
            json.dump({"traceEvents": self.chrome_events(), "displayTimeUnit": "ns"}, f)
        return path
