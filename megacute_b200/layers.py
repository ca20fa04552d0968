"""Group the per-layer copies of an op into one *node*.

The reference merges the same op of every layer into one kernel node so that its JIT emits the
op's code once (``megacute/layers.py:86-154``); that needs per-layer buffers restacked with a
constant row stride.  This runtime's kernel is ahead-of-time and reads every op from a descriptor
table, so nothing has to be restacked: a node is only a reporting unit (``prog.nodes``, the rows of
``Timeline.summary``).  Ops belong to the same node when they are the n-th op of their layer, have
the same kind and the same operand shapes.
"""

from __future__ import annotations

from .graph import Graph


def _signature(op):
    views = tuple((name, v.shape, v.buf.kind in ("param", "input")) for name, v in op.view_fields())
    return (op.kind, views, getattr(op, "act", None), getattr(op, "fn", None), getattr(op, "splits", None))


def merge_layers(g: Graph) -> list[list[int]]:
    """-> groups of op indices, in order of first appearance; each group lists its ops by layer."""
    groups: dict[tuple, list[int]] = {}
    seen_in_layer: dict = {}
    order = []
    for k, op in enumerate(g.ops):
        if op.layer is None:
            key = ("single", k)
        else:
            idx = seen_in_layer.get(op.layer, 0)
            seen_in_layer[op.layer] = idx + 1
            key = (idx, _signature(op))
        if key not in groups:
            groups[key] = []
            order.append(key)
        groups[key].append(k)
    return [groups[key] for key in order]
