"""megacute_b200: a B200-native persistent-megakernel runtime with the megacute Python API.

    import megacute_b200 as mc
    g = mc.Graph()
    x = g.input("x", (4096, 2048)); w = g.param("w", (8192, 2048))
    g.output(g.linear(x, w, act="gelu_tanh"))
    prog = mc.compile(g)
    y = prog(x=x_tensor, w=w_tensor)

The public names are those of the reference package (``megacute/__init__.py:11-17``): Graph, View,
Buffer, swiglu_weight, schedule, compile.  Importing this package also registers it under the
module name ``megacute`` (unless a package of that name is already imported), so graph builders
written as ``from megacute import Graph`` run unchanged.
"""

import sys as _sys

from .graph import Buffer, Graph, View, swiglu_weight  # noqa: F401
from .schedule import schedule  # noqa: F401


def compile(g, **kw):
    from .runtime import compile as _compile
    return _compile(g, **kw)


def argmax(logits, out=None):
    """Greedy sampling on the GPU (row-wise argmax of the logits); see ``runtime.argmax``."""
    from .runtime import argmax as _argmax
    return _argmax(logits, out)


_sys.modules.setdefault("megacute", _sys.modules[__name__])
