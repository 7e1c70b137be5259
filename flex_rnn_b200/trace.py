"""Tracing of a step function into a joint forward + backward graph.

The reference obtains the joint graph with ``functorch.compile.aot_function``
and, when a fake-tensor mode is active (that is, under ``torch.compile``),
re-runs the trace in a child process (flex_rnn/trace_isolated.py:3-39 in the
reference project).  Here the joint function ``(x, dy) -> (y, vjp(dy))`` is
traced in-process with ``make_fx`` on meta tensors.  For the duration of the
trace the dispatcher is put back into its plain eager state (active fake /
proxy modes suspended, the "below autograd" key exclusion that surrounds a
custom op's fake implementation lifted), so no child process is needed.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
from torch.fx.experimental.proxy_tensor import make_fx
from torch.utils._python_dispatch import _disable_current_modes

from .graph import StepGraph, from_fx

_TLS_INCLUDE = torch._C._dispatch_tls_local_include_set()
_TLS_EXCLUDE = torch._C._dispatch_tls_local_exclude_set()

#: stand-in sizes used while tracing; distinct and > 1 so that a traced
#: value's shape tells whether it varies over rows and/or columns
TRACE_M, TRACE_N = 3, 5


def as_tuple(x):
    return tuple(x) if isinstance(x, (tuple, list)) else (x,)


class clean_dispatch:
    """Context manager giving the dispatcher state of plain eager code: active
    fake / proxy modes are suspended and the thread-local dispatch-key sets are
    forced back to the values recorded when this module was imported (a custom
    op's fake implementation runs "below autograd", where ``torch.func.vjp``
    cannot work)."""

    def __enter__(self):
        self._a = torch._C._ForceDispatchKeyGuard(_TLS_INCLUDE, _TLS_EXCLUDE)
        self._b = _disable_current_modes()
        self._a.__enter__()
        self._b.__enter__()

    def __exit__(self, *exc):
        self._b.__exit__(*exc)
        self._a.__exit__(*exc)


def run_isolated(fn, *args):
    """Run ``fn(*args)`` with clean dispatcher state."""
    with clean_dispatch():
        return fn(*args)


def trace_joint(step: Callable, classes: Sequence[Tuple[int, int]], n_inputs: int,
                has_m: bool = True, has_n: bool = True,
                dims: Tuple[int, int] = (TRACE_M, TRACE_N)) -> Tuple[StepGraph, int, int]:
    with clean_dispatch():
        return _trace_joint(step, classes, n_inputs, has_m, has_n, dims)


def _trace_joint(step: Callable, classes: Sequence[Tuple[int, int]], n_inputs: int,
                 has_m: bool = True, has_n: bool = True,
                 dims: Tuple[int, int] = (TRACE_M, TRACE_N)) -> Tuple[StepGraph, int, int]:
    """Trace ``step`` on per-head tiles of ``dims`` = (rows, columns).

    The planner passes the real state size, as the reference does
    (flex_rnn/twopass.py:86-90), so that a step function that reads a size
    (``S.shape[-1] ** -0.5``) gets the constant it would get from ``naive``.

    ``classes[i]`` is ``(over_m, over_n)`` of argument ``i`` (inputs first, then
    states).  Returns the joint graph whose inputs are
    ``[*step args, *d_outputs, *d_new_states]`` and whose outputs are
    ``[*outputs, *new_states, *d_args]``, together with the number of outputs
    and of states.
    """
    tm = max(2, dims[0]) if has_m else 1
    tn = max(2, dims[1]) if has_n else 1
    if True:
        args = tuple(torch.empty(tm if c[0] else 1, tn if c[1] else 1, device="meta") for c in classes)
        counts: List[int] = []

        def flat(*a):
            y, s = step(*a)
            y, s = as_tuple(y), as_tuple(s)
            if not counts:
                counts.extend([len(y), len(s)])
            return tuple(t.float() for t in y) + tuple(t.float() for t in s)

        outs = flat(*args)
        n = len(args)

        def joint(*a):
            x, dy = a[:n], a[n:]
            y, pull = torch.func.vjp(flat, *x)
            return tuple(y) + tuple(pull(tuple(dy)))

        gm = make_fx(joint)(*args, *[torch.empty_like(o) for o in outs])
    g = from_fx(gm, "joint", (tm, tn))
    assert len(g.inputs) == n + len(outs)
    assert len(g.outputs) == len(outs) + n
    return g, counts[0], counts[1]
