"""Step-graph IR for the recurrent-kernel lowering.

A traced single-timestep function (forward and its vector-Jacobian product,
see ``trace.py``) is held as a flat list of nodes over per-head 2-D values.
Every value has one of four *shape classes*, written ``(over_m, over_n)``:

    (1,1)  "MN"  a full [M,N] tile        (the state, outer products ...)
    (1,0)  "M1"  one value per row m      (v, dy, row sums ...)
    (0,1)  "1N"  one value per column n   (q, k, decay rows ...)
    (0,0)  "11"  one value per head       (beta, dt, gates ...)

The reference keeps the same information as FX code *text* that it re-parses
(flex_rnn/graph.py:8-41 in the reference project); here the FX node objects
are read directly, sums carry explicit ``over_m`` / ``over_n`` flags instead of
dim lists, and literal operands are kept as Python floats.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

Shape = Tuple[int, int]  # (over_m, over_n), each 0 or 1
Arg = Union[str, float]

MN: Shape = (1, 1)
M1: Shape = (1, 0)
N1: Shape = (0, 1)  # "1N": varies over n only
S11: Shape = (0, 0)

#: elementwise ops with one tensor operand
UNARY = ("neg", "exp", "log", "sqrt", "rsqrt", "reciprocal", "abs", "sigmoid",
         "tanh", "copy", "log1p", "expm1", "relu", "sign")
#: elementwise ops with two operands (either may be a literal)
BINARY = ("mul", "add", "sub", "div", "gt", "lt", "ge", "le", "eq", "ne",
          "maximum", "minimum", "pow")


@dataclass
class Node:
    name: str
    op: str                      # one of UNARY, BINARY, "sum", "const", "where"
    args: List[Arg]              # value names or float literals
    shape: Shape = S11
    over_m: bool = False         # "sum" only: reduce over rows
    over_n: bool = False         # "sum" only: reduce over columns

    def value_args(self) -> List[str]:
        return [a for a in self.args if isinstance(a, str)]


@dataclass
class StepGraph:
    """Topologically ordered nodes computing ``outputs`` from ``inputs``."""
    name: str
    inputs: List[str]
    nodes: List[Node]
    outputs: List[str]
    shape: Dict[str, Shape] = field(default_factory=dict)

    # -- queries ---------------------------------------------------------
    def node_map(self) -> Dict[str, Node]:
        return {n.name: n for n in self.nodes}

    def used_inputs(self) -> List[bool]:
        used = set()
        for n in self.nodes:
            used.update(n.value_args())
        used.update(self.outputs)
        return [i in used for i in self.inputs]

    def depends_on(self, seeds: Iterable[str]) -> set:
        """Names of all values that (transitively) depend on any seed."""
        dep = set(seeds)
        for n in self.nodes:
            if any(a in dep for a in n.value_args()):
                dep.add(n.name)
        return dep

    # -- transforms (all return new graphs) --------------------------------
    def pruned(self, outputs: Sequence[str], name: Optional[str] = None,
               leaves: Sequence[str] = ()) -> "StepGraph":
        """Sub-graph computing ``outputs``; values named in ``leaves`` are
        cut out of the graph and appended to the inputs instead."""
        leaves = list(leaves)
        need = set(outputs)
        keep: List[Node] = []
        for n in reversed(self.nodes):
            if n.name in need and n.name not in leaves:
                need.update(n.value_args())
                keep.append(n)
        keep.reverse()
        ins = [i for i in self.inputs] + [l for l in leaves if l in need]
        g = StepGraph(name or self.name, ins, keep, list(outputs), dict(self.shape))
        return g

    def count_mn_ops(self) -> int:
        """Number of [M,N]-sized elementwise ops plus reductions whose operand
        is [M,N]: the per-element op count K used for algorithmic flops."""
        k = 0
        for n in self.nodes:
            if n.op == "sum":
                if self.shape[n.args[0]] == MN:
                    k += 1
            elif n.op not in ("copy", "const") and n.shape == MN:
                k += 1
        return k

    def code(self) -> str:
        """Readable listing (debugging aid)."""
        tag = {MN: "MN", M1: "M1", N1: "1N", S11: "11"}
        lines = [f"def {self.name}({', '.join(self.inputs)}):"]
        for n in self.nodes:
            extra = ""
            if n.op == "sum":
                extra = f" over={'m' * n.over_m}{'n' * n.over_n}"
            lines.append(f"    {n.name} = {n.op}({', '.join(map(str, n.args))}){extra}  # {tag[n.shape]}")
        lines.append("    return " + ", ".join(self.outputs))
        return "\n".join(lines)


# ---------------------------------------------------------------------------
# FX -> StepGraph
# ---------------------------------------------------------------------------

_ATEN_UNARY = {
    "neg": "neg", "exp": "exp", "log": "log", "sqrt": "sqrt", "rsqrt": "rsqrt",
    "reciprocal": "reciprocal", "abs": "abs", "sigmoid": "sigmoid", "tanh": "tanh",
    "log1p": "log1p", "expm1": "expm1", "relu": "relu", "sign": "sign", "sgn": "sign",
}
_ATEN_BINARY = {
    "mul": "mul", "add": "add", "sub": "sub", "div": "div", "gt": "gt", "lt": "lt",
    "ge": "ge", "le": "le", "eq": "eq", "ne": "ne", "maximum": "maximum",
    "minimum": "minimum", "pow": "pow",
}
_ATEN_ALIAS = ("clone", "_to_copy", "expand", "alias", "detach", "lift_fresh_copy",
               "contiguous", "to", "view", "_unsafe_view", "reshape")


class UnsupportedStepOp(NotImplementedError):
    pass


def _shape_of(t) -> Shape:
    s = tuple(t.shape)
    if len(s) != 2:
        raise UnsupportedStepOp(f"step values must stay 2-D per head, got shape {s}")
    return (int(s[0] > 1), int(s[1] > 1))


def from_fx(gm: torch.fx.GraphModule, name: str, dims: Tuple[int, int]) -> StepGraph:
    """Convert a traced joint graph to a :class:`StepGraph`.

    ``dims`` is the ``(M, N)`` the trace was made with; both must be > 1 there
    (the tracer substitutes small stand-in sizes), so that every traced value's
    shape tells its class unambiguously.
    """
    M, N = dims
    alias: Dict[str, Arg] = {}
    shape: Dict[str, Shape] = {}
    inputs: List[str] = []
    nodes: List[Node] = []
    outputs: List[str] = []

    def res(a) -> Arg:
        if isinstance(a, torch.fx.Node):
            r = alias.get(a.name, a.name)
            return r
        if isinstance(a, bool):
            return float(a)
        if isinstance(a, (int, float)):
            return float(a)
        raise UnsupportedStepOp(f"unsupported operand {a!r}")

    def emit(nm, op, args, shp, **kw):
        nodes.append(Node(nm, op, list(args), shp, **kw))
        shape[nm] = shp

    def cls(v) -> Shape:
        s = tuple(v.shape)
        if len(s) == 0:
            return S11
        if len(s) != 2 or s[0] not in (1, M) or s[1] not in (1, N):
            raise UnsupportedStepOp(f"value of shape {s} is not a per-head [M|1, N|1] tile")
        return (int(s[0] > 1), int(s[1] > 1))

    for fx in gm.graph.nodes:
        if fx.op == "placeholder":
            inputs.append(fx.name)
            shape[fx.name] = cls(fx.meta["val"])
            continue
        if fx.op == "output":
            flat = fx.args[0]
            for o in flat:
                outputs.append(res(o))  # type: ignore[arg-type]
            continue
        if fx.op != "call_function":
            raise UnsupportedStepOp(f"unsupported FX node kind {fx.op}")
        target = fx.target
        tname = getattr(target, "__name__", str(target))
        base = tname.split(".")[0]
        val = fx.meta.get("val")
        shp = cls(val) if val is not None else S11
        if base in _ATEN_ALIAS:
            src = res(fx.args[0])
            if isinstance(src, str) and val is not None and base in ("view", "_unsafe_view", "reshape"):
                if cls(val) != shape[src] and tuple(val.shape) != tuple(fx.args[0].meta["val"].shape):
                    raise UnsupportedStepOp("reshaping a per-head tile is not supported")
            alias[fx.name] = src
            continue
        if base in _ATEN_UNARY:
            emit(fx.name, _ATEN_UNARY[base], [res(fx.args[0])], shp)
        elif base in _ATEN_BINARY:
            a, b = res(fx.args[0]), res(fx.args[1])
            op = _ATEN_BINARY[base]
            alpha = fx.kwargs.get("alpha", 1)
            if op in ("add", "sub") and alpha != 1:
                t = fx.name + "_alpha"
                bs = shape[b] if isinstance(b, str) else S11
                emit(t, "mul", [b, float(alpha)], bs)
                b = t
            emit(fx.name, op, [a, b], shp)
        elif base == "rsub":
            emit(fx.name, "sub", [res(fx.args[1]), res(fx.args[0])], shp)
        elif base == "sum":
            src = res(fx.args[0])
            if not isinstance(src, str):
                raise UnsupportedStepOp("sum of a literal")
            if len(fx.args) == 1:
                dims_ = [0, 1]
                keep = False
            else:
                dims_ = list(fx.args[1]) if fx.args[1] is not None else [0, 1]
                keep = bool(fx.args[2]) if len(fx.args) > 2 else bool(fx.kwargs.get("keepdim", False))
            dims_ = sorted({d % 2 for d in dims_})
            if not keep and len(tuple(val.shape)) != 0:
                raise UnsupportedStepOp("only sum(..., keepdim=True) keeps the per-head 2-D form")
            ss = shape[src]
            om, on = (0 in dims_) and bool(ss[0]), (1 in dims_) and bool(ss[1])
            if not om and not on:
                alias[fx.name] = src
                continue
            emit(fx.name, "sum", [src], (ss[0] * (not om), ss[1] * (not on)), over_m=om, over_n=on)
        elif base in ("ones_like", "zeros_like", "full_like", "full", "zeros", "ones",
                      "scalar_tensor", "new_zeros", "new_ones", "new_full"):
            if base in ("zeros_like", "zeros", "new_zeros"):
                c = 0.0
            elif base in ("ones_like", "ones", "new_ones"):
                c = 1.0
            elif base == "scalar_tensor":
                c = float(fx.args[0])
            elif base == "new_full":
                c = float(fx.args[2])
            else:
                c = float(fx.args[1])
            emit(fx.name, "const", [c], S11)
        elif base == "where":
            emit(fx.name, "where", [res(a) for a in fx.args[:3]], shp)
        elif base == "sigmoid_backward":   # grad * y * (1 - y)
            g, y = res(fx.args[0]), res(fx.args[1])
            t0, t1 = fx.name + "_a", fx.name + "_b"
            ys = shape[y] if isinstance(y, str) else S11
            emit(t0, "sub", [1.0, y], ys)
            emit(t1, "mul", [y, t0], ys)
            emit(fx.name, "mul", [g, t1], shp)
        elif base == "tanh_backward":      # grad * (1 - y*y)
            g, y = res(fx.args[0]), res(fx.args[1])
            t0, t1 = fx.name + "_a", fx.name + "_b"
            ys = shape[y] if isinstance(y, str) else S11
            emit(t0, "mul", [y, y], ys)
            emit(t1, "sub", [1.0, t0], ys)
            emit(fx.name, "mul", [g, t1], shp)
        else:
            raise UnsupportedStepOp(
                f"operation aten.{tname} is not supported inside a step function "
                "(supported: + - * / < > exp log sqrt and sum(-1, keepdim=True))")
    g = StepGraph(name, inputs, nodes, outputs, shape)
    return g
