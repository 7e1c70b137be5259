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
         "tanh", "copy", "log1p", "expm1", "relu", "sign", "erf")
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

    def simplified_products(self) -> "StepGraph":
        """The same function with fewer full-tile operations, by two rewrites that only reassociate products:

        * a sum of an outer product, ``sum(a[M,1] * b[1,N])``, is a vector times a sum:
          over rows ``b * sum(a)``, over columns ``a * sum(b)``;
        * a product of a tile with two lower-rank factors in a row, ``(T * s) * y``, is ``T * (s * y)`` when
          ``s * y`` is itself lower-rank and ``T * s`` has no other use.

        (Rounding differs in the last bit from the unsimplified order.)"""
        nodes = [Node(n.name, n.op, list(n.args), n.shape, n.over_m, n.over_n) for n in self.nodes]
        shape = dict(self.shape)
        fresh = [0]

        def new_name(base: str) -> str:
            fresh[0] += 1
            return f"{base}_r{fresh[0]}"

        def join(a: Shape, b: Shape) -> Shape:
            return (max(a[0], b[0]), max(a[1], b[1]))

        changed = True
        while changed:
            changed = False
            uses: Dict[str, int] = {}
            for n in nodes:
                for a in n.value_args():
                    uses[a] = uses.get(a, 0) + 1
            for o in self.outputs:
                uses[o] = uses.get(o, 0) + 1
            by_name = {n.name: n for n in nodes}
            for idx, n in enumerate(nodes):
                # sum of an outer product
                if n.op == "sum" and isinstance(n.args[0], str) and n.args[0] in by_name and uses.get(n.args[0], 0) == 1:
                    pr = by_name[n.args[0]]
                    if pr.op == "mul" and pr.shape == MN and all(isinstance(a, str) for a in pr.args):
                        sa, sb = shape[pr.args[0]], shape[pr.args[1]]
                        if {sa, sb} == {M1, N1}:
                            a_m = pr.args[0] if sa == M1 else pr.args[1]
                            b_n = pr.args[1] if sa == M1 else pr.args[0]
                            repl: List[Node] = []
                            fa, fb = a_m, b_n
                            if n.over_m:
                                fa = new_name(n.name)
                                repl.append(Node(fa, "sum", [a_m], S11, True, False))
                                shape[fa] = S11
                            if n.over_n:
                                fb = new_name(n.name)
                                repl.append(Node(fb, "sum", [b_n], S11, False, True))
                                shape[fb] = S11
                            repl.append(Node(n.name, "mul", [fa, fb], n.shape))
                            nodes[idx:idx + 1] = repl
                            nodes.remove(pr)
                            changed = True
                            break
                # (T * s) * y  ->  T * (s * y)
                if n.op == "mul" and n.shape == MN and all(isinstance(a, str) for a in n.args):
                    for k in (0, 1):
                        x, y = n.args[k], n.args[1 - k]
                        m1 = by_name.get(x)
                        if (m1 is None or m1.op != "mul" or m1.shape != MN or uses.get(x, 0) != 1 or shape[y] == MN
                                or not all(isinstance(a, str) for a in m1.args)):
                            continue
                        for j in (0, 1):
                            tile, s = m1.args[j], m1.args[1 - j]
                            if shape[tile] == MN and shape[s] != MN and join(shape[s], shape[y]) != MN:
                                sy = new_name(n.name)
                                shape[sy] = join(shape[s], shape[y])
                                nodes[idx:idx + 1] = [Node(sy, "mul", [s, y], shape[sy]), Node(n.name, "mul", [tile, sy], MN)]
                                nodes.remove(m1)
                                changed = True
                                break
                        if changed:
                            break
                    if changed:
                        break
        return StepGraph(self.name, list(self.inputs), nodes, list(self.outputs), shape)

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
    "log1p": "log1p", "expm1": "expm1", "relu": "relu", "sign": "sign", "sgn": "sign", "erf": "erf",
}
_ATEN_BINARY = {
    "mul": "mul", "add": "add", "sub": "sub", "div": "div", "gt": "gt", "lt": "lt",
    "ge": "ge", "le": "le", "eq": "eq", "ne": "ne", "maximum": "maximum",
    "minimum": "minimum", "pow": "pow", "clamp_min": "maximum", "clamp_max": "minimum",
    "logical_and": "mul", "bitwise_and": "mul",      # operands are 0/1 masks here
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
        # an in-place form (autograd formulas use a few: fill_, sub_, logical_and_) is imported as the
        # out-of-place operation, and later readers of the overwritten tensor are pointed at the result
        mutated = None
        if base.endswith("_") and (base[:-1] in _ATEN_UNARY or base[:-1] in _ATEN_BINARY or base[:-1] == "fill"):
            mutated, base = fx.args[0], base[:-1]
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
        elif base == "mean":
            src = res(fx.args[0])
            dims_ = list(fx.args[1]) if len(fx.args) > 1 and fx.args[1] is not None else [0, 1]
            keep = bool(fx.args[2]) if len(fx.args) > 2 else bool(fx.kwargs.get("keepdim", False))
            if not isinstance(src, str) or (not keep and len(tuple(val.shape)) != 0):
                raise UnsupportedStepOp("only mean(..., keepdim=True) keeps the per-head 2-D form")
            full = tuple(fx.args[0].meta["val"].shape)
            dims_ = sorted({d % 2 for d in dims_})
            count = 1
            for d in dims_:
                count *= full[d]
            ss = shape[src]
            om, on = (0 in dims_) and bool(ss[0]), (1 in dims_) and bool(ss[1])
            cur = src
            if om or on:
                emit(fx.name + "_sum", "sum", [src], (ss[0] * (not om), ss[1] * (not on)), over_m=om, over_n=on)
                cur = fx.name + "_sum"
            # a broadcast dimension counts in the mean's divisor but not in the sum
            kept = (full[0] if (0 in dims_ and not om) else 1) * (full[1] if (1 in dims_ and not on) else 1)
            emit(fx.name, "mul", [cur, float(kept) / float(count)], shape[cur])
        elif base in ("ones_like", "zeros_like", "full_like", "full", "zeros", "ones", "fill", "empty_like", "empty",
                      "scalar_tensor", "new_zeros", "new_ones", "new_full", "new_empty"):
            if base in ("zeros_like", "zeros", "new_zeros", "empty_like", "empty", "new_empty"):
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
        elif base == "threshold_backward":   # grad * (x > threshold)
            g, x, thr = res(fx.args[0]), res(fx.args[1]), float(fx.args[2])
            xs = shape[x] if isinstance(x, str) else S11
            emit(fx.name + "_m", "gt", [x, thr], xs)
            emit(fx.name, "mul", [g, fx.name + "_m"], shp)
        elif base == "clamp":                # max(min(x, hi), lo)
            x = res(fx.args[0])
            lo = fx.args[1] if len(fx.args) > 1 else fx.kwargs.get("min")
            hi = fx.args[2] if len(fx.args) > 2 else fx.kwargs.get("max")
            cur = x
            if lo is not None:
                emit(fx.name + "_lo", "maximum", [cur, res(lo)], shp)
                cur = fx.name + "_lo"
            if hi is not None:
                emit(fx.name + "_hi", "minimum", [cur, res(hi)], shp)
                cur = fx.name + "_hi"
            alias[fx.name] = cur
        elif base in ("masked_fill", "masked_fill_"):   # where(mask, value, x)
            x, m, v = res(fx.args[0]), res(fx.args[1]), res(fx.args[2])
            emit(fx.name, "where", [m, v, x], shp)
            if base.endswith("_") and isinstance(fx.args[0], torch.fx.Node):
                alias[fx.args[0].name] = fx.name        # later readers of the mutated tensor see the new value
        elif base in ("elu", "elu_backward"):
            t = lambda k: f"{fx.name}_{k}"
            if base == "elu":
                x, rest = res(fx.args[0]), list(fx.args[1:])
            else:
                if bool(fx.args[4]):
                    raise UnsupportedStepOp("elu_backward on the result is not supported")
                x, rest = res(fx.args[5]), list(fx.args[1:4])
            alpha, scale, iscale = [float(v) for v in rest + [1.0, 1.0, 1.0][len(rest):]]
            xs = shape[x] if isinstance(x, str) else S11
            emit(t("p"), "gt", [x, 0.0], xs)
            emit(t("z"), "mul", [x, iscale], xs)
            emit(t("e"), "exp", [t("z")], xs)
            if base == "elu":                  # scale * (x > 0 ? x : alpha * (exp(input_scale x) - 1))
                emit(t("m"), "sub", [t("e"), 1.0], xs)
                emit(t("a"), "mul", [t("m"), alpha], xs)
                emit(t("w"), "where", [t("p"), x, t("a")], xs)
                emit(fx.name, "mul", [t("w"), scale], shp)
            else:                              # grad * scale * (x > 0 ? 1 : alpha * input_scale * exp(input_scale x))
                emit(t("a"), "mul", [t("e"), alpha * iscale], xs)
                emit(t("w"), "where", [t("p"), 1.0, t("a")], xs)
                emit(t("s"), "mul", [t("w"), scale], xs)
                emit(fx.name, "mul", [res(fx.args[0]), t("s")], shp)
        elif base == "logical_not":
            emit(fx.name, "sub", [1.0, res(fx.args[0])], shp)
        elif base in ("silu", "silu_backward", "softplus", "softplus_backward", "gelu", "gelu_backward"):
            grad = res(fx.args[0]) if base.endswith("_backward") else None
            x = res(fx.args[1] if grad is not None else fx.args[0])
            xs = shape[x] if isinstance(x, str) else S11
            t = lambda k: f"{fx.name}_{k}"
            if base.startswith("silu"):
                emit(t("s"), "sigmoid", [x], xs)
                if grad is None:
                    emit(fx.name, "mul", [x, t("s")], shp)
                else:                        # s * (1 + x * (1 - s))
                    emit(t("a"), "sub", [1.0, t("s")], xs)
                    emit(t("b"), "mul", [x, t("a")], xs)
                    emit(t("c"), "add", [t("b"), 1.0], xs)
                    emit(t("d"), "mul", [t("s"), t("c")], xs)
                    emit(fx.name, "mul", [grad, t("d")], shp)
            elif base.startswith("softplus"):
                rest = fx.args[2:] if grad is not None else fx.args[1:]
                beta = float(rest[0]) if len(rest) > 0 else float(fx.kwargs.get("beta", 1.0))
                thr = float(rest[1]) if len(rest) > 1 else float(fx.kwargs.get("threshold", 20.0))
                emit(t("z"), "mul", [x, beta], xs)
                emit(t("big"), "gt", [t("z"), thr], xs)
                if grad is None:             # log1p(exp(beta x)) / beta, x itself above the threshold
                    emit(t("zc"), "minimum", [t("z"), thr], xs)
                    emit(t("e"), "exp", [t("zc")], xs)
                    emit(t("l"), "log1p", [t("e")], xs)
                    emit(t("v"), "mul", [t("l"), 1.0 / beta], xs)
                    emit(fx.name, "where", [t("big"), x, t("v")], shp)
                else:
                    emit(t("s"), "sigmoid", [t("z")], xs)
                    emit(t("w"), "where", [t("big"), 1.0, t("s")], xs)
                    emit(fx.name, "mul", [grad, t("w")], shp)
            else:
                approx = fx.kwargs.get("approximate", "none")
                if approx != "none":
                    raise UnsupportedStepOp("gelu(approximate='tanh') is not supported inside a step function")
                emit(t("u"), "mul", [x, 0.7071067811865476], xs)
                emit(t("e"), "erf", [t("u")], xs)
                emit(t("c"), "add", [t("e"), 1.0], xs)
                emit(t("h"), "mul", [t("c"), 0.5], xs)             # Phi(x)
                if grad is None:
                    emit(fx.name, "mul", [x, t("h")], shp)
                else:                        # Phi(x) + x * phi(x)
                    emit(t("x2"), "mul", [x, x], xs)
                    emit(t("n"), "mul", [t("x2"), -0.5], xs)
                    emit(t("p"), "exp", [t("n")], xs)
                    emit(t("q"), "mul", [t("p"), 0.3989422804014327], xs)
                    emit(t("r"), "mul", [x, t("q")], xs)
                    emit(t("d"), "add", [t("h"), t("r")], xs)
                    emit(fx.name, "mul", [grad, t("d")], shp)
        else:
            raise UnsupportedStepOp(
                f"operation aten.{tname} is not supported inside a step function "
                "(supported: + - * / comparisons, where, exp log sqrt tanh sigmoid relu silu softplus gelu erf "
                "abs sign clamp maximum minimum pow, and sum(-1, keepdim=True))")
        if mutated is not None and isinstance(mutated, torch.fx.Node):
            alias[mutated.name] = alias.get(fx.name, fx.name)
    g = StepGraph(name, inputs, nodes, outputs, shape)
    return g
