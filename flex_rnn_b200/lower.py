"""Lowering of step graphs to sm_100a CUDA source (forward and backward kernel).

This replaces the reference's string-template generator (flex_rnn/to_cuda.py
and the three kernel templates in flex_rnn/twopass.py:202-339 of the reference
project).  Kernel shape, fixed for every step function:

* one CTA per (batch b, head h, tile of MB state rows); a thread owns R rows x
  C columns of every fp32 state in registers, L = N/C lanes of a warp share a
  row and 32/L row groups share a warp;
* ``sum(-1, keepdim)`` = in-thread sum over C then a warp-shuffle butterfly
  over the L lanes; no block barrier is needed for it;
* the per-timestep inputs are staged D timesteps ahead into a two-deep shared
  memory ring: 16-byte aligned contiguous rows by 1-D TMA bulk copies
  (``cp.async.bulk``) that complete on an mbarrier, anything else (scalars,
  odd strides) by plain loads held in registers for one chunk;
* the forward writes an fp32 state checkpoint every ``dck`` steps and the
  row sums the backward needs (``aux``);
* the backward is one reverse-time kernel: per checkpoint chunk it rebuilds
  the chunk's states (segment bases kept in shared-memory slots, states inside
  a segment recomputed from the base), keeps dstate in registers, writes
  per-row gradients directly and reduces per-column / per-head gradient
  partials over the row groups of the CTA through shared memory.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from .graph import MN, M1, N1, S11, Node, Shape, StepGraph

DT_F32, DT_BF16, DT_F16, DT_F64 = 0, 1, 2, 3
ELT = {DT_F32: 4, DT_BF16: 2, DT_F16: 2, DT_F64: 8}
CTYPE = {DT_F32: "float", DT_BF16: "u16", DT_F16: "u16", DT_F64: "double"}

ERR_STAGE_TIMEOUT = 1      # a staged-input TMA copy did not complete in time
ERR_CKPT_TIMEOUT = 2       # a checkpoint TMA copy did not complete in time


class LoweringError(NotImplementedError):
    pass


@dataclass
class TensorSpec:
    """Shape, element strides, dtype code and base alignment of one tensor."""
    shape: Tuple[int, ...]
    stride: Tuple[int, ...]
    dt: int
    aligned16: bool = True

    def st(self, dim: int) -> int:
        return self.stride[dim] if self.shape[dim] > 1 else 0


@dataclass
class Tile:
    """Thread tiling of one kernel."""
    R: int          # state rows per thread
    C: int          # state columns per thread
    MB: int         # state rows per CTA
    M: int
    N: int

    def __post_init__(self):
        assert self.N % self.C == 0 and self.MB % self.R == 0 and self.M % self.MB == 0
        self.L = self.N // self.C                # lanes per row
        assert self.L <= 32 and 32 % self.L == 0, "a state row must fit in one warp"
        self.G = 32 // self.L                    # row groups per warp
        self.V = 4 if self.C % 4 == 0 else (2 if self.C % 2 == 0 else 1)
        self.NCH = self.C // self.V              # column chunks per thread
        self.RG = self.MB // self.R              # row groups per CTA
        self.NT = self.RG * self.L               # threads per CTA
        assert self.NT % 32 == 0, f"CTA of {self.NT} threads is not a whole number of warps"
        assert self.NT <= 1024

    def col(self, j: int, e: int = 0) -> str:
        """C expression: global column of chunk j, element e."""
        return f"(cb + {j * self.V * self.L + e})"


def choose_tile(M: int, N: int, want_r: int, want_c: int, want_mb: Optional[int] = None) -> Tile:
    """Largest legal tile not exceeding the wanted R x C (powers of two)."""
    def pow2_le(x):
        return 1 << (max(1, x).bit_length() - 1)
    # columns per thread: N / L for a power-of-two number of lanes L <= 32, as close to the wish as possible
    cands = [N // L for L in (1, 2, 4, 8, 16, 32) if N % L == 0]
    if not cands:
        raise LoweringError(f"N={N} cannot be split over the lanes of a warp")
    C = min(cands, key=lambda c: (abs(math.log2(c) - math.log2(max(1, want_c))), -c))
    R = min(pow2_le(want_r), M)
    while M % R:
        R //= 2
    MB = M if want_mb is None else min(want_mb, M)
    while M % MB or MB % R:
        MB += 1
    L = N // C
    # a CTA must be whole warps and at most 1024 threads
    while (MB // R) * L > 1024:
        if R * 2 <= MB and M % (R * 2) == 0 and MB % (R * 2) == 0:
            R *= 2
        else:
            raise LoweringError("cannot fit the row tile in one CTA")
    while ((MB // R) * (N // C)) % 32:
        if R > 1:
            R //= 2
        elif MB < M:
            MB = min(M, MB * 2)
            while M % MB:
                MB += 1
        elif C > 1 and C % 2 == 0 and N // (C // 2) <= 32:
            C //= 2
        else:
            raise LoweringError(f"state {M}x{N} is too small for a 32-thread CTA")
    return Tile(R, C, MB, M, N)


@dataclass
class StagedItem:
    """One per-timestep vector staged through shared memory."""
    key: str                 # graph value name it feeds (or aux/dy tag)
    cls: Shape               # N1 (row), M1 (col) or S11 (scalar)
    dt: int
    ptr: str                 # kernel parameter name
    length: int              # elements per timestep inside the CTA
    base: str                # C expr: element offset of (b, t=0, h, m0)
    stride_t: int            # elements between timesteps
    inner: int               # element stride inside the vector
    tma: bool
    off: int = 0             # byte offset inside a stage buffer
    rowb: int = 0            # bytes per timestep inside the stage buffer
    tmap: Optional[dict] = None   # tensor-map description when the item is fetched by one tiled TMA load per chunk


@dataclass
class KernelSource:
    name: str
    source: str
    grid: Tuple[int, int, int]
    block: int
    smem_bytes: int
    params: List[str]        # parameter names in order
    param_decl: List[str] = field(default_factory=list)   # C declarations of the parameters
    info: Dict[str, object] = field(default_factory=dict)
    tmaps: List[dict] = field(default_factory=list)       # tensor maps to encode per launch (see KernelBuilder.plan)


# ---------------------------------------------------------------------------
# small code-writer
# ---------------------------------------------------------------------------

class W:
    def __init__(self):
        self.lines: List[str] = []
        self.ind = 0

    def __call__(self, s: str = ""):
        for ln in s.split("\n"):
            self.lines.append(("  " * self.ind + ln) if ln else "")

    def open(self, s: str):
        self(s + " {")
        self.ind += 1

    def close(self, s: str = ""):
        self.ind -= 1
        self("}" + s)

    def text(self) -> str:
        return "\n".join(self.lines) + "\n"


def flit(x: float) -> str:
    if math.isinf(x):
        return "(-INFINITY)" if x < 0 else "INFINITY"
    if math.isnan(x):
        return "NAN"
    s = repr(float(x))
    if "e" not in s and "." not in s:
        s += ".0"
    return s + "f"


def vname(n: str) -> str:
    return "v_" + n.replace(".", "_")


def _pick_cnt(maxcnt: int, dt: int, *aligns: int) -> int:
    """Largest power-of-two element count <= maxcnt such that 16 bytes is not
    exceeded and every given element offset granularity is a multiple of it."""
    cnt = 1
    while (cnt * 2 <= maxcnt and maxcnt % (cnt * 2) == 0 and cnt * 2 * ELT[dt] <= 16
           and all(a % (cnt * 2) == 0 for a in aligns)):
        cnt *= 2
    return cnt


# ---------------------------------------------------------------------------
# graph body emission
# ---------------------------------------------------------------------------

def op_expr(n: Node, a: List[str]) -> str:
    """C expression of one elementwise node given its operand expressions."""
    op = n.op
    if op == "mul":
        return f"{a[0]} * {a[1]}"
    if op == "add":
        return f"{a[0]} + {a[1]}"
    if op == "sub":
        return f"{a[0]} - {a[1]}"
    if op == "div":
        return f"frnn_divf({a[0]}, {a[1]})"
    if op == "neg":
        return f"-{a[0]}"
    if op in ("copy", "const"):
        return a[0]
    if op == "exp":
        return f"frnn_expf({a[0]})"
    if op == "log":
        return f"frnn_logf({a[0]})"
    if op == "sqrt":
        return f"frnn_sqrtf({a[0]})"
    if op == "rsqrt":
        return f"frnn_rcpf(frnn_sqrtf({a[0]}))"
    if op == "reciprocal":
        return f"frnn_rcpf({a[0]})"
    if op == "erf":
        return f"erff({a[0]})"
    if op == "abs":
        return f"fabsf({a[0]})"
    if op == "sigmoid":
        return f"frnn_rcpf(1.0f + frnn_expf(-{a[0]}))"
    if op == "tanh":
        return f"(1.0f - 2.0f * frnn_rcpf(1.0f + frnn_expf(2.0f * {a[0]})))"
    if op == "log1p":
        return f"frnn_logf(1.0f + {a[0]})"
    if op == "expm1":
        return f"(frnn_expf({a[0]}) - 1.0f)"
    if op == "relu":
        return f"fmaxf({a[0]}, 0.0f)"
    if op == "sign":
        return f"(({a[0]} > 0.0f) ? 1.0f : (({a[0]} < 0.0f) ? -1.0f : 0.0f))"
    if op in ("gt", "lt", "ge", "le", "eq", "ne"):
        sym = {"gt": ">", "lt": "<", "ge": ">=", "le": "<=", "eq": "==", "ne": "!="}[op]
        return f"(({a[0]} {sym} {a[1]}) ? 1.0f : 0.0f)"
    if op == "maximum":
        return f"fmaxf({a[0]}, {a[1]})"
    if op == "minimum":
        return f"fminf({a[0]}, {a[1]})"
    if op == "pow":
        if not isinstance(n.args[1], str) and float(n.args[1]) == 2.0:
            return f"{a[0]} * {a[0]}"
        if not isinstance(n.args[1], str) and float(n.args[1]) == 3.0:
            return f"{a[0]} * {a[0]} * {a[0]}"
        return f"powf({a[0]}, {a[1]})"
    if op == "where":
        return f"(({a[0]} != 0.0f) ? {a[1]} : {a[2]})"
    raise LoweringError(f"no lowering for op {op}")


class Body:
    """Emits per-thread code for graph nodes over R x C register tiles."""

    def __init__(self, w: W, tile: Tile, shapes: Dict[str, Shape], pack2: bool = False, col_major: bool = False,
                 max_acc: int = 4):
        self.w = w
        self.max_acc = max(1, max_acc)   # independent accumulators per kept element of a sum
        self.t = tile
        self.shape = dict(shapes)
        self.pack2 = pack2            # packed fp32x2 arithmetic for column-varying values
        self.col_major = col_major    # full-tile loops with the columns outermost
        self.partial: Dict[str, bool] = {}     # value is a per-row-group partial sum
        self.alias: Dict[str, str] = {}        # value name -> name of the register tile that holds it
        self.fused: Dict[str, Node] = {}       # products folded into the packed FMA of their only consumer
        self.predeclared: set = set()          # values whose register arrays are declared in an enclosing scope

    # -- packed fp32x2 arithmetic (sm_100 `fma.rn.f32x2`) ---------------------------------------
    # Values that vary along the columns are processed two columns at a time: one packed instruction
    # does the work of two scalar ones, which halves the issue slots the arithmetic needs (the scan
    # kernels are issue-bound, not pipe-bound).  The register arrays stay scalar; a pair is
    # (x[c], x[c+1]) and ptxas allocates it to an aligned register pair.
    def can_pack(self) -> bool:
        return self.pack2 and self.t.C % 2 == 0

    def child(self) -> "Body":
        """A body for a nested scope: sees this body's values, keeps the same options."""
        return Body(self.w, self.t, self.shape, self.pack2, self.col_major, self.max_acc)

    def varies_c(self, a) -> bool:
        return isinstance(a, str) and bool(self.shape[a][1])

    def pair(self, a, r: str, c: str, neg: bool = False) -> str:
        """float2 expression of operand ``a`` at columns (c, c+1) of row r."""
        sg = "-" if neg else ""
        if self.varies_c(a):
            assert not neg
            return f"frnn_pk_make({self.at(a, r, c)}, {self.at(a, r, c + ' + 1')})"
        x = self.at(a, r, c)
        return f"frnn_pk_make({sg}({x}), {sg}({x}))"

    def fuse_group(self, group: Sequence[Node], all_nodes: Sequence[Node], keep: Iterable[str]):
        """Choose the products of ``group`` to fold into their consumer: a
        product used exactly once, by an add / sub of its own shape or by a sum,
        emitted in the same group, and not needed by anyone else."""
        if not self.can_pack():
            return
        keep = set(keep)
        uses: Dict[str, int] = {}
        for n in all_nodes:
            for a in n.value_args():
                uses[a] = uses.get(a, 0) + 1
        by_name = {n.name: n for n in group}
        for u in group:
            for a in u.value_args():
                m = by_name.get(a)
                if m is None or m.op != "mul" or uses.get(a, 0) != 1 or a in keep or not m.shape[1]:
                    continue
                ok = False
                if u.op == "add" and u.shape == m.shape:
                    ok = True
                elif u.op == "sub" and u.shape == m.shape:
                    other = u.args[0] if u.args[1] == a else u.args[1]
                    if u.args[1] == a:            # z - x*y: negate a factor that is cheap to negate
                        ok = any(not self.varies_c_node(x, by_name, all_nodes) for x in m.args)
                    else:                         # x*y - z
                        ok = not self.varies_c_node(other, by_name, all_nodes)
                elif u.op == "sum" and u.args[0] == a:
                    ok = self._pair_sum_mode(u, m.shape) is not None
                if ok:
                    self.fused[a] = m
                    break                         # one product per consumer

    def varies_c_node(self, a, by_name, all_nodes) -> bool:
        if not isinstance(a, str):
            return False
        if a in self.shape:
            return bool(self.shape[a][1])
        for n in all_nodes:
            if n.name == a:
                return bool(n.shape[1])
        return True

    def _fma_operands(self, u: Node, r: str, c: str) -> Optional[Tuple[str, str, str]]:
        """(X, Y, Z) with u = X*Y + Z for an add / sub with a folded product."""
        for k, a in enumerate(u.args):
            if isinstance(a, str) and a in self.fused:
                m, z = self.fused[a], u.args[1 - k]
                x, y = m.args
                if u.op == "add":
                    return self.pair(x, r, c), self.pair(y, r, c), self.pair(z, r, c)
                if k == 1:                        # z - x*y
                    if not self.varies_c(x):
                        return self.pair(x, r, c, neg=True), self.pair(y, r, c), self.pair(z, r, c)
                    return self.pair(x, r, c), self.pair(y, r, c, neg=True), self.pair(z, r, c)
                return self.pair(x, r, c), self.pair(y, r, c), self.pair(z, r, c, neg=True)   # x*y - z
        return None

    def pair_expr(self, n: Node, r: str, c: str) -> Optional[str]:
        """Packed expression of an elementwise node, or None if it has none."""
        if n.op not in ("add", "sub", "mul") or not n.shape[1]:
            return None
        f = self._fma_operands(n, r, c) if n.op in ("add", "sub") else None
        if f:
            return f"frnn_fma2({f[0]}, {f[1]}, {f[2]})"
        a, b = n.args
        if n.op == "mul":
            return f"frnn_mul2({self.pair(a, r, c)}, {self.pair(b, r, c)})"
        if n.op == "add":
            return f"frnn_add2({self.pair(a, r, c)}, {self.pair(b, r, c)})"
        if not self.varies_c(b):
            return f"frnn_add2({self.pair(a, r, c)}, {self.pair(b, r, c, neg=True)})"
        return f"frnn_fma2({self.pair(b, r, c)}, frnn_pk_make(-1.0f, -1.0f), {self.pair(a, r, c)})"

    def pair_loops(self, s: Shape, body):
        """Like loops() for a column-varying shape, two columns per iteration."""
        w = self.w
        opened = 0
        if s[0]:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {self.t.R}; r++)")
            opened += 1
        w("#pragma unroll")
        w.open(f"for (int c = 0; c < {self.t.C}; c += 2)")
        w(body("r" if s[0] else "0", "c"))
        for _ in range(opened + 1):
            w.close()

    # element accessor of a value (or literal) at tile position (r, c)
    def at(self, a, r: str, c: str) -> str:
        if not isinstance(a, str):
            return flit(a)
        s = self.shape[a]
        n = vname(self.alias.get(a, a))
        if s == MN:
            return f"{n}[{r}*{self.t.C}+{c}]"
        if s == M1:
            return f"{n}[{r}]"
        if s == N1:
            return f"{n}[{c}]"
        return f"{n}[0]"

    def size(self, s: Shape) -> int:
        return (self.t.R if s[0] else 1) * (self.t.C if s[1] else 1)

    def declare(self, name: str, s: Shape):
        self.shape[name] = s
        if name not in self.predeclared:
            self.w(f"float {vname(name)}[{self.size(s)}];")

    def loops(self, s: Shape, body):
        w = self.w
        order = [(1, "c", self.t.C), (0, "r", self.t.R)] if (self.col_major and s == MN) else \
                [(0, "r", self.t.R), (1, "c", self.t.C)]
        opened = 0
        for dim, var, ext in order:
            if s[dim]:
                w("#pragma unroll")
                w.open(f"for (int {var} = 0; {var} < {ext}; {var}++)")
                opened += 1
        w(body("r" if s[0] else "0", "c" if s[1] else "0"))
        for _ in range(opened):
            w.close()

    def _check_partial(self, n: Node) -> bool:
        """Propagate the 'partial over row groups' property; only operations
        linear in the partial value keep the deferred reduction valid."""
        ps = [isinstance(a, str) and self.partial.get(a, False) for a in n.args]
        if not any(ps):
            return False
        ok = False
        if n.op in ("neg", "copy"):
            ok = True
        elif n.op == "mul":
            ok = sum(ps) == 1
        elif n.op in ("add", "sub"):
            ok = all(ps) and all(isinstance(a, str) for a in n.args)
        elif n.op == "div":
            ok = ps[0] and not ps[1]
        elif n.op == "sum":
            ok = not n.over_m
        if ok and n.shape[0] == 0:
            for a, p in zip(n.args, ps):
                if isinstance(a, str) and not p and self.shape[a][0]:
                    ok = False
        if not ok or n.shape[0]:
            raise LoweringError(
                f"value {n.name} applies a non-linear or row-dependent operation to a "
                "sum over rows; this backward form is not supported")
        return True

    def node(self, n: Node, allow_over_m: bool):
        w, t = self.w, self.t
        if n.name in self.fused:
            # evaluated inside its consumer; only the bookkeeping happens here
            self.partial[n.name] = self._check_partial(n)
            self.shape[n.name] = n.shape
            return
        if n.op == "sum" and self.can_pack() and self._pair_sum(n, allow_over_m):
            return
        if n.op == "sum":
            src = n.args[0]
            ss = self.shape[src]
            if n.over_m and not allow_over_m:
                raise LoweringError("Only torch.sum(x, dim=-1, keepdim=True) is supported in the forward pass")
            if n.over_m and self.partial.get(src, False):
                raise LoweringError("nested sums over rows are not supported")
            self.partial[n.name] = bool(n.over_m) or self._check_partial(n)
            self.declare(n.name, n.shape)
            rs = "r" if n.shape[0] else "0"
            cs = "c" if n.shape[1] else "0"
            # independent accumulators for every kept element, filled with the reduced
            # index outermost so that consecutive FMAs belong to different chains
            red_r = n.over_m and ss[0]
            red_c = n.over_n and ss[1]
            kept = self.size(n.shape)
            chain = (t.R if red_r else 1) * (t.C if red_c else 1)
            nacc = max(1, min(4, self.max_acc, chain // 4))
            while kept * nacc > 32 and nacc > 1:
                nacc //= 2
            w.open("")
            w(f"float acc[{kept * nacc}];")
            w("#pragma unroll")
            w(f"for (int q = 0; q < {kept * nacc}; q++) acc[q] = 0.0f;")
            # loop nest: reduced dims outside, kept dims inside
            opened = 0
            if red_r:
                w("#pragma unroll")
                w.open(f"for (int r = 0; r < {t.R}; r++)")
                opened += 1
            if red_c:
                w("#pragma unroll")
                w.open(f"for (int c = 0; c < {t.C}; c++)")
                opened += 1
            if n.shape[0]:
                w("#pragma unroll")
                w.open(f"for (int r = 0; r < {t.R}; r++)")
                opened += 1
            if n.shape[1]:
                w("#pragma unroll")
                w.open(f"for (int c = 0; c < {t.C}; c++)")
                opened += 1
            kidx = "0"
            if n.shape == M1:
                kidx = "r"
            elif n.shape == N1:
                kidx = "c"
            ridx = "c" if red_c else "r"
            if red_r and red_c:
                ridx = f"(r * {t.C} + c)"
            w(f"acc[({kidx}) * {nacc} + ({ridx}) % {nacc}] += {self.at(src, 'r', 'c')};")
            for _ in range(opened):
                w.close()
            # totals, then (for sums over n) the butterflies of all kept elements together
            w("#pragma unroll")
            w.open(f"for (int k = 0; k < {kept}; k++)")
            tot = " + ".join(f"acc[k * {nacc} + {q}]" for q in range(nacc))
            if nacc == 4:
                tot = f"(acc[k * 4] + acc[k * 4 + 1]) + (acc[k * 4 + 2] + acc[k * 4 + 3])"
            w(f"{vname(n.name)}[k] = {tot};")
            w.close()
            if red_c and t.L > 1:
                off = t.L // 2
                while off > 0:
                    w("#pragma unroll")
                    w(f"for (int k = 0; k < {kept}; k++) {vname(n.name)}[k] += frnn_shfl_xor({vname(n.name)}[k], {off});")
                    off //= 2
            w.close()
            return
        self.partial[n.name] = self._check_partial(n)
        self.declare(n.name, n.shape)
        if self.can_pack() and self.pair_expr(n, "r", "c") is not None:
            self.pair_loops(n.shape, lambda r, c: (
                f"{{ const frnn_pk v2 = {self.pair_expr(n, r, c)}; "
                f"{self.at(n.name, r, c)} = v2.x; {self.at(n.name, r, c + ' + 1')} = v2.y; }}"))
            return
        self.loops(n.shape, lambda r, c: f"{self.at(n.name, r, c)} = {op_expr(n, [self.at(x, r, c) for x in n.args])};")

    @staticmethod
    def _pair_sum_mode(n: Node, ss: Shape) -> Optional[Tuple[bool, bool]]:
        """(rows reduced, columns reduced) if the packed form applies to this sum."""
        if not ss[1]:
            return None
        red_r = bool(n.over_m and ss[0])
        red_c = bool(n.over_n)
        if not (red_r or red_c) or (n.shape[1] and red_c):
            return None
        return red_r, red_c

    def _pair_sum(self, n: Node, allow_over_m: bool) -> bool:
        """Sum of a column-varying value with packed accumulators: over the
        columns (both lanes are partial sums, added at the end) or over the rows
        (the kept columns go in pairs).  False: not applicable, use the scalar form."""
        w, t = self.w, self.t
        src = n.args[0]
        ss = self.shape[src]
        mode = self._pair_sum_mode(n, ss)
        if mode is None:
            return False
        red_r, red_c = mode
        if n.over_m and not allow_over_m:
            raise LoweringError("Only torch.sum(x, dim=-1, keepdim=True) is supported in the forward pass")
        if n.over_m and self.partial.get(src, False):
            raise LoweringError("nested sums over rows are not supported")
        self.partial[n.name] = bool(n.over_m) or self._check_partial(n)
        self.declare(n.name, n.shape)
        m = self.fused.get(src)
        keep_r = bool(n.shape[0])
        if red_c:
            kept = t.R if keep_r else 1
            chain = (t.C // 2) * (t.R if red_r else 1)
        else:
            kept = t.C // 2
            chain = t.R
        nacc = max(1, min(2 if red_c else 4, self.max_acc, chain // 4))
        while kept * nacc > 16 and nacc > 1:
            nacc //= 2
        w.open("")
        w(f"frnn_pk acc2[{kept * nacc}];")
        w("#pragma unroll")
        w(f"for (int q = 0; q < {kept * nacc}; q++) acc2[q] = frnn_pk_make(0.0f, 0.0f);")
        opened = 0
        if ss[0]:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            opened += 1
        w("#pragma unroll")
        w.open(f"for (int c = 0; c < {t.C}; c += 2)")
        opened += 1
        rs = "r" if ss[0] else "0"
        if red_c:
            kidx = "r" if keep_r else "0"
            ridx = f"(r * {t.C // 2} + (c >> 1))" if red_r else "(c >> 1)"
        else:
            kidx, ridx = "(c >> 1)", "r"
        acc = f"acc2[({kidx}) * {nacc} + ({ridx}) % {nacc}]"
        if m is not None:
            x, y = m.args
            w(f"{acc} = frnn_fma2({self.pair(x, rs, 'c')}, {self.pair(y, rs, 'c')}, {acc});")
        else:
            w(f"{acc} = frnn_add2({acc}, {self.pair(src, rs, 'c')});")
        for _ in range(opened):
            w.close()
        w("#pragma unroll")
        w.open(f"for (int k = 0; k < {kept}; k++)")
        tot = f"acc2[k * {nacc}]"
        for q in range(1, nacc):
            tot = f"frnn_add2({tot}, acc2[k * {nacc} + {q}])"
        if nacc == 4:
            tot = f"frnn_add2(frnn_add2(acc2[k * 4], acc2[k * 4 + 1]), frnn_add2(acc2[k * 4 + 2], acc2[k * 4 + 3]))"
        w(f"const frnn_pk tot = {tot};")
        if red_c:
            w(f"{vname(n.name)}[k] = tot.x + tot.y;")
        else:
            w(f"{vname(n.name)}[2 * k] = tot.x; {vname(n.name)}[2 * k + 1] = tot.y;")
        w.close()
        if red_c and t.L > 1:
            off = t.L // 2
            while off > 0:
                w("#pragma unroll")
                w(f"for (int k = 0; k < {kept}; k++) {vname(n.name)}[k] += frnn_shfl_xor({vname(n.name)}[k], {off});")
                off //= 2
        w.close()
        return True

    def graph(self, g: StepGraph, allow_over_m: bool = False, keep: Iterable[str] = ()):
        self.fuse_group(g.nodes, g.nodes, set(g.outputs) | set(keep))
        for n in g.nodes:
            self.node(n, allow_over_m)


# ---------------------------------------------------------------------------
# problem description shared by both kernels
# ---------------------------------------------------------------------------

@dataclass
class Problem:
    B: int
    T: int
    H: int
    M: int
    N: int
    inputs: List[TensorSpec]             # 5-D specs of the step inputs
    in_names: List[str]                  # graph value name of each input
    states: List[TensorSpec]             # 4-D specs of the initial states
    st_names: List[str]
    out_dt: List[int]                    # dtype code of each output
    naux: int

    def in_cls(self, i: int) -> Shape:
        s = self.inputs[i].shape
        return (int(s[3] > 1), int(s[4] > 1))

    def st_cls(self) -> Shape:
        return (int(self.M > 1), int(self.N > 1))


def _elem_off(spec: TensorSpec, dims: Sequence[Tuple[int, str]]) -> str:
    """C expression (long) sum of idx*stride over the given (dim, index expr)."""
    terms = [f"(long)({e})*{spec.st(d)}L" for d, e in dims if spec.st(d) != 0]
    return " + ".join(terms) if terms else "0L"


def _spec_bytes(spec: TensorSpec) -> int:
    """Bytes from the tensor's first element to the end of its last one."""
    if any(n == 0 for n in spec.shape):
        return 0
    return (1 + sum((n - 1) * s for n, s in zip(spec.shape, spec.stride) if n > 1)) * ELT[spec.dt]


def _contig(shape: Sequence[int]) -> Tuple[int, ...]:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return tuple(reversed(st))


def _merge_nodes(graphs: Sequence[StepGraph]) -> List[Node]:
    seen, out = set(), []
    for g in graphs:
        for n in g.nodes:
            if n.name not in seen:
                seen.add(n.name)
                out.append(n)
    return out


class KernelBuilder:
    """Staging machinery shared by the forward and backward emitters:

    raw ring   two buffers of D timesteps of every per-timestep vector in its
               I/O dtype, filled by TMA bulk copies (or plain loads);
    work buf   one buffer of D timesteps in fp32 holding what the scan loop
               actually reads: converted inputs plus every value of the step
               graph that depends on inputs only and is not a full tile
               ("hoisted": e.g. beta*k, v - aux, exp(dt*A)), computed once per
               CTA by all threads when a raw chunk has arrived.
    """

    def __init__(self, p: Problem, tile: Tile, dstage: int, use_tma: bool):
        self.p = p
        self.t = tile
        self.D = dstage
        self.use_tma = use_tma
        self.w = W()
        self.items: List[StagedItem] = []
        self.params: List[str] = []
        self.param_decl: List[str] = []
        self.param_bytes: Dict[str, int] = {}
        self.const_scalars: Dict[str, str] = {}    # time-invariant [1,1] inputs kept in registers
        self.tensor_tma = True                     # use tiled tensor-map loads where possible

    # -- parameters ----------------------------------------------------------
    def add_param(self, name: str, ctype: str, const: bool, nbytes: int = 0):
        """``nbytes``: how many bytes from the pointer on the kernel may touch
        (what the checked build registers for this parameter)."""
        self.params.append(name)
        q = "const " if const else ""
        r = " __restrict__" if const else ""
        self.param_decl.append(f"{q}{ctype}*{r} {name}")
        self.param_bytes[name] = int(nbytes)

    def emit_bounds_prologue(self):
        """Checked build only: thread 0 registers every pointer parameter with
        its byte extent and the CTA's dynamic shared memory, then the CTA
        synchronises.  ``@SMEM_BYTES@`` is filled in when the source is final."""
        w = self.w
        w("#ifdef FRNN_BOUNDS")
        w.open("if (threadIdx.x == 0)")
        w("frnn_bounds_begin(err, smem, @SMEM_BYTES@L);")
        for name, nbytes in self.param_bytes.items():
            w(f"frnn_bounds_add({name}, {nbytes}L);")
        w.close()
        w("frnn_block_sync();")
        w("#endif")

    # -- raw staging plan ------------------------------------------------------
    def add_item(self, key: str, cls: Shape, spec: TensorSpec, ptr: str, dims: Dict[str, int], const_off: int = 0):
        """``dims`` maps 'b','t','h','v' (the vector dim) to tensor dim indices;
        ``const_off`` is a constant element offset added to the tensor's base."""
        t = self.t
        length = {N1: self.p.N, M1: t.MB, S11: 1}[cls]
        inner = spec.st(dims["v"]) if cls != S11 else 1
        base_dims = [(dims["b"], "b"), (dims["h"], "h")]
        if cls == M1:
            base_dims.append((dims["v"], "m0"))
        base = _elem_off(spec, base_dims)
        e = ELT[spec.dt]
        st_t = spec.st(dims["t"])
        tma = (self.use_tma and cls != S11 and (inner == 1 or length == 1) and spec.aligned16
               and (length * e) % 16 == 0 and (st_t * e) % 16 == 0
               and (spec.st(dims["b"]) * e) % 16 == 0 and (spec.st(dims["h"]) * e) % 16 == 0
               and (cls != M1 or (t.MB * spec.st(dims["v"]) * e) % 16 == 0))
        rowb = (length * e + 15) // 16 * 16
        if const_off:
            base = f"{const_off}L + " + base
        item = StagedItem(key, cls, spec.dt, ptr, length, base, st_t, inner, tma, 0, rowb)
        # a dim of extent > 1 with stride 0 (an input expanded over B, T or H) has no tensor-map form:
        # such inputs take the per-timestep bulk copies, which index with the given strides
        expanded = any(spec.shape[dims[d]] > 1 and spec.stride[dims[d]] == 0 for d in ("b", "t", "h", "v"))
        if (tma and self.tensor_tma and not expanded and length <= 256 and self.D <= 256
                and (const_off * e) % 16 == 0):
            # one 4-D box (vector, head, D timesteps, batch) per chunk instead of one bulk copy per timestep
            ext = lambda d: spec.shape[d] if spec.shape[d] > 1 else 1
            pad = max(16, (ext(dims["v"]) * e + 15) // 16 * 16)
            stb = lambda d: spec.st(d) * e if spec.st(d) else pad
            item.tmap = {
                "src": ptr, "off_bytes": const_off * e, "elt": e,
                "dims": [ext(dims["v"]), ext(dims["h"]), ext(dims["t"]), ext(dims["b"])],
                "strides_bytes": [stb(dims["h"]), stb(dims["t"]), stb(dims["b"])],
                "box": [length, 1, self.D, 1],
                "coord": ["m0" if cls == M1 else "0", "h" if spec.st(dims["h"]) else "0", None,
                          "b" if spec.st(dims["b"]) else "0"],
            }
        self.items.append(item)

    def plan(self, graphs: Sequence[StepGraph], outputs_needed: Sequence[str] = ()) -> List[StepGraph]:
        """Lay out the raw ring, decide what is hoisted into the work buffer and
        return the graphs rewritten to read those values as inputs."""
        off = 0
        for it in sorted(self.items, key=lambda i: not i.tma):
            if it.tma and it.tmap:
                off = (off + 127) // 128 * 128     # a tiled tensor copy needs a 128-byte aligned destination
            it.off = off
            off += it.rowb * self.D
        self.stage_bytes = (off + 127) // 128 * 128
        self.tma_items = [i for i in self.items if i.tma]
        self.plain_items = [i for i in self.items if not i.tma]
        self.item_by_key = {i.key: i for i in self.items}
        self.tmaps: List[dict] = []
        for k, it in enumerate(i for i in self.tma_items if i.tmap):
            it.tmap["name"] = f"tm{k}"
            it.tmap["param_index"] = len(self.params)
            it.tmap["src_index"] = self.params.index(it.tmap["src"])
            self.params.append(f"tm{k}")
            self.param_decl.append(f"FRNN_TMAP_PARAM tm{k}")
            self.tmaps.append(it.tmap)

        avail: Dict[str, Shape] = {i.key: i.cls for i in self.items}
        for nm in self.const_scalars:
            avail[nm] = S11
        self.hoisted: List[Node] = []
        for n in _merge_nodes(graphs):
            if n.op == "sum" or n.shape == MN or n.name in avail:
                continue
            if all(a in avail for a in n.value_args()):
                avail[n.name] = n.shape
                self.hoisted.append(n)
        hoisted_names = {n.name for n in self.hoisted}
        used_outside = set(outputs_needed)
        for g in graphs:
            for n in g.nodes:
                if n.name not in hoisted_names:
                    used_outside.update(n.value_args())
            used_outside.update(g.outputs)
        frontier = [nm for nm in avail if nm in used_outside and nm not in self.const_scalars]
        # work-buffer layout: per timestep all 1N values, then M1, then scalars
        self.wk: Dict[str, Tuple[Shape, int]] = {}
        pos = 0
        for cls, ln in ((N1, self.p.N), (M1, self.t.MB), (S11, 1)):
            pos = (pos + 3) // 4 * 4
            for nm in frontier:
                if avail[nm] == cls:
                    self.wk[nm] = (cls, pos)
                    pos += ln
        self.wk_row = (pos + 3) // 4 * 4
        self.wk_bytes = (self.wk_row * 4 * self.D + 127) // 128 * 128 if self.wk else 0
        self.avail = avail
        out = []
        for g in graphs:
            g2 = g.pruned(g.outputs, g.name, leaves=[nm for nm in frontier if nm not in g.inputs])
            out.append(g2)
        return out

    # -- code pieces -------------------------------------------------------------
    def emit_thread_ids(self):
        w, t = self.w, self.t
        w("const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;")
        w(f"const int l = lane % {t.L}, g = lane / {t.L};")
        w(f"const int rg = warp * {t.G} + g;   // row group inside the CTA")
        w(f"const int m0 = blockIdx.x * {t.MB}, h = blockIdx.y, b = blockIdx.z;")
        w(f"const int row0 = m0 + rg * {t.R};  // first state row of this thread")
        w(f"const int cb = {t.V} * l;          // first state column of this thread")
        w("(void)row0; (void)cb; (void)m0; (void)h; (void)b; (void)warp;")

    def emit_tma_issue(self, fn: str):
        """Device function issuing the TMA copies of one chunk (warp 0 calls):
        one tiled tensor-map load per item where a map exists, else one 1-D
        bulk copy per item and timestep."""
        w = self.w
        tens = [i for i in self.tma_items if i.tmap]
        flat = [i for i in self.tma_items if not i.tmap]
        n = len(flat)
        flat_bytes = sum(i.length * ELT[i.dt] for i in flat)
        tens_bytes = sum(i.length * ELT[i.dt] * self.D for i in tens)
        w(f"// TMA copies of one chunk: {len(tens)} tiled loads of {self.D} timesteps, "
          f"{n} bulk copies per timestep")
        uniq = self._uniq_ptr_items(flat)
        args = [f"const void* {i.ptr}" for i in uniq] + [f"const frnn_tmap* {i.tmap['name']}" for i in tens]
        self.tma_issue_call = ", ".join([i.ptr for i in uniq] + [f"&{i.tmap['name']}" for i in tens])
        w.open(f"FRNN_DEV void {fn}(unsigned char* stage, u64* bar, int t0, int nv, int lane, int b, int h, int m0"
               + (", " + ", ".join(args) if args else "") + ")")
        if self.tma_items:
            w.open("if (lane == 0)")
            w(f"frnn_mbar_expect_tx(bar, {tens_bytes}u + (u32)nv * {flat_bytes}u);")
            for it in tens:
                c = it.tmap["coord"]
                w(f"frnn_tma_load_4d(stage + {it.off}, {it.tmap['name']}, {c[0]}, {c[1]}, t0, {c[3]}, bar);")
            w.close()
        if n:
            w("frnn_warp_sync();")
            w.open(f"for (int i = lane; i < nv * {n}; i += 32)")
            w(f"const int k = i % {n}, tl = i / {n};")
            w.open("switch (k)")
            for k, it in enumerate(flat):
                e = ELT[it.dt]
                w(f"case {k}: frnn_bulk_g2s_c(stage + {it.off} + tl * {it.rowb}, "
                  f"(const unsigned char*){it.ptr} + ({it.base} + (long)(t0 + tl) * {it.stride_t}L) * {e}, "
                  f"{it.length * e}u, bar); break;")
            w.close()
            w.close()
        w.close()
        w()

    @staticmethod
    def _uniq_ptr_items(items):
        seen, out = set(), []
        for i in items:
            if i.ptr not in seen:
                seen.add(i.ptr)
                out.append(i)
        return out

    def plain_regs(self) -> List[Tuple[StagedItem, int]]:
        """(item, registers per thread) for the register-prefetched items."""
        return [(it, (self.D * it.length + self.t.NT - 1) // self.t.NT) for it in self.plain_items]

    def emit_plain_decl(self):
        for k, (it, cnt) in enumerate(self.plain_regs()):
            self.w(f"{CTYPE[it.dt]} pl{k}[{cnt}];")

    def emit_plain_load(self, t0: str, nv: str):
        """Plain global loads of one chunk into registers (no wait on them)."""
        w, t = self.w, self.t
        for k, (it, cnt) in enumerate(self.plain_regs()):
            w("#pragma unroll")
            w.open(f"for (int q = 0; q < {cnt}; q++)")
            w(f"const int e = tid + q * {t.NT}, tl = e / {it.length}, j = e % {it.length};")
            w(f"pl{k}[q] = 0;")
            w(f"if (tl < {nv}) pl{k}[q] = frnn_ld_raw<{CTYPE[it.dt]}>({it.ptr}, "
              f"{it.base} + (long)({t0} + tl) * {it.stride_t}L + (long)j * {it.inner}L);")
            w.close()

    def emit_plain_direct(self, stage: str, t0: str, nv: str, tidv: str, nthr: int):
        """Threads ``tidv`` in [0, nthr): copy one chunk of the plainly loaded
        items from global memory straight into the raw stage buffer."""
        w = self.w
        for it in self.plain_items:
            w.open(f"for (int e = {tidv}; e < ({nv}) * {it.length}; e += {nthr})")
            w(f"const int tl = e / {it.length}, j = e % {it.length};")
            w(f"(({CTYPE[it.dt]}*)({stage} + {it.off} + tl * {it.rowb}))[j] = frnn_ld_raw<{CTYPE[it.dt]}>({it.ptr}, "
              f"{it.base} + (long)({t0} + tl) * {it.stride_t}L + (long)j * {it.inner}L);")
            w.close()

    def emit_plain_store(self, stage: str):
        w, t = self.w, self.t
        for k, (it, cnt) in enumerate(self.plain_regs()):
            w("#pragma unroll")
            w.open(f"for (int q = 0; q < {cnt}; q++)")
            w(f"const int e = tid + q * {t.NT}, tl = e / {it.length}, j = e % {it.length};")
            w(f"if (tl < {self.D}) (({CTYPE[it.dt]}*)({stage} + {it.off} + tl * {it.rowb}))[j] = pl{k}[q];")
            w.close()

    def emit_convert(self, raw: str, wk: str, nv: str, tidv: str = "tid", nthr: Optional[int] = None):
        """Threads ``tidv`` in [0, nthr) (default: the whole CTA): raw chunk -> fp32
        work buffer, evaluating hoisted nodes."""
        w, t = self.w, self.t
        nthr = nthr or t.NT
        hoisted = {n.name: n for n in self.hoisted}

        def closure(targets: List[str]) -> List[str]:
            need, order = set(), []

            def visit(nm):
                if nm in need:
                    return
                need.add(nm)
                if nm in hoisted:
                    for a in hoisted[nm].value_args():
                        visit(a)
                order.append(nm)
            for tg in targets:
                visit(tg)
            return order

        for cls, ln in ((N1, self.p.N), (M1, t.MB), (S11, 1)):
            targets = [nm for nm, (c, _) in self.wk.items() if c == cls]
            if not targets:
                continue
            order = closure(targets)
            vw = 4 if ln % 4 == 0 else (2 if ln % 2 == 0 else 1)   # elements per thread and iteration
            w.open(f"for (int e = {tidv}; e < {nv} * {ln // vw}; e += {nthr})")
            w(f"const int tl = e / {ln // vw}, i = (e % {ln // vw}) * {vw}; (void)i;")

            def one(c, cls=cls):
                # a value of another class inside this loop has one element (a column vector of a one-row state,
                # say): it is read like a scalar
                return c == S11 or c != cls
            for nm in order:
                hn = "h_" + nm.replace(".", "_")
                if nm in hoisted:
                    n = hoisted[nm]
                    width = 1 if one(n.shape) else vw
                    w(f"float {hn}[{width}];")
                    for q in range(width):
                        ops = []
                        for a in n.args:
                            if not isinstance(a, str):
                                ops.append(flit(a))
                            else:
                                aw = 1 if one(self.avail[a]) else vw
                                ops.append(f"h_{a.replace('.', '_')}[{q if aw > 1 else 0}]")
                        w(f"{hn}[{q}] = {op_expr(n, ops)};")
                elif nm in self.const_scalars:
                    w(f"float {hn}[1]; {hn}[0] = {self.const_scalars[nm]};")
                else:
                    it = self.item_by_key[nm]
                    if one(it.cls):
                        w(f"float {hn}[1]; {hn}[0] = frnn_io<{it.dt}>::ld({raw} + {it.off} + tl * {it.rowb}, 0);")
                    else:
                        w(f"float {hn}[{vw}]; frnn_ldv<{it.dt},{vw}>({raw} + {it.off} + tl * {it.rowb}, i, {hn});")
            for nm in targets:
                hn = "h_" + nm.replace(".", "_")
                if cls == S11:
                    w(f"{wk}[tl * {self.wk_row} + {self.wk[nm][1]}] = {hn}[0];")
                else:
                    w(f"frnn_stv<0,{vw}>({wk}, tl * {self.wk_row} + {self.wk[nm][1]} + i, {hn});")
            w.close()

    def emit_wk_read(self, body: Body, name: str, wkt: str):
        """Read one work-buffer value of the current timestep into registers.
        ``wkt`` points at the timestep's row of the work buffer."""
        w, t = self.w, self.t
        cls, off = self.wk[name]
        body.declare(name, cls)
        n = vname(name)
        if cls == N1:
            cnt = _pick_cnt(t.V, DT_F32)
            for j in range(t.NCH):
                for q in range(t.V // cnt):
                    w(f"frnn_ldv<0,{cnt}>({wkt}, {off} + cb + {j * t.V * t.L + q * cnt}, &{n}[{j * t.V + q * cnt}]);")
        elif cls == M1:
            cnt = _pick_cnt(t.R, DT_F32, t.R)
            for q in range(t.R // cnt):
                w(f"frnn_ldv<0,{cnt}>({wkt}, {off} + rg * {t.R} + {q * cnt}, &{n}[{q * cnt}]);")
        else:
            w(f"{n}[0] = {wkt}[{off}];")

    def emit_const_input(self, body: Body, name: str, cls: Shape, spec: TensorSpec, ptr: str,
                         dims: Dict[str, int]):
        """Load a time-invariant input straight from global memory (once)."""
        w, t = self.w, self.t
        body.declare(name, cls)
        n = vname(name)
        base = _elem_off(spec, [(dims["b"], "b"), (dims["h"], "h")])
        if cls == S11:
            w(f"{n}[0] = frnn_io<{spec.dt}>::ld({ptr}, {base});")
            return
        if cls == N1:
            for j in range(t.NCH):
                for e in range(t.V):
                    w(f"{n}[{j * t.V + e}] = frnn_io<{spec.dt}>::ld({ptr}, {base} + (long){t.col(j, e)} * {spec.st(dims['n'])}L);")
        elif cls == M1:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            w(f"{n}[r] = frnn_io<{spec.dt}>::ld({ptr}, {base} + (long)(row0 + r) * {spec.st(dims['m'])}L);")
            w.close()
        else:
            self.emit_tile_global(n, spec, ptr, base, dims["m"], dims["n"], load=True)

    def emit_tile_global(self, arr: str, spec: TensorSpec, ptr: str, base: str, dm: int, dn: int,
                         load: bool, add: bool = False):
        """Strided global load / store of an R x C register tile (any strides)."""
        w, t = self.w, self.t
        sm, sn = spec.st(dm), spec.st(dn)
        if sn == 1 and t.V > 1 and spec.aligned16 and (sm * ELT[spec.dt]) % 16 == 0 and not add \
                and all((s * ELT[spec.dt]) % 16 == 0 for s in spec.stride[:-1]):
            cnt = _pick_cnt(t.V, spec.dt)
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            for j in range(t.NCH):
                for q in range(t.V // cnt):
                    idx = f"{base} + (long)(row0 + r) * {sm}L + cb + {j * t.V * t.L + q * cnt}"
                    fn = "frnn_ldv" if load else "frnn_stv"
                    w(f"{fn}<{spec.dt},{cnt}>({ptr}, {idx}, &{arr}[r * {t.C} + {j * t.V + q * cnt}]);")
            w.close()
            return
        w("#pragma unroll")
        w.open(f"for (int r = 0; r < {t.R}; r++)")
        for j in range(t.NCH):
            for e in range(t.V):
                idx = f"{base} + (long)(row0 + r) * {sm}L + (long){t.col(j, e)} * {sn}L"
                el = f"{arr}[r * {t.C} + {j * t.V + e}]"
                if load:
                    w(f"{el} = frnn_io<{spec.dt}>::ld({ptr}, {idx});")
                elif add:
                    w(f"frnn_atomic_add_c((float*){ptr} + ({idx}), {el});")
                else:
                    w(f"frnn_io<{spec.dt}>::st({ptr}, {idx}, {el});")
        w.close()

    def emit_obuf_put(self, arr: str, obuf: str, row_expr: str, vidx: int, nvals: int):
        """Lane 0 of each row group parks R per-row values of one timestep in the
        shared output buffer (row ``row_expr``, value slot ``vidx``)."""
        w, t = self.w, self.t
        cnt = _pick_cnt(t.R, DT_F32, t.R)
        w.open("if (l == 0)")
        for q in range(t.R // cnt):
            w(f"frnn_stv<0,{cnt}>({obuf}, ({row_expr}) * {nvals * t.MB} + {vidx * t.MB} + rg * {t.R} + {q * cnt}, &{arr}[{q * cnt}]);")
        w.close()

    def emit_obuf_flush(self, obuf: str, nrows: str, vidx: int, nvals: int, dt: int, ptr: str, idx_of_row, stride_m: int,
                        aligned: bool, tidv: str = "tid", nthr: Optional[int] = None):
        """All threads: write ``nrows`` parked timesteps of value slot ``vidx`` to
        global memory with wide stores.  ``idx_of_row(s)`` gives the element
        offset of row m0 at parked row ``s``."""
        w, t = self.w, self.t
        vw = 8 if ELT[dt] == 2 else 4
        while t.MB % vw:
            vw //= 2
        fast = stride_m == 1 and aligned
        w.open(f"for (int it = {tidv}; it < ({nrows}) * {t.MB // vw}; it += {nthr or t.NT})")
        w(f"const int s = it / {t.MB // vw}, mm = (it % {t.MB // vw}) * {vw};")
        w(f"float v[{vw}];")
        cnt = min(4, vw)
        for q in range(vw // cnt):
            w(f"frnn_ldv<0,{cnt}>({obuf}, s * {nvals * t.MB} + {vidx * t.MB} + mm + {q * cnt}, &v[{q * cnt}]);")
        if fast:
            w(f"frnn_stv<{dt},{vw}>({ptr}, {idx_of_row('s')} + mm, v);")
        else:
            w("#pragma unroll")
            w(f"for (int q = 0; q < {vw}; q++) frnn_io<{dt}>::st({ptr}, {idx_of_row('s')} + (long)(mm + q) * {stride_m}L, v[q]);")
        w.close()

    def emit_row_vec_store(self, arr: str, dt: int, ptr: str, idx0: str, stride_m: int, aligned: bool,
                           atomic: bool = False):
        """Lane 0 of each row group stores R per-row values (rows row0..row0+R)."""
        w, t = self.w, self.t
        w.open("if (l == 0)")
        if atomic:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            w(f"frnn_atomic_add_c((float*){ptr} + ({idx0} + (long)(row0 + r) * {stride_m}L), {arr}[r]);")
            w.close()
        elif stride_m == 1 and aligned:
            cnt = _pick_cnt(t.R, dt, t.R)
            for q in range(t.R // cnt):
                w(f"frnn_stv<{dt},{cnt}>({ptr}, {idx0} + row0 + {q * cnt}, &{arr}[{q * cnt}]);")
        else:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            w(f"frnn_io<{dt}>::st({ptr}, {idx0} + (long)(row0 + r) * {stride_m}L, {arr}[r]);")
            w.close()
        w.close()


IN_DIMS = {"b": 0, "t": 1, "h": 2, "m": 3, "n": 4}


def _in_dims(cls: Shape) -> Dict[str, int]:
    d = dict(IN_DIMS)
    d["v"] = 4 if cls == N1 else 3
    return d


def _header(src_prelude: str) -> str:
    return src_prelude.replace("#pragma once", "")


def _stage_inputs(kb: KernelBuilder, p: Problem, used: Sequence[bool], allow_mn: bool) -> List[int]:
    """Register the time-varying inputs as staged items; return the indices of
    the time-invariant ones (loaded once into registers)."""
    const_inputs = []
    for i, spec in enumerate(p.inputs):
        if not used[i]:
            continue
        cls = p.in_cls(i)
        if cls == MN and spec.shape[1] != 1:
            raise LoweringError("an input that is a full matrix per head must not depend on time")
        if cls == MN and not allow_mn:
            raise LoweringError("matrix-per-head inputs are not supported by the backward kernel yet")
        if spec.shape[1] == 1:
            const_inputs.append(i)
            if cls == S11:
                kb.const_scalars[p.in_names[i]] = f"{vname(p.in_names[i])}[0]"
        else:
            kb.add_item(p.in_names[i], cls, spec, f"in{i}", _in_dims(cls))
    return const_inputs


# ---------------------------------------------------------------------------
# forward kernel
# ---------------------------------------------------------------------------

def emit_forward(p: Problem, g: StepGraph, aux_names: List[str], n_out: int, tile: Tile,
                 dstage: int, dck: int, use_tma: bool, min_blocks: int, prelude: str,
                 kname: str = "frnn_fw", final_ckpt: bool = False, step_unroll: int = 2, pack2: bool = False,
                 col_major: bool = False, max_acc: int = 2) -> KernelSource:
    """Forward scan.  ``g`` computes [*outputs, *new_states, *aux] from
    [*inputs, *states].  Kernel parameters, in order: used inputs, initial
    states, outputs, final states, checkpoints, aux, error word.  With
    ``final_ckpt`` one more fp32 checkpoint (the final state) is stored at
    index ceil(T/dck)."""
    kb = KernelBuilder(p, tile, dstage, use_tma)
    w, t = kb.w, tile
    ns = len(p.states)
    used = g.used_inputs()
    stcls = p.st_cls()

    ck_bytes = p.B * p.H * ((p.T + dck - 1) // dck + (1 if final_ckpt else 0)) * p.M * p.N * 4
    for i, spec in enumerate(p.inputs):
        if used[i]:
            kb.add_param(f"in{i}", "void", True, _spec_bytes(spec))
    for k in range(ns):
        kb.add_param(f"s0_{k}", "void", True, _spec_bytes(p.states[k]))
    for j in range(n_out):
        kb.add_param(f"out{j}", "void", False, p.B * p.T * p.H * p.M * ELT[p.out_dt[j]])
    for k in range(ns):
        kb.add_param(f"sT_{k}", "void", False, _spec_bytes(p.states[k]))
    for k in range(ns):
        kb.add_param(f"ck{k}", "float", False, ck_bytes)
    kb.add_param("aux", "float", False, len(aux_names) * p.B * p.H * p.T * p.M * 4)
    kb.add_param("err", "int", False, 4)

    const_inputs = _stage_inputs(kb, p, used, allow_mn=True)
    (g2,) = kb.plan([g])
    stage_bytes = kb.stage_bytes
    BAR_BYTES = 128
    off_wk = BAR_BYTES + stage_bytes      # one raw buffer: it is free again as soon as a chunk is converted
    n_ob = n_out + len(aux_names)         # per-row results parked in shared memory, written out once per chunk
    off_ob = off_wk + kb.wk_bytes
    ob_bytes = (dstage * n_ob * t.MB * 4 + 127) // 128 * 128
    smem_bytes = off_ob + ob_bytes
    nchunk = (p.T + dstage - 1) // dstage
    nck = (p.T + dck - 1) // dck
    nck_store = nck + (1 if final_ckpt else 0)

    w(_header(prelude))
    w(f"// forward scan: B={p.B} T={p.T} H={p.H} M={p.M} N={p.N}; tile R={t.R} C={t.C} L={t.L} MB={t.MB}; "
      f"stage {dstage} steps, checkpoint every {dck}")
    kb.emit_tma_issue("fw_issue")
    w(f'extern "C" __global__ void __launch_bounds__({t.NT}, {min_blocks})')
    w.open(f"{kname}({', '.join(kb.param_decl)})")
    w("FRNN_DYN_SMEM(smem);")
    kb.emit_thread_ids()
    kb.emit_bounds_prologue()
    w("u64* full = (u64*)smem;")
    w(f"unsigned char* stage = smem + {BAR_BYTES};")
    w(f"float* wk = (float*)(smem + {off_wk});")
    w(f"float* obuf = (float*)(smem + {off_ob});")
    has_tma = bool(kb.tma_items)
    if has_tma:
        w.open("if (tid == 0)")
        w("frnn_mbar_init(&full[0], 1); frnn_mbar_init(&full[1], 1); frnn_mbar_init_fence();")
        w.close()
        w("frnn_block_sync();")
    kb.emit_plain_decl()
    tma_call = (", " + kb.tma_issue_call) if has_tma else ""
    if kb.plain_items:
        kb.emit_plain_load("0", f"min({dstage}, {p.T})")
        kb.emit_plain_store("stage")
    if has_tma:
        w.open("if (warp == 0)")
        w(f"fw_issue(stage, &full[0], 0, min({dstage}, {p.T}), lane, b, h, m0{tma_call});")
        w.close()

    body = Body(w, t, g2.shape, pack2, col_major, max_acc)
    ckspec = TensorSpec((p.B, p.H, nck_store, p.M, p.N), _contig((p.B, p.H, nck_store, p.M, p.N)), DT_F32)
    for k in range(ns):
        body.declare(p.st_names[k], stcls)
        kb.emit_tile_global(vname(p.st_names[k]), p.states[k], f"s0_{k}",
                            _elem_off(p.states[k], [(0, "b"), (1, "h")]), 2, 3, load=True)
    for i in const_inputs:
        kb.emit_const_input(body, p.in_names[i], p.in_cls(i), p.inputs[i], f"in{i}", IN_DIMS)

    w("#pragma unroll 1")
    w.open(f"for (int c = 0; c < {nchunk}; c++)")
    w(f"const int t0 = c * {dstage}, nv = min({dstage}, {p.T} - t0);")
    w("unsigned char* sp = stage;")
    if kb.plain_items:
        w(f"if (c + 1 < {nchunk}) {{")
        w.ind += 1
        kb.emit_plain_load(f"(t0 + {dstage})", f"min({dstage}, {p.T} - t0 - {dstage})")
        w.ind -= 1
        w("}")
    if has_tma:
        w(f"if (!frnn_mbar_wait(&full[0], c & 1, err, {ERR_STAGE_TIMEOUT})) return;")
    w("frnn_block_sync();   // previous chunk's work buffer is no longer read; plain stores are visible")
    kb.emit_convert("sp", "wk", "nv")
    w("frnn_block_sync();   // work buffer complete; the raw buffer may be refilled")
    if has_tma:
        w.open(f"if (warp == 0 && c + 1 < {nchunk})")
        w(f"fw_issue(sp, &full[0], t0 + {dstage}, min({dstage}, {p.T} - t0 - {dstage}), lane, b, h, m0{tma_call});")
        w.close()
    sub_len = math.gcd(dstage, dck)
    w("#pragma unroll 1")
    w.open(f"for (int tl0 = 0; tl0 < nv; tl0 += {sub_len})")
    w.open(f"if ((t0 + tl0) % {dck} == 0)")
    for k in range(ns):
        base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, f"(t0 + tl0) / {dck}")])
        kb.emit_tile_global(vname(p.st_names[k]), ckspec, f"ck{k}", base, 3, 4, load=False)
    w.close()
    w(f"const int tl1 = min(tl0 + {sub_len}, nv);")
    w(f"#pragma unroll {step_unroll}")
    w.open("for (int tl = tl0; tl < tl1; tl++)")
    w("const int t = t0 + tl;")
    w(f"const float* wkt = wk + tl * {kb.wk_row}; (void)wkt;")
    sub = body.child()
    w.open("")
    for nm in g2.inputs:
        if nm in kb.wk and g2.used_inputs()[g2.inputs.index(nm)]:
            kb.emit_wk_read(sub, nm, "wkt")
    sub.graph(g2, allow_over_m=False)
    outs = g2.outputs
    yspec_shape = (p.B, p.T, p.H, p.M)
    for j in range(n_out):
        o = outs[j]
        ys = TensorSpec(yspec_shape, _contig(yspec_shape), p.out_dt[j])
        w(f"float yv{j}[{t.R}];")
        w("#pragma unroll")
        w(f"for (int r = 0; r < {t.R}; r++) yv{j}[r] = {sub.at(o, 'r', '0')};")
        kb.emit_obuf_put(f"yv{j}", "obuf", "tl", j, n_ob)
    ashape = (max(1, p.naux), p.B, p.H, p.T, p.M)
    aspec = TensorSpec(ashape, _contig(ashape), DT_F32)
    for a, an in enumerate(aux_names):
        w(f"float av{a}[{t.R}];")
        w("#pragma unroll")
        w(f"for (int r = 0; r < {t.R}; r++) av{a}[r] = {sub.at(an, 'r', '0')};")
        kb.emit_obuf_put(f"av{a}", "obuf", "tl", n_out + a, n_ob)
    for k in range(ns):
        o = outs[n_out + k]
        sub.loops(stcls, lambda r, c, k=k, o=o: f"{body.at(p.st_names[k], r, c)} = {sub.at(o, r, c)};")
    w.close()
    w.close()  # tl loop
    w.close()  # tl0 loop
    if n_ob:
        w("frnn_block_sync();   // the chunk's outputs and row sums are parked in shared memory")
        for j in range(n_out):
            ys = TensorSpec(yspec_shape, _contig(yspec_shape), p.out_dt[j])
            kb.emit_obuf_flush("obuf", "nv", j, n_ob, p.out_dt[j], f"out{j}",
                               lambda sx, ys=ys: _elem_off(ys, [(0, "b"), (1, f"t0 + {sx}"), (2, "h"), (3, "m0")]), 1,
                               (p.M * ELT[p.out_dt[j]]) % 16 == 0 and (t.MB * ELT[p.out_dt[j]]) % 16 == 0)
        for a, an in enumerate(aux_names):
            kb.emit_obuf_flush("obuf", "nv", n_out + a, n_ob, DT_F32, "aux",
                               lambda sx, a=a: _elem_off(aspec, [(0, str(a)), (1, "b"), (2, "h"), (3, f"t0 + {sx}"), (4, "m0")]), 1,
                               (p.M * 4) % 16 == 0 and (t.MB * 4) % 16 == 0)
    if kb.plain_items:
        w(f"if (c + 1 < {nchunk}) {{")
        w.ind += 1
        kb.emit_plain_store("stage")
        w.ind -= 1
        w("}")
    w.close()  # chunk loop
    for k in range(ns):
        kb.emit_tile_global(vname(p.st_names[k]), p.states[k], f"sT_{k}",
                            _elem_off(p.states[k], [(0, "b"), (1, "h")]), 2, 3, load=False)
        if final_ckpt:
            base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, str(nck))])
            kb.emit_tile_global(vname(p.st_names[k]), ckspec, f"ck{k}", base, 3, 4, load=False)
    w.close()
    return KernelSource(kname, w.text().replace("@SMEM_BYTES@", str(smem_bytes)), (p.M // t.MB, p.H, p.B), t.NT, smem_bytes,
                        kb.params, kb.param_decl,
                        {"stage_bytes": stage_bytes, "wk_bytes": kb.wk_bytes, "tma_items": len(kb.tma_items),
                         "plain_items": len(kb.plain_items), "nck": nck_store, "hoisted": [n.name for n in kb.hoisted],
                         "tile": [t.R, t.C, t.MB], "packed": bool(pack2)},
                        kb.tmaps)


# ---------------------------------------------------------------------------
# backward kernel
# ---------------------------------------------------------------------------

@dataclass
class GradOut:
    """How the gradient of one step input leaves the backward kernel."""
    index: int               # input index
    cls: Shape
    spec: TensorSpec         # spec of the tensor the kernel writes (fp32 if atomic)
    value: str               # graph value name
    over_t: bool             # input broadcast over T: accumulate over time in-kernel
    atomic: bool             # input broadcast over B, T or H: atomicAdd into fp32


@dataclass
class Reverse:
    """Exact-up-to-rounding inverse of an additive re-step: S_t = S_{t+1} -/+ X_t."""
    graph: StepGraph          # computes the increments [X_k] from inputs and aux
    sign: List[int]           # +1 if S' = S + X, -1 if S' = S - X
    resync: int               # chunks between reloads of an exact forward checkpoint


def can_split_post(g_re: StepGraph, g_bw: StepGraph, st_names: Sequence[str]) -> bool:
    """Whether the backward step can read the post-step state as an input instead of recomputing it: no node may
    need both a value derived from the post-step state and the pre-step state."""
    ns_names = list(g_re.outputs)
    if any(n in g_bw.inputs for n in ns_names):
        return False
    probe = g_bw.pruned(g_bw.outputs, g_bw.name, leaves=ns_names)
    if not all(n in probe.inputs for n in ns_names):
        return False                      # the backward does not use the post-step state at all
    dep_next = probe.depends_on(ns_names) - set(ns_names)
    dep_cur = probe.depends_on(st_names)
    return not (dep_next & dep_cur) and not (set(ns_names) & dep_cur)


def emit_backward(p: Problem, g_re: StepGraph, g_bw: StepGraph, aux_names: List[str], n_out: int,
                  grads: List[GradOut], dy_names: List[str], dnext_names: List[str], tile: Tile,
                  seg: int, nslots: int, use_tma: bool, prelude: str, kname: str = "frnn_bw",
                  kflush: int = 1, ring_bufs: int = 2, reverse: Optional[Reverse] = None,
                  step_unroll: int = 2, min_blocks: int = 1, pack2: bool = False,
                  col_major: bool = False, helper_warps: int = 0, max_acc: int = 1,
                  tmem_slots: int = 0, post_split: bool = False, unroll_segment: int = 0) -> KernelSource:
    """Reverse-time kernel.

    ``g_re`` computes the new states from [*inputs, *states, *aux];
    ``g_bw`` computes [*d_inputs, *d_states] from
    [*inputs, *states, *d_outputs, *d_new_states, *aux].

    Generic mode: a checkpoint chunk is D = seg * nslots steps; segment bases
    are rebuilt forward into shared-memory slots and the states inside a
    segment are recomputed from the base.  Reverse mode (additive re-steps
    only): the state is stepped *backwards* with the saved row sums, no slots;
    D = seg is the staging chunk and every ``reverse.resync`` chunks the state
    is reloaded from an exact forward checkpoint (checkpoint interval
    D * resync).

    Per-column and per-head gradient partials of ``kflush`` consecutive steps
    are collected in a shared ring and reduced over the row groups together.

    With ``helper_warps`` > 0 the CTA is warp-specialised: the tile's threads
    (the compute warps) only run the scan - work-buffer reads, arithmetic,
    shuffles, stores of partials - while the extra warps stage the inputs (TMA
    issue, conversion of each raw chunk into one of two fp32 work buffers,
    hoisted nodes) and reduce and store the gradient partials of one half of
    the ring while the compute warps fill the other.  The two sides meet only
    on mbarriers (work buffer full / empty, ring half full / empty), every wait
    time-bounded; the compute warps never wait for a block-wide barrier.

    With ``post_split`` (generic mode, when ``can_split_post`` holds) the step
    is evaluated in two parts, as in the reverse mode: the part that needs only
    the post-step state S_{t+1} runs while the state registers still hold it -
    they do, from the step handled just before - and the part that needs the
    pre-step state S_t after S_t has been fetched; the post-step state is then
    never recomputed inside the backward step.  The first part of step t-1 is
    issued right after the second part of step t (for the last step of a chunk:
    at the start of the chunk, before its segment bases are rebuilt), and the
    forward stores one more fp32 checkpoint, the final state.

    With ``tmem_slots`` = nslots > 0 (generic mode, helper warps on) the segment
    bases live in Tensor Memory instead of shared memory: each thread parks its
    register tile in its own lane (tcgen05.st) and fetches it back (tcgen05.ld),
    so four bases of a 128x128 state fit on the SM beside one shared-memory
    landing slot for the checkpoint copy, and a chunk of 8 steps costs 10
    re-steps instead of 16.  The CTA allocates the columns at start and frees
    them on every path out (the scan runs inside a function object; after it
    returns, normally or on a timed-out wait, each warp checks in and the
    allocating warp frees the columns).

    Parameters, in order: used inputs, d_outputs, d_final_states,
    checkpoints, aux, d_initial_states, input gradients, error word.
    """
    rev = reverse is not None
    D = seg if rev else seg * nslots
    kb = KernelBuilder(p, tile, D, use_tma)
    w, t = kb.w, tile
    if t.MB != p.M:
        # Rows split over several CTAs (a state too large for the registers of one SM): rows are independent
        # recurrences, only the gradients summed over rows couple them, and those must then be accumulated
        # across CTAs with atomic adds into fp32 (the planner marks them ``atomic``).
        for go in grads:
            if go.cls in (N1, S11) and not go.atomic:
                raise LoweringError("rows split over CTAs need atomically accumulated column gradients")
    ws = helper_warps > 0
    NCT = t.NT
    # Register file: the hardware allots registers to a CTA as if its thread count were rounded up to whole
    # warpgroups (128 threads).  When the compute warps fill whole warpgroups, the helpers are one more warpgroup,
    # and the two sides rebalance their registers at kernel start (the helpers need few, the scan needs many).
    regs_launch = regs_compute = regs_helper = 0
    if ws and NCT % 128 == 0:
        helper_warps = 4
        regs_launch = min(248, 65536 // (max(1, min_blocks) * (NCT + 128)) // 8 * 8)
        regs_helper = min(regs_launch, 56)
        regs_compute = min(248, (regs_launch + (regs_launch - regs_helper) * 128 // NCT) // 8 * 8)
    elif ws:
        helper_warps = 1
    HT = 32 * helper_warps
    ring_bufs = max(1, min(2, ring_bufs))
    if NCT + HT > 1024:
        raise LoweringError("too many threads for one CTA")
    ns = len(p.states)
    stcls = p.st_cls()
    nin = len(p.inputs)
    alias_next: List[str] = []
    if rev:
        # the post-step state is in registers before the reverse step: let the backward graph read it
        # instead of recomputing it, provided no node needs both the post-step and the pre-step state
        ns_names = list(g_re.outputs)
        probe = g_bw.pruned(g_bw.outputs, g_bw.name, leaves=[n for n in ns_names if n not in g_bw.inputs])
        dep_next = probe.depends_on(ns_names) - set(ns_names)
        dep_cur = probe.depends_on(p.st_names)
        if not (dep_next & dep_cur) and not (set(ns_names) & dep_cur) and all(n in probe.inputs for n in ns_names):
            g_bw = probe
            alias_next = ns_names
    split = False
    if (not rev) and post_split:
        if not can_split_post(g_re, g_bw, p.st_names):
            raise LoweringError("this step's backward cannot be split at the post-step state")
        ns_names = list(g_re.outputs)
        g_bw = g_bw.pruned(g_bw.outputs, g_bw.name, leaves=[n for n in ns_names if n not in g_bw.inputs])
        alias_next = ns_names
        split = True
    g_bw = g_bw.simplified_products()
    graphs = [g_bw] + ([reverse.graph] if rev else [g_re])
    used_lists = [g.used_inputs() for g in graphs]
    used = [any(u[i] for u in used_lists) for i in range(nin)]
    used_bw0 = g_bw.used_inputs()
    dy_used = [used_bw0[nin + ns + j] for j in range(n_out)]
    nchunk = (p.T + D - 1) // D
    dck = D * (reverse.resync if rev else 1)
    nck = (p.T + dck - 1) // dck
    nck_store = nck + (1 if (rev or split) else 0)

    for i in range(nin):
        if used[i]:
            kb.add_param(f"in{i}", "void", True, _spec_bytes(p.inputs[i]))
    for j in range(n_out):
        kb.add_param(f"dy{j}", "void", True, p.B * p.T * p.H * p.M * ELT[p.out_dt[j]])
    for k in range(ns):
        kb.add_param(f"dsT_{k}", "void", True, p.B * p.H * p.M * p.N * ELT[p.states[k].dt])
    for k in range(ns):
        kb.add_param(f"ck{k}", "float", True, p.B * p.H * nck_store * p.M * p.N * 4)
    kb.add_param("aux", "float", True, p.naux * p.B * p.H * p.T * p.M * 4)
    for k in range(ns):
        kb.add_param(f"ds0_{k}", "void", False, _spec_bytes(p.states[k]))
    for go in grads:
        kb.add_param(f"dx{go.index}", "void", False, _spec_bytes(go.spec))
    kb.add_param("err", "int", False, 4)

    const_inputs = _stage_inputs(kb, p, used, allow_mn=True)
    ashape = (max(1, p.naux), p.B, p.H, p.T, p.M)
    for a, an in enumerate(aux_names):
        sp_a = TensorSpec(ashape[1:], _contig(ashape)[1:], DT_F32)
        kb.add_item(an, M1, sp_a, "aux", {"b": 0, "h": 1, "t": 2, "v": 3}, const_off=a * p.B * p.H * p.T * p.M)
    yshape = (p.B, p.T, p.H, p.M)
    for j in range(n_out):
        if dy_used[j]:
            ys = TensorSpec(yshape, _contig(yshape), p.out_dt[j])
            kb.add_item(dy_names[j], M1, ys, f"dy{j}", {"b": 0, "t": 1, "h": 2, "v": 3})
    planned = kb.plan(graphs)
    g_bw2, g_aux2 = planned[0], planned[1]
    stage_bytes = kb.stage_bytes

    # gradient-partial ring: per step and row group all 1N gradients, then all 11 gradients
    pm_vec = [go for go in grads if go.cls == N1]
    pm_sc = [go for go in grads if go.cls == S11]
    vw = 4 if p.N % 4 == 0 else (2 if p.N % 2 == 0 else 1)
    redw = len(pm_vec) * p.N + len(pm_sc)
    redw_pad = (redw + 3) // 4 * 4
    step_floats = t.RG * redw_pad
    ring_bytes = ring_bufs * kflush * step_floats * 4 if redw else 0
    tm = (not rev) and ws and tmem_slots > 0
    if tm and tmem_slots != nslots:
        raise LoweringError("the Tensor Memory slots must be the segment slots")
    nphys = 0 if rev else (1 if tm else max(nslots, 2))
    tile_regs = t.R * t.C
    tm_slot_cols = ((NCT + 127) // 128) * ns * tile_regs          # columns of one slot: a tile per state and warpgroup
    tm_cols = 32
    while tm and tm_cols < nslots * tm_slot_cols:
        tm_cols *= 2
    if tm and tm_cols > 512 // max(1, min_blocks):
        raise LoweringError("the segment bases do not fit the Tensor Memory of one SM")
    slot_elems = t.MB * p.N           # rows of this CTA
    slot_bytes = slot_elems * 4
    ck_tma = (not rev) and use_tma and slot_bytes % 16 == 0
    BAR_BYTES = 128
    wk_bufs = 2 if ws else 1
    wk_floats = kb.wk_bytes // 4
    off_stage = BAR_BYTES
    off_wk = off_stage + stage_bytes       # one raw buffer (free again once a chunk is converted)
    off_slots = off_wk + wk_bufs * kb.wk_bytes
    off_ring = off_slots + nphys * ns * slot_bytes
    # per-row gradients written every step (dv ...) are parked next to the ring and stored at flush time
    row_st = [go for go in grads if go.cls == M1 and not go.over_t and not go.atomic] if redw else []
    off_ob = off_ring + ring_bytes
    ob_bytes = ring_bufs * kflush * len(row_st) * t.MB * 4
    smem_bytes = off_ob + ob_bytes
    # mbarriers: 0 staged inputs, 2 checkpoint copy; with helper warps 3,4 work buffer full, 5,6 work buffer empty,
    # 7,8 ring half full, 9,10 ring half empty
    B_RAW, B_CK, B_WKF, B_WKE, B_RGF, B_RGE = 0, 2, 3, 5, 7, 9

    w(_header(prelude))
    mode = f"reverse re-step, resync every {dck} steps" if rev else f"chunk {D} = {nslots} segments x {seg} steps"
    w(f"// backward scan: B={p.B} T={p.T} H={p.H} M={p.M} N={p.N}; tile R={t.R} C={t.C} L={t.L}; {mode}; "
      f"gradient partials flushed every {kflush} steps"
      + (f"; {helper_warps} helper warp(s) stage the inputs and flush the partials" if ws else ""))
    kb.emit_tma_issue("bw_issue")

    w(f'extern "C" __global__ void __launch_bounds__({NCT + HT}, {min_blocks})')
    w.open(f"{kname}({', '.join(kb.param_decl)})")
    w("FRNN_DYN_SMEM(smem);")
    kb.emit_thread_ids()
    kb.emit_bounds_prologue()
    w("u64* full = (u64*)smem;        // mbarriers")
    w(f"unsigned char* stage = smem + {off_stage};")
    w(f"float* wk = (float*)(smem + {off_wk});")
    if nphys:
        w(f"float* slots = (float*)(smem + {off_slots});")
    if redw:
        w(f"float* ring = (float*)(smem + {off_ring});")
        w(f"float* obuf = (float*)(smem + {off_ob}); (void)obuf;")
    has_tma = bool(kb.tma_items)
    w.open("if (tid == 0)")
    w(f"frnn_mbar_init(&full[{B_RAW}], 1); frnn_mbar_init(&full[1], 1); frnn_mbar_init(&full[{B_CK}], 1);")
    if ws:
        w(f"frnn_mbar_init(&full[{B_WKF}], {HT}); frnn_mbar_init(&full[{B_WKF + 1}], {HT});")
        w(f"frnn_mbar_init(&full[{B_WKE}], {NCT}); frnn_mbar_init(&full[{B_WKE + 1}], {NCT});")
        w(f"frnn_mbar_init(&full[{B_RGF}], {NCT}); frnn_mbar_init(&full[{B_RGF + 1}], {NCT});")
        w(f"frnn_mbar_init(&full[{B_RGE}], {HT}); frnn_mbar_init(&full[{B_RGE + 1}], {HT});")
        w(f"frnn_mbar_init(&full[11], {NCT}); frnn_mbar_init(&full[14], {HT});   // rendezvous of the compute / helper threads")
    if tm:
        w("((int*)&full[13])[0] = 0;      // warps that are done with Tensor Memory")
    w("frnn_mbar_init_fence();")
    w.close()
    if tm:
        w.open("if (warp == 0)")
        w(f"frnn_tmem_alloc((u32*)&full[12], {tm_cols}u);")
        w("frnn_tmem_fence_before_sync();")
        w.close()
    w("frnn_block_sync();")
    if tm:
        w("frnn_tmem_fence_after_sync();")
        w("const u32 tm_base = *(volatile u32*)&full[12];")
        w(f"const u32 tm_mine = tm_base + frnn_tmem_lane_base(warp) + (u32)(warp >> 2) * {ns * tile_regs}u;   // this thread's lane, this warpgroup's columns")
    tma_call = (", " + kb.tma_issue_call) if has_tma else ""
    ckspec = TensorSpec((p.B, p.H, nck_store, p.M, p.N), _contig((p.B, p.H, nck_store, p.M, p.N)), DT_F32)
    first_c = nchunk - 1
    nv_first = p.T - first_c * D

    def csync(why: str = ""):
        """Barrier over the compute warps.  With helper warps it is an mbarrier rendezvous with a bounded wait,
        not a hardware barrier: should one warp leave on a timed-out wait, the others must not wait for it for ever."""
        if not ws:
            w("frnn_block_sync();" + (f"   // {why}" if why else ""))
            return
        w(f"frnn_mbar_arrive(&full[11]);" + (f"   // {why}" if why else ""))
        w(f"if (!frnn_mbar_wait(&full[11], cs_par, err, {ERR_STAGE_TIMEOUT})) return;")
        w("cs_par ^= 1;")

    # element offsets inside one ring row
    ring_off: Dict[int, int] = {}
    pos = 0
    for go in pm_vec:
        ring_off[go.index] = pos
        pos += p.N
    for go in pm_sc:
        ring_off[go.index] = pos
        pos += 1

    # time-invariant per-column / per-head gradients: work item (ring row s, element j) always falls to the
    # same thread and accumulator, which sums it over the row groups and over time; atomics combine at the end
    tinv = [go for go in pm_vec + pm_sc if go.over_t]
    ntel = sum(p.N if go.cls == N1 else 1 for go in tinv)
    FT = HT if ws else NCT                      # threads that run the flush
    ftid = "hl" if ws else "tid"
    nred_per_thread = (kflush * ntel + FT - 1) // FT if tinv else 0

    def tinv_locate(jexpr: str):
        """Emit `ro` (offset in a ring row) for compact element index jexpr."""
        w("int ro = 0;")
        cum = 0
        for go in tinv:
            n_el = p.N if go.cls == N1 else 1
            w(f"if ({jexpr} >= {cum} && {jexpr} < {cum + n_el}) ro = {ring_off[go.index]} + ({jexpr} - {cum});")
            cum += n_el

    def emit_racc_decl():
        if tinv:
            w(f"float racc[{max(1, nred_per_thread)}];")
            w("#pragma unroll")
            w(f"for (int q = 0; q < {max(1, nred_per_thread)}; q++) racc[q] = 0.0f;")

    def emit_racc_final():
        if not tinv:
            return
        w("#pragma unroll")
        w.open(f"for (int q = 0; q < {nred_per_thread}; q++)")
        w(f"const int it = {ftid} + q * {FT}, j = it % {ntel};")
        w.open(f"if (it < {kflush * ntel})")
        cum = 0
        for go in tinv:
            n_el = p.N if go.cls == N1 else 1
            w.open(f"if (j >= {cum} && j < {cum + n_el})")
            dims = [(0, "b"), (2, "h")] + ([(4, f"(j - {cum})")] if go.cls == N1 else [])
            w(f"frnn_atomic_add_c((float*)dx{go.index} + ({_elem_off(go.spec, dims)}), racc[q]);")
            w.close()
            cum += n_el
        w.close()
        w.close()

    def flush_body(half: str, rcnt: str, rt_first: str):
        """Reduce the ``rcnt`` collected steps of ring half ``half`` over the row groups and write the
        gradients; run by the threads ``ftid`` in [0, FT)."""
        w(f"const float* rr = ring + ({half}) * {kflush * step_floats};")
        for vi, go in enumerate(row_st):
            kb.emit_obuf_flush(f"(obuf + ({half}) * {kflush * len(row_st) * t.MB})", rcnt, vi, len(row_st), go.spec.dt,
                               f"dx{go.index}",
                               lambda sx, go=go: _elem_off(go.spec, [(0, "b"), (1, f"({rt_first}) - {sx}"), (2, "h"), (3, "m0")]),
                               go.spec.st(3),
                               go.spec.aligned16 and all((go.spec.st(d) * ELT[go.spec.dt]) % 16 == 0 for d in (0, 1, 2)),
                               tidv=ftid, nthr=FT)
        nq = p.N // vw
        stream_vec = [go for go in pm_vec if not go.over_t]
        if stream_vec:
            w(f"for (int it = {ftid}; it < ({rcnt}) * {len(stream_vec) * nq}; it += {FT}) {{")
            w.ind += 1
            w(f"const int s = it / {len(stream_vec) * nq}, rem = it % {len(stream_vec) * nq}, vi = rem / {nq}, c0 = (rem % {nq}) * {vw};")
            w(f"const int tt = ({rt_first}) - s; (void)tt;")
            w(f"float a[{vw}];")
            w("#pragma unroll")
            w(f"for (int q = 0; q < {vw}; q++) a[q] = 0.0f;")
            w("int ro = 0;")
            for k, go in enumerate(stream_vec):
                w(f"if (vi == {k}) ro = {ring_off[go.index]};")
            w(f"const float* src = rr + s * {step_floats} + ro + c0;")
            w("#pragma unroll 4")
            w.open(f"for (int gi = 0; gi < {t.RG}; gi++)")
            w(f"float v[{vw}];")
            w(f"frnn_ldv<0,{vw}>(src, gi * {redw_pad}, v);")
            w("#pragma unroll")
            w(f"for (int q = 0; q < {vw}; q++) a[q] += v[q];")
            w.close()
            for k, go in enumerate(stream_vec):
                w.open(f"if (vi == {k})")
                idx = _elem_off(go.spec, [(0, "b"), (1, "tt"), (2, "h")])
                sn = go.spec.st(4)
                if go.atomic:
                    w("#pragma unroll")
                    w(f"for (int q = 0; q < {vw}; q++) frnn_atomic_add_c((float*)dx{go.index} + ({idx} + (long)(c0 + q) * {sn}L), a[q]);")
                elif sn == 1 and go.spec.aligned16 and all((go.spec.st(d) * ELT[go.spec.dt]) % (vw * ELT[go.spec.dt]) == 0 for d in (0, 1, 2)):
                    w(f"frnn_stv<{go.spec.dt},{vw}>(dx{go.index}, {idx} + c0, a);")
                else:
                    w("#pragma unroll")
                    w(f"for (int q = 0; q < {vw}; q++) frnn_io<{go.spec.dt}>::st(dx{go.index}, {idx} + (long)(c0 + q) * {sn}L, a[q]);")
                w.close()
            w.ind -= 1
            w("}")
        stream_sc = [go for go in pm_sc if not go.over_t]
        if stream_sc:
            w(f"for (int it = {ftid}; it < ({rcnt}) * {len(stream_sc)}; it += {FT}) {{")
            w.ind += 1
            w(f"const int s = it / {len(stream_sc)}, si = it % {len(stream_sc)}, tt = ({rt_first}) - s; (void)tt;")
            w("int ro = 0;")
            for k, go in enumerate(stream_sc):
                w(f"if (si == {k}) ro = {ring_off[go.index]};")
            w("float a = 0.0f;")
            w(f"for (int gi = 0; gi < {t.RG}; gi++) a += rr[s * {step_floats} + gi * {redw_pad} + ro];")
            for k, go in enumerate(stream_sc):
                w.open(f"if (si == {k})")
                idx = _elem_off(go.spec, [(0, "b"), (1, "tt"), (2, "h")])
                if go.atomic:
                    w(f"frnn_atomic_add_c((float*)dx{go.index} + ({idx}), a);")
                else:
                    w(f"frnn_io<{go.spec.dt}>::st(dx{go.index}, {idx}, a);")
                w.close()
            w.ind -= 1
            w("}")
        if tinv:
            w("#pragma unroll")
            w.open(f"for (int q = 0; q < {nred_per_thread}; q++)")
            w(f"const int it = {ftid} + q * {FT}, s = it / {ntel}, j = it % {ntel};")
            w.open(f"if (s < ({rcnt}))")
            tinv_locate("j")
            w("float a = 0.0f;")
            w(f"for (int gi = 0; gi < {t.RG}; gi++) a += rr[s * {step_floats} + gi * {redw_pad} + ro];")
            w("racc[q] += a;")
            w.close()
            w.close()

    # ================================================================== helper warps
    if ws:
        w.open(f"if (tid >= {NCT})")
        if regs_launch and regs_helper < regs_launch:
            w(f"frnn_regs_release<{regs_helper}>();")
        w(f"const int hl = tid - {NCT}, hlane = hl & 31; (void)hlane;")
        hbody = Body(w, t, {}, False, False)
        for i in const_inputs:
            if p.in_cls(i) == S11:      # time-invariant scalars feed hoisted nodes: the helpers evaluate those
                kb.emit_const_input(hbody, p.in_names[i], S11, p.inputs[i], f"in{i}", IN_DIMS)
        # rendezvous of the helper threads (bounded, like the compute warps')
        hsync = "frnn_warp_sync();" if helper_warps == 1 else (
            f"frnn_mbar_arrive(&full[14]); if (!frnn_mbar_wait(&full[14], hs_par, err, {ERR_STAGE_TIMEOUT})) return; hs_par ^= 1;")
        w("u32 hs_par = 0; (void)hs_par;")
        emit_racc_decl()
        w("int hg = 0; (void)hg;   // flush groups served so far")

        def h_issue(t0e: str, nve: str):
            """Helper: start the copies of one chunk into the raw buffer (it must be free)."""
            if kb.plain_items:
                kb.emit_plain_direct("stage", t0e, nve, "hl", HT)
            if has_tma:
                w.open("if (hl < 32)")
                w(f"bw_issue(stage, &full[{B_RAW}], {t0e}, {nve}, hlane, b, h, m0{tma_call});")
                w.close()

        def h_convert(ce: str, nve: str):
            """Helper: raw chunk number ``ce`` (in processing order) -> work buffer ce & 1."""
            if has_tma:
                w(f"if (!frnn_mbar_wait(&full[{B_RAW}], ({ce}) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
            if kb.plain_items:
                w(hsync + "   // plain copies of the chunk are visible")
            w(f"if (({ce}) >= 2 && !frnn_mbar_wait(&full[{B_WKE} + (({ce}) & 1)], ((({ce}) >> 1) - 1) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
            w(f"float* wkh = wk + (({ce}) & 1) * {wk_floats}; (void)wkh;")
            kb.emit_convert("stage", "wkh", nve, tidv="hl", nthr=HT)
            w(f"frnn_mbar_arrive(&full[{B_WKF} + (({ce}) & 1)]);")
            w(hsync + "   // every helper thread is done reading the raw buffer")

        h_issue(str(first_c * D), str(nv_first))
        w.open("")
        h_convert("0", str(nv_first))
        w.close()
        if nchunk > 1:
            h_issue(str((first_c - 1) * D), str(D))
        w("#pragma unroll 1")
        w.open(f"for (int c = 0; c < {nchunk}; c++)")
        w(f"const int kc = {nchunk - 1} - c, t0 = kc * {D}, nv = min({D}, {p.T} - t0);")
        w.open(f"if (c + 1 < {nchunk})")
        h_convert("c + 1", str(D))
        w.open(f"if (c + 2 < {nchunk})")
        h_issue(f"(kc - 2) * {D}", str(D))
        w.close()
        w.close()
        if redw:
            w("#pragma unroll 1")
            w.open(f"for (int g1 = nv; g1 > 0; g1 -= {kflush})")
            w(f"const int hh = hg % {ring_bufs}, hcnt = min({kflush}, g1), ht = t0 + g1 - 1;")
            w(f"if (!frnn_mbar_wait(&full[{B_RGF} + hh], (hg / {ring_bufs}) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
            flush_body("hh", "hcnt", "ht")
            w(f"frnn_mbar_arrive(&full[{B_RGE} + hh]);")
            w("hg++;")
            w.close()
        w.close()   # chunk loop
        emit_racc_final()
        w("return;")
        w.close()   # helper role

    # ================================================================== compute warps
    if regs_launch and regs_compute > regs_launch:
        w(f"frnn_regs_acquire<{regs_compute}>();")
    if tm:
        w("auto scan = [&]() -> void {")
        w.ind += 1
    if not ws:
        kb.emit_plain_decl()

    def ck_fetch(kexpr: str, physexpr: str):
        """Start the copy of checkpoint ``kexpr`` into physical slot ``physexpr``."""
        if ck_tma:
            w.open("if (tid == 0)")
            w("frnn_async_proxy_fence();")
            w(f"frnn_mbar_expect_tx(&full[{B_CK}], {ns * slot_bytes}u);")
            for k in range(ns):
                base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, kexpr), (3, "m0")])
                w(f"frnn_bulk_g2s_c(slots + ((long)({physexpr}) * {ns} + {k}) * {slot_elems}, ck{k} + {base}, {slot_bytes}u, &full[{B_CK}]);")
            w.close()
        else:
            for k in range(ns):
                base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, kexpr), (3, "m0")])
                w(f"for (int e = tid; e < {slot_elems}; e += {NCT}) "
                  f"slots[((long)({physexpr}) * {ns} + {k}) * {slot_elems} + e] = ck{k}[{base} + e];")

    if not ws:
        if kb.plain_items:
            kb.emit_plain_load(str(first_c * D), str(nv_first))
            kb.emit_plain_store("stage")
        if has_tma:
            w.open("if (warp == 0)")
            w(f"bw_issue(stage, &full[{B_RAW}], {first_c * D}, {nv_first}, lane, b, h, m0{tma_call});")
            w.close()
    if not rev:
        ck_fetch(str(first_c), "0")

    body = Body(w, t, g_bw2.shape, pack2, col_major, max_acc)
    body.shape.update(g_aux2.shape)
    dshape = (p.B, p.H, p.M, p.N)
    for k in range(ns):
        body.declare(dnext_names[k], stcls)
        dspec = TensorSpec(dshape, _contig(dshape), p.states[k].dt)
        kb.emit_tile_global(vname(dnext_names[k]), dspec, f"dsT_{k}",
                            _elem_off(dspec, [(0, "b"), (1, "h")]), 2, 3, load=True)
        body.declare(p.st_names[k], stcls)
    for i in const_inputs:
        kb.emit_const_input(body, p.in_names[i], p.in_cls(i), p.inputs[i], f"in{i}", IN_DIMS)
    for go in grads:
        if go.over_t and go.cls == M1:
            w(f"float gacc{go.index}[{t.R}];")
            w("#pragma unroll")
            w(f"for (int r = 0; r < {t.R}; r++) gacc{go.index}[r] = 0.0f;")
        if go.cls == MN:
            # matrix-per-head inputs are time-invariant: their gradient tile accumulates in registers
            w(f"float gmat{go.index}[{t.R * t.C}];")
            w("#pragma unroll")
            w(f"for (int i = 0; i < {t.R * t.C}; i++) gmat{go.index}[i] = 0.0f;")
    if not ws:
        emit_racc_decl()
    w("int rcnt = 0, rhalf = 0, rt_first = 0, gidx = 0; (void)rcnt; (void)rhalf; (void)rt_first; (void)gidx;")
    w("u32 cs_par = 0; (void)cs_par;")

    def emit_flush():
        """The collected steps are complete: reduce them over the row groups and write the gradients
        (or, with helper warps, hand the ring half over to them)."""
        if not redw:
            return
        w.open("if (rcnt > 0)")
        if ws:
            w(f"frnn_mbar_arrive(&full[{B_RGF} + rhalf]);   // this thread's partials of the group are in the ring")
            w(f"gidx++; rhalf = gidx % {ring_bufs};")
        else:
            w("frnn_block_sync();   // all partials of this group are in the ring")
            flush_body("rhalf", "rcnt", "rt_first")
            if ring_bufs == 1:
                w("frnn_block_sync();   // single ring: readers done before the next group is written")
            else:
                w("rhalf ^= 1;")
        w("rcnt = 0;")
        w.close()

    def tmem_rw(jexpr: str, store: bool):
        """Register tiles of all states <-> Tensor Memory slot ``jexpr``."""
        for k in range(ns):
            fn = "frnn_tmem_st" if store else "frnn_tmem_ld"
            w(f"{fn}<{tile_regs}>(tm_mine + (u32)({jexpr}) * {tm_slot_cols}u + {k * tile_regs}u, {vname(p.st_names[k])});")
        if not store:
            w("frnn_tmem_wait_ld();")

    def slot_rw(physexpr: str, store: bool):
        for k in range(ns):
            arr = vname(p.st_names[k])
            basee = f"((long)({physexpr}) * {ns} + {k}) * {slot_elems}"
            cnt = _pick_cnt(t.V, DT_F32)
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            for j in range(t.NCH):
                for q in range(t.V // cnt):
                    idx = f"{basee} + (rg * {t.R} + r) * {p.N} + cb + {j * t.V * t.L + q * cnt}"
                    fn = "frnn_stv" if store else "frnn_ldv"
                    w(f"{fn}<0,{cnt}>(slots, {idx}, &{arr}[r * {t.C} + {j * t.V + q * cnt}]);")
            w.close()

    def read_wk_inputs(sub: Body, g: StepGraph):
        used_g = dict(zip(g.inputs, g.used_inputs()))
        for nm in g.inputs:
            if nm in kb.wk and used_g.get(nm, False):
                kb.emit_wk_read(sub, nm, "wkt")

    def emit_restep(tlexpr: str):
        w.open("")
        w(f"const int tl = {tlexpr};")
        w(f"const float* wkt = wkc + tl * {kb.wk_row}; (void)wkt;")
        sub = body.child()
        read_wk_inputs(sub, g_aux2)
        sub.graph(g_aux2)
        for k in range(ns):
            o = g_aux2.outputs[k]
            sub.loops(stcls, lambda r, c, k=k, o=o: f"{body.at(p.st_names[k], r, c)} = {sub.at(o, r, c)};")
        w.close()

    def emit_unstep():
        """S_t = S_{t+1} -/+ X_t (reverse mode); expects tl, wkt in scope."""
        w.open("")
        sub = body.child()
        read_wk_inputs(sub, g_aux2)
        # the update of the state registers is written as one more node, so that the product
        # that forms the increment folds into a packed multiply-add
        upd = [Node(f"unstep{k}", "sub" if reverse.sign[k] > 0 else "add", [p.st_names[k], g_aux2.outputs[k]], stcls)
               for k in range(ns)]
        nodes = list(g_aux2.nodes) + upd
        sub.fuse_group(nodes, nodes, ())
        for n in g_aux2.nodes:
            sub.node(n, False)
        for k, u in enumerate(upd):
            st = p.st_names[k]
            if sub.can_pack() and sub.pair_expr(u, "r", "c") is not None:
                sub.pair_loops(stcls, lambda r, c, u=u, st=st: (
                    f"{{ const frnn_pk v2 = {sub.pair_expr(u, r, c)}; "
                    f"{body.at(st, r, c)} = v2.x; {body.at(st, r, c + ' + 1')} = v2.y; }}"))
            else:
                sgn = "-" if u.op == "sub" else "+"
                sub.loops(stcls, lambda r, c, st=st, u=u, sgn=sgn:
                          f"{body.at(st, r, c)} = {body.at(st, r, c)} {sgn} {sub.at(u.args[1], r, c)};")
        w.close()

    step_parts: Dict[str, object] = {}

    def step_body() -> Body:
        """The Body both parts of the backward step are emitted with (made once: which products are folded
        into which consumer must not change between two emissions of a part)."""
        if "sub" not in step_parts:
            sub = body.child()
            phase1: List[Node] = []
            phase2: List[Node] = list(g_bw2.nodes)
            if alias_next:
                # part 1 (state registers hold S_{t+1}): every node that does not need S_t
                for k, nm in enumerate(alias_next):
                    sub.alias[nm] = p.st_names[k]
                    sub.shape[nm] = stcls
                dep_cur = g_bw2.depends_on(p.st_names)
                if split:
                    # only what reads the post-step state (and what that needs) has to run before S_t is fetched;
                    # everything else waits, so that little more than a few vectors lives across the fetch
                    early = set(g_bw2.depends_on(alias_next)) - set(alias_next)
                    names = {n.name for n in g_bw2.nodes}
                    for n in reversed(g_bw2.nodes):
                        if n.name in early:
                            early.update(a for a in n.value_args() if a in names)
                    phase1 = [n for n in g_bw2.nodes if n.name in early]
                    phase2 = [n for n in g_bw2.nodes if n.name not in early]
                else:
                    phase1 = [n for n in g_bw2.nodes if n.name not in dep_cur]
                    phase2 = [n for n in g_bw2.nodes if n.name in dep_cur]
                # a product is only folded into a consumer of its own part: between the parts the state
                # registers change from S_{t+1} to S_t
                sub.fuse_group(phase1, g_bw2.nodes, g_bw2.outputs)
                sub.fuse_group(phase2, g_bw2.nodes, g_bw2.outputs)
            else:
                sub.fuse_group(g_bw2.nodes, g_bw2.nodes, set(g_bw2.outputs))
            step_parts.update(sub=sub, phase1=phase1, phase2=phase2)
        return step_parts["sub"]

    def part_inputs(nodes: Sequence[Node], extra: Iterable[str] = ()) -> set:
        names = set(extra)
        for n in nodes:
            names.update(n.value_args())
        return names

    def read_wk_named(sub: Body, names: set):
        used_g = dict(zip(g_bw2.inputs, g_bw2.used_inputs()))
        for nm in g_bw2.inputs:
            if nm in kb.wk and used_g.get(nm, False) and nm in names:
                kb.emit_wk_read(sub, nm, "wkt")

    def crossing_values() -> List[Node]:
        """Values of part 1 that part 2 or the outputs read: they live across the fetch of S_t."""
        step_body()
        later = part_inputs(step_parts["phase2"], g_bw2.outputs)
        return [n for n in step_parts["phase1"] if n.name in later and n.name not in step_parts["sub"].fused]

    def emit_part1(tlexpr: str):
        """Split mode: part 1 of the step at chunk position ``tlexpr``; the state registers hold S_{t+1}."""
        sub = step_body()
        w.open("")
        w(f"const int tl = {tlexpr}, t = t0 + tl; (void)t;")
        w(f"const float* wkt = wkc + tl * {kb.wk_row}; (void)wkt;")
        read_wk_named(sub, part_inputs(step_parts["phase1"]))
        for n in step_parts["phase1"]:
            sub.node(n, True)
        w.close()

    def emit_bw_step():
        """The backward step proper; expects tl, t, wkt in scope (split mode: its second part and the outputs)."""
        sub = step_body()
        if split:
            read_wk_named(sub, part_inputs(step_parts["phase2"], g_bw2.outputs))
            for n in step_parts["phase2"]:
                sub.node(n, True)
        elif alias_next:
            read_wk_inputs(sub, g_bw2)
            for n in step_parts["phase1"]:
                sub.node(n, True)
            emit_unstep()
            for n in step_parts["phase2"]:
                sub.node(n, True)
        else:
            read_wk_inputs(sub, g_bw2)
            if rev:
                emit_unstep()
            for n in g_bw2.nodes:
                sub.node(n, True)
        outs = g_bw2.outputs
        if redw:
            w.open("if (rcnt == 0)")
            w("rt_first = t;")
            if ws:
                w(f"if (gidx >= {ring_bufs} && !frnn_mbar_wait(&full[{B_RGE} + rhalf], ((gidx / {ring_bufs}) - 1) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
            w.close()
        for go in grads:
            if go.cls != M1:
                continue
            val = go.value
            if sub.partial.get(val, False):
                raise LoweringError("per-row gradient came out as a sum over rows")
            w(f"float gv{go.index}[{t.R}];")
            w("#pragma unroll")
            w(f"for (int r = 0; r < {t.R}; r++) gv{go.index}[r] = {sub.at(val, 'r', '0')};")
            if go.over_t:
                w("#pragma unroll")
                w(f"for (int r = 0; r < {t.R}; r++) gacc{go.index}[r] += gv{go.index}[r];")
            elif go in row_st:
                kb.emit_obuf_put(f"gv{go.index}", "obuf", f"rhalf * {kflush} + rcnt", row_st.index(go), len(row_st))
            else:
                idx0 = _elem_off(go.spec, [(0, "b"), (1, "t"), (2, "h")])
                kb.emit_row_vec_store(f"gv{go.index}", go.spec.dt, f"dx{go.index}", idx0, go.spec.st(3),
                                      go.spec.aligned16 and all((go.spec.st(d) * ELT[go.spec.dt]) % 16 == 0 for d in (0, 1, 2)),
                                      atomic=go.atomic)
        for go in grads:
            if go.cls != MN:
                continue
            if sub.partial.get(go.value, False):
                raise LoweringError("matrix gradient came out as a sum over rows")
            sub.loops(MN, lambda r, c, go=go: f"gmat{go.index}[{r}*{t.C}+{c}] += {sub.at(go.value, r, c)};")
        if redw:
            w(f"float* rb = ring + (rhalf * {kflush} + rcnt) * {step_floats} + rg * {redw_pad};")
            for go in pm_vec:
                val = go.value
                is_pm = sub.partial.get(val, False)
                w(f"float pv{go.index}[{t.C}];")
                w("#pragma unroll")
                if is_pm:
                    w(f"for (int c = 0; c < {t.C}; c++) pv{go.index}[c] = {sub.at(val, '0', 'c')};")
                else:
                    w(f"for (int c = 0; c < {t.C}; c++) pv{go.index}[c] = (rg == 0) ? {sub.at(val, '0', 'c')} : 0.0f;")
                cnt = _pick_cnt(t.V, DT_F32, p.N)
                for j in range(t.NCH):
                    for q in range(t.V // cnt):
                        w(f"frnn_stv<0,{cnt}>(rb, {ring_off[go.index]} + cb + {j * t.V * t.L + q * cnt}, &pv{go.index}[{j * t.V + q * cnt}]);")
            for go in pm_sc:
                val = go.value
                is_pm = sub.partial.get(val, False)
                gate = "" if is_pm else "(rg == 0) ? "
                tail = "" if is_pm else " : 0.0f"
                w(f"if (l == 0) rb[{ring_off[go.index]}] = {gate}{sub.at(val, '0', '0')}{tail};")
            w("rcnt++;")
        for k in range(ns):
            o = outs[nin + k]
            sub.loops(stcls, lambda r, c, k=k, o=o: f"{body.at(dnext_names[k], r, c)} = {sub.at(o, r, c)};")

    if split:
        # values of the step's first part that its second part reads live across the fetch of S_t
        for n in crossing_values():
            body.declare(n.name, n.shape)
            step_parts["sub"].predeclared.add(n.name)
            step_parts["sub"].shape[n.name] = n.shape
    # ------------------------------------------------------------------ chunk loop
    w("#pragma unroll 1")
    w.open(f"for (int c = 0; c < {nchunk}; c++)")
    w(f"const int kc = {nchunk - 1} - c, t0 = kc * {D}, nv = min({D}, {p.T} - t0);")
    if ws:
        w(f"if (!frnn_mbar_wait(&full[{B_WKF} + (c & 1)], (c >> 1) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
        w(f"const float* wkc = wk + (c & 1) * {wk_floats}; (void)wkc;")
    else:
        w("unsigned char* sp = stage;")
        if kb.plain_items:
            w("if (kc > 0) {")
            w.ind += 1
            kb.emit_plain_load(f"(t0 - {D})", str(D))
            w.ind -= 1
            w("}")
        if has_tma:
            w(f"if (!frnn_mbar_wait(&full[{B_RAW}], c & 1, err, {ERR_STAGE_TIMEOUT})) return;")
        w("frnn_block_sync();   // previous chunk's work buffer is no longer read; plain stores are visible")
        kb.emit_convert("sp", "wk", "nv")
        w("frnn_block_sync();   // work buffer complete; the raw buffer may be refilled")
        if has_tma:
            w.open("if (warp == 0 && kc >= 1)")
            w(f"bw_issue(sp, &full[{B_RAW}], (kc - 1) * {D}, {D}, lane, b, h, m0{tma_call});")
            w.close()
        w("const float* wkc = wk; (void)wkc;")

    if rev:
        # reload an exact forward state at the end of this chunk when it is a checkpoint boundary
        w.open(f"if (c == 0 || (t0 + nv) % {dck} == 0)")
        w(f"const int kck = (c == 0) ? {nck} : (t0 + nv) / {dck};")
        for k in range(ns):
            base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, "kck")])
            kb.emit_tile_global(vname(p.st_names[k]), ckspec, f"ck{k}", base, 3, 4, load=True)
        w.close()
        kf = max(1, kflush)
        w("#pragma unroll 1")
        w.open(f"for (int g1 = nv; g1 > 0; g1 -= {kf})")
        w(f"const int g0 = max(g1 - {kf}, 0);")
        w(f"#pragma unroll {step_unroll}")
        w.open("for (int tl = g1 - 1; tl >= g0; tl--)")
        w("const int t = t0 + tl; (void)t;")
        w(f"const float* wkt = wkc + tl * {kb.wk_row}; (void)wkt;")
        w.open("")
        emit_bw_step()
        w.close()
        w.close()
        emit_flush()
        w.close()
    else:
        w(f"const int par = c & 1, nseg = (nv + {seg - 1}) / {seg}; (void)par;")
        w(f"#define PHYS(j) (par ? ({nphys - 1} - (j)) : (j))")
        if split:
            # the state registers hold the post-step state of the chunk's last step: the final state (first chunk
            # handled) or the pre-step state of the step handled just before
            w.open("if (c == 0)")
            for k in range(ns):
                base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, str(nck))])
                kb.emit_tile_global(vname(p.st_names[k]), ckspec, f"ck{k}", base, 3, 4, load=True)
            w.close()
            emit_part1("nv - 1")
        if ck_tma:
            w(f"if (!frnn_mbar_wait(&full[{B_CK}], c & 1, err, {ERR_CKPT_TIMEOUT})) return;")
        elif ws:
            csync("the plainly copied checkpoint is complete")
        # phase A: rebuild the segment bases
        slot_rw("0" if tm else "PHYS(0)", store=False)
        if tm:
            # the landing slot is free as soon as every thread holds its tile: fetch the next checkpoint a chunk ahead
            csync("every thread has read the landing slot")
            w.open("if (kc > 0)")
            ck_fetch("kc - 1", "0")
            w.close()
            tmem_rw("0", store=True)
        w("#pragma unroll 1")
        w.open("for (int j = 1; j < nseg; j++)")
        w("#pragma unroll" if unroll_segment else "#pragma unroll 1")
        w.open(f"for (int i = 0; i < {seg}; i++)")
        emit_restep(f"(j - 1) * {seg} + i")
        w.close()
        if tm:
            tmem_rw("j", store=True)
        else:
            slot_rw("PHYS(j)", store=True)
        w.close()
        if tm:
            w("frnn_tmem_wait_st();")
        # phase B: walk the chunk backwards
        w("#pragma unroll" if unroll_segment >= 2 else "#pragma unroll 1")
        w.open(f"for (int j = {(nslots if tm else nphys) - 1}; j >= 0; j--)")
        w.open("if (j < nseg)")
        w(f"const int seglen = min({seg}, nv - j * {seg});")
        # with ``unroll_segment`` the steps of a segment (and their re-steps) form one straight-line block
        w("#pragma unroll" if unroll_segment else "#pragma unroll 1")
        w.open(f"for (int i = {seg - 1}; i >= 0; i--)" if unroll_segment else "for (int i = seglen - 1; i >= 0; i--)")
        if unroll_segment:
            w.open("if (i < seglen)")
        if tm:
            tmem_rw("j", store=False)
        else:
            slot_rw("PHYS(j)", store=False)
        w("#pragma unroll" if unroll_segment else "#pragma unroll 1")
        w.open("for (int i2 = 0; i2 < i; i2++)")
        emit_restep(f"j * {seg} + i2")
        w.close()
        w.open("")
        w(f"const int tl = j * {seg} + i, t = t0 + tl; (void)t;")
        w(f"const float* wkt = wkc + tl * {kb.wk_row}; (void)wkt;")
        emit_bw_step()
        w.close()
        if redw and kflush > 1:
            w(f"if (rcnt == {kflush}) {{")
            w.ind += 1
            emit_flush()
            w.ind -= 1
            w("}")
        elif redw:
            emit_flush()
        if split:
            w.open(f"if (j * {seg} + i > 0)")
            emit_part1(f"j * {seg} + i - 1")
            w.close()
        if unroll_segment:
            w.close()   # if i < seglen
        w.close()   # i loop
        w.close()   # if j < nseg
        if not tm:
            w.open(f"if (j == {nphys - 1} && kc > 0)")
            csync("every thread is done with the slot that is overwritten next")
            ck_fetch("kc - 1", f"PHYS({nphys - 1})")
            w.close()
        w.close()   # j loop
        if redw and kflush > 1:
            emit_flush()
        w("#undef PHYS")
    if ws:
        w(f"frnn_mbar_arrive(&full[{B_WKE} + (c & 1)]);   // this thread no longer reads the chunk's work buffer")
    elif kb.plain_items:
        w("if (kc > 0) {")
        w.ind += 1
        kb.emit_plain_store("stage")
        w.ind -= 1
        w("}")
    w.close()   # chunk loop

    for k in range(ns):
        kb.emit_tile_global(vname(dnext_names[k]), p.states[k], f"ds0_{k}",
                            _elem_off(p.states[k], [(0, "b"), (1, "h")]), 2, 3, load=False)
    for go in grads:
        if go.over_t and go.cls == M1:
            idx0 = _elem_off(go.spec, [(0, "b"), (2, "h")])
            kb.emit_row_vec_store(f"gacc{go.index}", DT_F32, f"dx{go.index}", idx0, go.spec.st(3), False, atomic=True)
        if go.cls == MN:
            kb.emit_tile_global(f"gmat{go.index}", go.spec, f"dx{go.index}", _elem_off(go.spec, [(0, "b"), (2, "h")]),
                                3, 4, load=False, add=True)
    if not ws:
        emit_racc_final()
    if tm:
        w.ind -= 1
        w("};")
        w("scan();")
        w("// out of the scan, normally or after a timed-out wait: check in, and the allocating warp frees Tensor Memory")
        w("frnn_warp_sync();")
        w("if (lane == 0) frnn_smem_add((int*)&full[13], 1);")
        w.open("if (warp == 0)")
        w("const u64 t_exit = frnn_now_ns();")
        w(f"while (frnn_smem_add((int*)&full[13], 0) < {NCT // 32} && frnn_now_ns() - t_exit < 2 * FRNN_WAIT_LIMIT_NS) {{}}")
        w(f"frnn_tmem_dealloc(tm_base, {tm_cols}u);")
        w.close()
    w.close()
    return KernelSource(kname, w.text().replace("@SMEM_BYTES@", str(smem_bytes)), (p.M // t.MB, p.H, p.B), NCT + HT, smem_bytes,
                        kb.params, kb.param_decl,
                        {"stage_bytes": stage_bytes, "wk_bytes": kb.wk_bytes, "slot_bytes": slot_bytes if nphys else 0,
                         "ring_bytes": ring_bytes, "tma_items": len(kb.tma_items), "plain_items": len(kb.plain_items),
                         "nck": nck_store, "D": D, "dck": dck, "ck_tma": ck_tma, "kflush": kflush, "ring_bufs": ring_bufs,
                         "reverse": rev, "hoisted": [n.name for n in kb.hoisted], "tile": [t.R, t.C, t.MB],
                         "packed": bool(pack2), "helper_warps": helper_warps, "tmem_cols": tm_cols if tm else 0,
                         "seg": seg, "nslots": nslots, "post_split": split}, kb.tmaps)
