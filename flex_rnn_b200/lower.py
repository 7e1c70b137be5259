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
from typing import Dict, List, Optional, Sequence, Tuple

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
    C = min(pow2_le(want_c), N)
    while N % C:
        C //= 2
    while N // C > 32:
        C *= 2
    if N % C or 32 % (N // C):
        raise LoweringError(f"N={N} cannot be split over the lanes of a warp")
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
        elif C > 1 and N // (C // 2) <= 32:
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

class Body:
    """Emits per-thread code for graph nodes over R x C register tiles."""

    def __init__(self, w: W, tile: Tile, shapes: Dict[str, Shape]):
        self.w = w
        self.t = tile
        self.shape = dict(shapes)
        self.partial: Dict[str, bool] = {}     # value is a per-row-group partial sum

    # element accessor of a value (or literal) at tile position (r, c)
    def at(self, a, r: str, c: str) -> str:
        if not isinstance(a, str):
            return flit(a)
        s = self.shape[a]
        n = vname(a)
        if s == MN:
            return f"{n}[{r}*{self.t.C}+{c}]"
        if s == M1:
            return f"{n}[{r}]"
        if s == N1:
            return f"{n}[{c}]"
        return f"{n}[0]"

    def size(self, s: Shape) -> int:
        return (self.t.R if s[0] else 1) * (self.t.C if s[1] else 1)

    def declare(self, name: str, s: Shape, init: Optional[str] = None):
        self.shape[name] = s
        self.w(f"float {vname(name)}[{self.size(s)}];")
        if init is not None:
            self.loops(s, lambda r, c: f"{self.at(name, r, c)} = {init};")

    def loops(self, s: Shape, body):
        w = self.w
        if s[0]:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {self.t.R}; r++)")
        if s[1]:
            w("#pragma unroll")
            w.open(f"for (int c = 0; c < {self.t.C}; c++)")
        w(body("r" if s[0] else "0", "c" if s[1] else "0"))
        if s[1]:
            w.close()
        if s[0]:
            w.close()

    def expr(self, n: Node, r: str, c: str) -> str:
        a = [self.at(x, r, c) for x in n.args]
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
        if op == "copy":
            return a[0]
        if op == "const":
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
            # outer loops over the kept dims, inner accumulation over the reduced dims
            w.open("")
            if n.shape[0]:
                w("#pragma unroll")
                w.open(f"for (int r = 0; r < {t.R}; r++)")
            if n.shape[1]:
                w("#pragma unroll")
                w.open(f"for (int c = 0; c < {t.C}; c++)")
            w("float acc = 0.0f;")
            if n.over_m and ss[0]:
                w("#pragma unroll")
                w.open(f"for (int r = 0; r < {t.R}; r++)")
            if n.over_n and ss[1]:
                w("#pragma unroll")
                w.open(f"for (int c = 0; c < {t.C}; c++)")
            w(f"acc += {self.at(src, 'r', 'c')};")
            if n.over_n and ss[1]:
                w.close()
            if n.over_m and ss[0]:
                w.close()
            if n.over_n and ss[1] and t.L > 1:
                w(f"acc = frnn_row_sum<{t.L}>(acc);")
            w(f"{self.at(n.name, rs, cs)} = acc;")
            if n.shape[1]:
                w.close()
            if n.shape[0]:
                w.close()
            w.close()
            return
        self.partial[n.name] = self._check_partial(n)
        self.declare(n.name, n.shape)
        self.loops(n.shape, lambda r, c: f"{self.at(n.name, r, c)} = {self.expr(n, r, c)};")

    def graph(self, g: StepGraph, allow_over_m: bool = False):
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


class KernelBuilder:
    """State shared by the forward and backward emitters."""

    def __init__(self, p: Problem, tile: Tile, dstage: int, use_tma: bool):
        self.p = p
        self.t = tile
        self.D = dstage
        self.use_tma = use_tma
        self.w = W()
        self.items: List[StagedItem] = []
        self.params: List[str] = []
        self.param_decl: List[str] = []

    # -- parameters ----------------------------------------------------------
    def add_param(self, name: str, ctype: str, const: bool):
        self.params.append(name)
        q = "const " if const else ""
        r = " __restrict__" if const else ""
        self.param_decl.append(f"{q}{ctype}*{r} {name}")

    # -- staging plan ----------------------------------------------------------
    def add_item(self, key: str, cls: Shape, spec: TensorSpec, ptr: str, dims: Dict[str, int]):
        """``dims`` maps 'b','t','h','v' (the vector dim) to tensor dim indices."""
        t = self.t
        length = {N1: self.p.N, M1: t.MB, S11: 1}[cls]
        inner = spec.st(dims["v"]) if cls != S11 else 1
        base_dims = [(dims["b"], "b"), (dims["h"], "h")]
        if cls == M1:
            base_dims.append((dims["v"], "m0"))
        base = _elem_off(spec, base_dims)
        e = ELT[spec.dt]
        st_t = spec.st(dims["t"])
        tma = (self.use_tma and cls != S11 and inner == 1 and spec.aligned16
               and (length * e) % 16 == 0 and (st_t * e) % 16 == 0
               and (spec.st(dims["b"]) * e) % 16 == 0 and (spec.st(dims["h"]) * e) % 16 == 0
               and (cls != M1 or (t.MB * spec.st(dims["v"]) * e) % 16 == 0))
        rowb = (length * e + 15) // 16 * 16
        self.items.append(StagedItem(key, cls, spec.dt, ptr, length, base, st_t, inner, tma, 0, rowb))

    def layout_stage(self) -> int:
        off = 0
        # TMA items first (16-byte aligned rows), then plain ones
        for it in sorted(self.items, key=lambda i: not i.tma):
            it.off = off
            off += it.rowb * self.D
        self.stage_bytes = (off + 127) // 128 * 128
        self.tma_items = [i for i in self.items if i.tma]
        self.plain_items = [i for i in self.items if not i.tma]
        return self.stage_bytes

    # -- code pieces -------------------------------------------------------------
    def emit_thread_ids(self):
        w, t = self.w, self.t
        w("const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;")
        w(f"const int l = lane % {t.L}, g = lane / {t.L};")
        w(f"const int rg = warp * {t.G} + g;   // row group inside the CTA")
        w(f"const int m0 = blockIdx.x * {t.MB}, h = blockIdx.y, b = blockIdx.z;")
        w(f"const int row0 = m0 + rg * {t.R};  // first state row of this thread")
        w(f"const int cb = {t.V} * l;          // first state column of this thread")
        w("(void)row0; (void)cb; (void)m0; (void)h; (void)b;")

    def emit_tma_issue(self, fn: str):
        """Device function issuing the bulk copies of one chunk (warp 0 calls)."""
        w = self.w
        n = len(self.tma_items)
        bytes_per_step = sum(i.length * ELT[i.dt] for i in self.tma_items)
        w(f"// bulk copies of one chunk: {n} vectors per timestep, {bytes_per_step} bytes per timestep")
        self.tma_issue_args = ", ".join(f"const void* {i.ptr}" for i in self._uniq_ptr_items(self.tma_items))
        self.tma_issue_call = ", ".join(i.ptr for i in self._uniq_ptr_items(self.tma_items))
        w.open(f"FRNN_DEV void {fn}(unsigned char* stage, u64* bar, int t0, int nv, int lane, int b, int h, int m0"
               + (", " + self.tma_issue_args if n else "") + ")")
        if n:
            w(f"if (lane == 0) frnn_mbar_expect_tx(bar, (u32)nv * {bytes_per_step}u);")
            w("frnn_warp_sync();")
            w.open(f"for (int i = lane; i < nv * {n}; i += 32)")
            w(f"const int k = i % {n}, tl = i / {n};")
            w.open("switch (k)")
            for k, it in enumerate(self.tma_items):
                e = ELT[it.dt]
                w(f"case {k}: frnn_bulk_g2s(stage + {it.off} + tl * {it.rowb}, "
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
            w(f"if (tl < {nv}) pl{k}[q] = (({'const ' + CTYPE[it.dt]}*){it.ptr})"
              f"[{it.base} + (long)({t0} + tl) * {it.stride_t}L + (long)j * {it.inner}L];")
            w.close()

    def emit_plain_store(self, stage: str):
        w, t = self.w, self.t
        for k, (it, cnt) in enumerate(self.plain_regs()):
            w("#pragma unroll")
            w.open(f"for (int q = 0; q < {cnt}; q++)")
            w(f"const int e = tid + q * {t.NT}, tl = e / {it.length}, j = e % {it.length};")
            w(f"if (tl < {self.D}) (({CTYPE[it.dt]}*)({stage} + {it.off} + tl * {it.rowb}))[j] = pl{k}[q];")
            w.close()

    def emit_item_read(self, body: Body, it: StagedItem, sp: str, name: str):
        """Read one staged vector of the current timestep into registers."""
        w, t = self.w, self.t
        body.declare(name, it.cls)
        n = vname(name)
        src = f"({sp} + {it.off} + tl * {it.rowb})"
        if it.cls == N1:
            cnt = _pick_cnt(t.V, it.dt)
            for j in range(t.NCH):
                for q in range(t.V // cnt):
                    w(f"frnn_ldv<{it.dt},{cnt}>({src}, cb + {j * t.V * t.L + q * cnt}, &{n}[{j * t.V + q * cnt}]);")
        elif it.cls == M1:
            cnt = _pick_cnt(t.R, it.dt, t.R)
            for q in range(t.R // cnt):
                w(f"frnn_ldv<{it.dt},{cnt}>({src}, rg * {t.R} + {q * cnt}, &{n}[{q * cnt}]);")
        else:
            w(f"{n}[0] = frnn_io<{it.dt}>::ld({src}, 0);")

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
        if cls in (N1, MN):
            ncol = dims["n"]
        if cls in (M1, MN):
            nrow = dims["m"]
        if cls == N1:
            for j in range(t.NCH):
                for e in range(t.V):
                    w(f"{n}[{j * t.V + e}] = frnn_io<{spec.dt}>::ld({ptr}, {base} + (long){t.col(j, e)} * {spec.st(ncol)}L);")
        elif cls == M1:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            w(f"{n}[r] = frnn_io<{spec.dt}>::ld({ptr}, {base} + (long)(row0 + r) * {spec.st(nrow)}L);")
            w.close()
        else:
            self.emit_tile_global(n, spec, ptr, base, nrow, ncol, load=True)

    def emit_tile_global(self, arr: str, spec: TensorSpec, ptr: str, base: str, dm: int, dn: int,
                         load: bool, add: bool = False):
        """Strided global load / store of an R x C register tile (any strides)."""
        w, t = self.w, self.t
        sm, sn = spec.st(dm), spec.st(dn)
        if sn == 1 and t.V > 1 and spec.aligned16 and (sm * ELT[spec.dt]) % 16 == 0 and not add:
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
                    w(f"frnn_atomic_add((float*){ptr} + ({idx}), {el});")
                else:
                    w(f"frnn_io<{spec.dt}>::st({ptr}, {idx}, {el});")
        w.close()

    def emit_row_vec_store(self, arr: str, dt: int, ptr: str, idx0: str, stride_m: int, aligned: bool,
                           atomic: bool = False):
        """Lane 0 of each row group stores R per-row values (rows row0..row0+R)."""
        w, t = self.w, self.t
        w.open("if (l == 0)")
        if atomic:
            w("#pragma unroll")
            w.open(f"for (int r = 0; r < {t.R}; r++)")
            w(f"frnn_atomic_add((float*){ptr} + ({idx0} + (long)(row0 + r) * {stride_m}L), {arr}[r]);")
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


# ---------------------------------------------------------------------------
# forward kernel
# ---------------------------------------------------------------------------

def emit_forward(p: Problem, g: StepGraph, aux_names: List[str], n_out: int, tile: Tile,
                 dstage: int, dck: int, use_tma: bool, min_blocks: int, prelude: str,
                 kname: str = "frnn_fw") -> KernelSource:
    """Forward scan.  ``g`` computes [*outputs, *new_states, *aux] from
    [*inputs, *states].  Kernel parameters, in order: used inputs, initial
    states, outputs, final states, checkpoints, aux, error word."""
    kb = KernelBuilder(p, tile, dstage, use_tma)
    w, t = kb.w, tile
    ns = len(p.states)
    used = g.used_inputs()
    stcls = p.st_cls()

    for i, spec in enumerate(p.inputs):
        if used[i]:
            kb.add_param(f"in{i}", "void", True)
    for k in range(ns):
        kb.add_param(f"s0_{k}", "void", True)
    for j in range(n_out):
        kb.add_param(f"out{j}", "void", False)
    for k in range(ns):
        kb.add_param(f"sT_{k}", "void", False)
    for k in range(ns):
        kb.add_param(f"ck{k}", "float", False)
    kb.add_param("aux", "float", False)
    kb.add_param("err", "int", False)

    const_inputs = []
    for i, spec in enumerate(p.inputs):
        if not used[i]:
            continue
        cls = p.in_cls(i)
        if cls == MN or spec.shape[1] == 1:
            if cls == MN and spec.shape[1] != 1:
                raise LoweringError("an input that is a full matrix per head must not depend on time")
            const_inputs.append(i)
        else:
            kb.add_item(p.in_names[i], cls, spec, f"in{i}", _in_dims(cls))
    stage_bytes = kb.layout_stage()
    BAR_BYTES = 128
    smem_bytes = BAR_BYTES + 2 * stage_bytes
    nchunk = (p.T + dstage - 1) // dstage
    nck = (p.T + dck - 1) // dck

    w(_header(prelude))
    w(f"// forward scan: B={p.B} T={p.T} H={p.H} M={p.M} N={p.N}; tile R={t.R} C={t.C} L={t.L} MB={t.MB}; "
      f"stage {dstage} steps, checkpoint every {dck}")
    kb.emit_tma_issue("fw_issue")
    w(f'extern "C" __global__ void __launch_bounds__({t.NT}, {min_blocks})')
    w.open(f"{kname}({', '.join(kb.param_decl)})")
    w("FRNN_DYN_SMEM(smem);")
    kb.emit_thread_ids()
    w("u64* full = (u64*)smem;")
    w(f"unsigned char* stage = smem + {BAR_BYTES};")
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
        if nchunk > 1:
            w(f"fw_issue(stage + {stage_bytes}, &full[1], {dstage}, min({dstage}, {p.T - dstage}), lane, b, h, m0{tma_call});")
        w.close()
    w("frnn_block_sync();")

    body = Body(w, t, g.shape)
    # states
    for k in range(ns):
        body.declare(p.st_names[k], stcls)
        kb.emit_tile_global(vname(p.st_names[k]), p.states[k], f"s0_{k}",
                            _elem_off(p.states[k], [(0, "b"), (1, "h")]), 2, 3, load=True)
    for i in const_inputs:
        kb.emit_const_input(body, p.in_names[i], p.in_cls(i), p.inputs[i], f"in{i}", IN_DIMS)

    w("#pragma unroll 1")
    w.open(f"for (int c = 0; c < {nchunk}; c++)")
    w(f"const int buf = c & 1, t0 = c * {dstage}, nv = min({dstage}, {p.T} - t0);")
    w(f"unsigned char* sp = stage + buf * {stage_bytes};")
    if kb.plain_items:
        w(f"if (c + 1 < {nchunk}) {{")
        w.ind += 1
        kb.emit_plain_load(f"(t0 + {dstage})", f"min({dstage}, {p.T} - t0 - {dstage})")
        w.ind -= 1
        w("}")
    if has_tma:
        w(f"if (!frnn_mbar_wait(&full[buf], (c >> 1) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
    w("#pragma unroll 1")
    w.open("for (int tl = 0; tl < nv; tl++)")
    w("const int t = t0 + tl;")
    # checkpoint of the state before step t
    w.open(f"if (t % {dck} == 0)")
    for k in range(ns):
        ckspec = TensorSpec((p.B, p.H, nck, p.M, p.N), _contig((p.B, p.H, nck, p.M, p.N)), DT_F32)
        base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, f"t / {dck}")])
        kb.emit_tile_global(vname(p.st_names[k]), ckspec, f"ck{k}", base, 3, 4, load=False)
    w.close()
    sub = Body(w, t, body.shape)
    w.open("")
    for it in kb.items:
        kb.emit_item_read(sub, it, "sp", it.key)
    sub.graph(g, allow_over_m=False)
    outs = g.outputs
    # outputs y_j -> out[b, t, h, m]
    yspec_shape = (p.B, p.T, p.H, p.M)
    for j in range(n_out):
        o = outs[j]
        ys = TensorSpec(yspec_shape, _contig(yspec_shape), p.out_dt[j])
        w(f"float yv{j}[{t.R}];")
        w("#pragma unroll")
        w(f"for (int r = 0; r < {t.R}; r++) yv{j}[r] = {sub.at(o, 'r', '0')};")
        kb.emit_row_vec_store(f"yv{j}", p.out_dt[j], f"out{j}",
                              _elem_off(ys, [(0, "b"), (1, "t"), (2, "h")]), 1,
                              (p.M * ELT[p.out_dt[j]]) % 16 == 0)
    # aux row sums -> aux[a, b, h, t, m]
    ashape = (max(1, p.naux), p.B, p.H, p.T, p.M)
    aspec = TensorSpec(ashape, _contig(ashape), DT_F32)
    for a, an in enumerate(aux_names):
        w(f"float av{a}[{t.R}];")
        w("#pragma unroll")
        w(f"for (int r = 0; r < {t.R}; r++) av{a}[r] = {sub.at(an, 'r', '0')};")
        kb.emit_row_vec_store(f"av{a}", DT_F32, "aux",
                              _elem_off(aspec, [(0, str(a)), (1, "b"), (2, "h"), (3, "t")]), 1,
                              (p.M * 4) % 16 == 0)
    # new state
    for k in range(ns):
        o = outs[n_out + k]
        sub.loops(stcls, lambda r, c, k=k, o=o: f"{body.at(p.st_names[k], r, c)} = {sub.at(o, r, c)};")
    w.close()
    w.close()  # tl loop
    if kb.plain_items:
        w(f"if (c + 1 < {nchunk}) {{")
        w.ind += 1
        kb.emit_plain_store(f"(stage + (buf ^ 1) * {stage_bytes})")
        w.ind -= 1
        w("}")
    w("frnn_block_sync();")
    if has_tma:
        w.open(f"if (warp == 0 && c + 2 < {nchunk})")
        w(f"fw_issue(sp, &full[buf], t0 + {2 * dstage}, min({dstage}, {p.T} - t0 - {2 * dstage}), lane, b, h, m0{tma_call});")
        w.close()
    w.close()  # chunk loop
    for k in range(ns):
        # final state, laid out like the initial state
        kb.emit_tile_global(vname(p.st_names[k]), p.states[k], f"sT_{k}",
                            _elem_off(p.states[k], [(0, "b"), (1, "h")]), 2, 3, load=False)
    w.close()
    return KernelSource(kname, w.text(), (p.M // t.MB, p.H, p.B), t.NT, smem_bytes, kb.params, kb.param_decl,
                        {"stage_bytes": stage_bytes, "tma_items": len(kb.tma_items),
                         "plain_items": len(kb.plain_items), "nck": nck})


def _contig(shape: Sequence[int]) -> Tuple[int, ...]:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return tuple(reversed(st))


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


def emit_backward(p: Problem, g_re: StepGraph, g_bw: StepGraph, aux_names: List[str], n_out: int,
                  grads: List[GradOut], dstate_names: List[str], dy_names: List[str],
                  dnext_names: List[str], tile: Tile, seg: int, nslots: int, use_tma: bool,
                  prelude: str, kname: str = "frnn_bw", red_bufs: int = 2) -> KernelSource:
    """Reverse-time kernel.

    ``g_re`` computes the new states from [*inputs, *states, *aux];
    ``g_bw`` computes [*d_inputs, *d_states] from
    [*inputs, *states, *d_outputs, *d_new_states, *aux].
    Checkpoint chunk length D = seg * nslots.  Parameters, in order: used
    inputs, d_outputs, d_final_states, checkpoints, aux, d_initial_states,
    input gradients (those in ``grads``), error word.
    """
    D = seg * nslots
    kb = KernelBuilder(p, tile, D, use_tma)
    w, t = kb.w, tile
    if t.MB != p.M:
        raise LoweringError("the backward kernel needs all rows of a head in one CTA")
    ns = len(p.states)
    stcls = p.st_cls()
    nin = len(p.inputs)
    used_re, used_bw = g_re.used_inputs(), g_bw.used_inputs()
    used = [used_re[i] or used_bw[i] for i in range(nin)]
    dy_used = [used_bw[nin + ns + j] for j in range(n_out)]
    nck = (p.T + D - 1) // D

    for i in range(nin):
        if used[i]:
            kb.add_param(f"in{i}", "void", True)
    for j in range(n_out):
        kb.add_param(f"dy{j}", "void", True)
    for k in range(ns):
        kb.add_param(f"dsT_{k}", "void", True)
    for k in range(ns):
        kb.add_param(f"ck{k}", "float", True)
    kb.add_param("aux", "float", True)
    for k in range(ns):
        kb.add_param(f"ds0_{k}", "void", False)
    for go in grads:
        kb.add_param(f"dx{go.index}", "void", False)
    kb.add_param("err", "int", False)

    const_inputs = []
    for i, spec in enumerate(p.inputs):
        if not used[i]:
            continue
        cls = p.in_cls(i)
        if cls == MN:
            raise LoweringError("matrix-per-head inputs are not supported by the backward kernel yet")
        if spec.shape[1] == 1:
            const_inputs.append(i)
        else:
            kb.add_item(p.in_names[i], cls, spec, f"in{i}", _in_dims(cls))
    ashape = (max(1, p.naux), p.B, p.H, p.T, p.M)
    aspec = TensorSpec(ashape, _contig(ashape), DT_F32)
    for a, an in enumerate(aux_names):
        sp_a = TensorSpec(ashape[1:], _contig(ashape)[1:], DT_F32)
        kb.add_item(an, M1, sp_a, "aux", {"b": 0, "h": 1, "t": 2, "v": 3})
        kb.items[-1].base = f"{a * p.B * p.H * p.T * p.M}L + " + kb.items[-1].base
    yshape = (p.B, p.T, p.H, p.M)
    for j in range(n_out):
        if dy_used[j]:
            ys = TensorSpec(yshape, _contig(yshape), p.out_dt[j])
            kb.add_item(dy_names[j], M1, ys, f"dy{j}", {"b": 0, "t": 1, "h": 2, "v": 3})
    stage_bytes = kb.layout_stage()

    # partial-sum exchange layout: per row group, all 1N gradients then all 11 gradients
    pm_vec = [go for go in grads if go.cls == N1]
    pm_sc = [go for go in grads if go.cls == S11]
    redw = len(pm_vec) * p.N + len(pm_sc)
    redw_pad = (redw + 3) // 4 * 4
    red_bytes = red_bufs * t.RG * redw_pad * 4 if redw else 0
    nphys = max(nslots, 2)
    slot_elems = p.M * p.N
    slot_bytes = slot_elems * 4
    ck_tma = use_tma and slot_bytes % 16 == 0
    BAR_BYTES = 128
    off_stage = BAR_BYTES
    off_slots = off_stage + 2 * stage_bytes
    off_red = off_slots + nphys * ns * slot_bytes
    smem_bytes = off_red + red_bytes

    w(_header(prelude))
    w(f"// backward scan: B={p.B} T={p.T} H={p.H} M={p.M} N={p.N}; tile R={t.R} C={t.C} L={t.L}; "
      f"chunk {D} = {nslots} segments x {seg} steps")
    kb.emit_tma_issue("bw_issue")

    # ---- restep and backward step as device functions over register tiles ----
    sz = lambda s: (t.R if s[0] else 1) * (t.C if s[1] else 1)

    w(f'extern "C" __global__ void __launch_bounds__({t.NT}, 1)')
    w.open(f"{kname}({', '.join(kb.param_decl)})")
    w("FRNN_DYN_SMEM(smem);")
    kb.emit_thread_ids()
    w("u64* full = (u64*)smem;        // [0],[1]: staged inputs   [2]: checkpoint copy")
    w(f"unsigned char* stage = smem + {off_stage};")
    w(f"float* slots = (float*)(smem + {off_slots});")
    if redw:
        w(f"float* red = (float*)(smem + {off_red});")
    has_tma = bool(kb.tma_items)
    w.open("if (tid == 0)")
    w("frnn_mbar_init(&full[0], 1); frnn_mbar_init(&full[1], 1); frnn_mbar_init(&full[2], 1); frnn_mbar_init_fence();")
    w.close()
    w("frnn_block_sync();")
    kb.emit_plain_decl()
    tma_call = (", " + kb.tma_issue_call) if has_tma else ""

    ckspec = TensorSpec((p.B, p.H, nck, p.M, p.N), _contig((p.B, p.H, nck, p.M, p.N)), DT_F32)

    def ck_fetch(kexpr: str, physexpr: str):
        """Start the copy of checkpoint ``kexpr`` into physical slot ``physexpr``."""
        if ck_tma:
            w.open("if (tid == 0)")
            w("frnn_async_proxy_fence();")
            w(f"frnn_mbar_expect_tx(&full[2], {ns * slot_bytes}u);")
            for k in range(ns):
                base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, kexpr)])
                w(f"frnn_bulk_g2s(slots + ((long)({physexpr}) * {ns} + {k}) * {slot_elems}, ck{k} + {base}, {slot_bytes}u, &full[2]);")
            w.close()
        else:
            for k in range(ns):
                base = _elem_off(ckspec, [(0, "b"), (1, "h"), (2, kexpr)])
                w(f"for (int e = tid; e < {slot_elems}; e += {t.NT}) "
                  f"slots[((long)({physexpr}) * {ns} + {k}) * {slot_elems} + e] = ck{k}[{base} + e];")

    first_k = nck - 1
    nv_first = p.T - first_k * D
    if kb.plain_items:
        kb.emit_plain_load(str(first_k * D), str(nv_first))
        kb.emit_plain_store("stage")
    if has_tma:
        w.open("if (warp == 0)")
        w(f"bw_issue(stage, &full[0], {first_k * D}, {nv_first}, lane, b, h, m0{tma_call});")
        if nck > 1:
            w(f"bw_issue(stage + {stage_bytes}, &full[1], {(first_k - 1) * D}, {D}, lane, b, h, m0{tma_call});")
        w.close()
    ck_fetch(str(first_k), "0")
    w("frnn_block_sync();")

    body = Body(w, t, g_bw.shape)
    body.shape.update(g_re.shape)
    # d_state registers, seeded with the gradient of the final state (contiguous [B,H,M,N])
    dshape = (p.B, p.H, p.M, p.N)
    for k in range(ns):
        body.declare(dnext_names[k], stcls)
        dspec = TensorSpec(dshape, _contig(dshape), p.states[k].dt)
        kb.emit_tile_global(vname(dnext_names[k]), dspec, f"dsT_{k}",
                            _elem_off(dspec, [(0, "b"), (1, "h")]), 2, 3, load=True)
        body.declare(p.st_names[k], stcls)
    for i in const_inputs:
        kb.emit_const_input(body, p.in_names[i], p.in_cls(i), p.inputs[i], f"in{i}", IN_DIMS)
    # accumulators for gradients of time-invariant inputs
    for go in grads:
        if go.over_t and go.cls == M1:
            w(f"float gacc{go.index}[{t.R}];")
            w(f"#pragma unroll")
            w(f"for (int r = 0; r < {t.R}; r++) gacc{go.index}[r] = 0.0f;")
    nred_per_thread = (redw + t.NT - 1) // t.NT if redw else 0
    if any(go.over_t and go.cls != M1 for go in grads):
        w(f"float racc[{max(1, nred_per_thread)}];")
        w(f"#pragma unroll")
        w(f"for (int q = 0; q < {max(1, nred_per_thread)}; q++) racc[q] = 0.0f;")
    w("int rpar = 0; (void)rpar;")

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

    def emit_restep(tlexpr: str):
        w.open("")
        w(f"const int tl = {tlexpr};")
        sub = Body(w, t, body.shape)
        for it in kb.items:
            if it.key in g_re.inputs and g_re.used_inputs()[g_re.inputs.index(it.key)]:
                kb.emit_item_read(sub, it, "sp", it.key)
        sub.graph(g_re)
        for k in range(ns):
            o = g_re.outputs[k]
            sub.loops(stcls, lambda r, c, k=k, o=o: f"{body.at(p.st_names[k], r, c)} = {sub.at(o, r, c)};")
        w.close()

    w("#pragma unroll 1")
    w.open(f"for (int c = 0; c < {nck}; c++)")
    w(f"const int kc = {nck - 1} - c, t0 = kc * {D}, nv = min({D}, {p.T} - t0), buf = c & 1, par = c & 1;")
    w(f"const int nseg = (nv + {seg - 1}) / {seg};")
    w(f"unsigned char* sp = stage + buf * {stage_bytes};")
    w(f"#define PHYS(j) (par ? ({nphys - 1} - (j)) : (j))")
    if kb.plain_items:
        w("if (kc > 0) {")
        w.ind += 1
        kb.emit_plain_load(f"(t0 - {D})", str(D))
        w.ind -= 1
        w("}")
    if has_tma:
        w(f"if (!frnn_mbar_wait(&full[buf], (c >> 1) & 1, err, {ERR_STAGE_TIMEOUT})) return;")
    if ck_tma:
        w(f"if (!frnn_mbar_wait(&full[2], c & 1, err, {ERR_CKPT_TIMEOUT})) return;")
    # phase A: rebuild the segment bases
    slot_rw("PHYS(0)", store=False)
    w("#pragma unroll 1")
    w.open("for (int j = 1; j < nseg; j++)")
    w("#pragma unroll 1")
    w.open(f"for (int i = 0; i < {seg}; i++)")
    emit_restep(f"(j - 1) * {seg} + i")
    w.close()
    slot_rw("PHYS(j)", store=True)
    w.close()
    # phase B: walk the chunk backwards
    w("#pragma unroll 1")
    w.open(f"for (int j = {nphys - 1}; j >= 0; j--)")
    w.open("if (j < nseg)")
    w(f"const int seglen = min({seg}, nv - j * {seg});")
    w("#pragma unroll 1")
    w.open("for (int i = seglen - 1; i >= 0; i--)")
    slot_rw("PHYS(j)", store=False)
    w("#pragma unroll 1")
    w.open("for (int i2 = 0; i2 < i; i2++)")
    emit_restep(f"j * {seg} + i2")
    w.close()
    # ---- the backward step proper
    w.open("")
    w(f"const int tl = j * {seg} + i, t = t0 + tl;")
    sub = Body(w, t, body.shape)
    bw_used = dict(zip(g_bw.inputs, g_bw.used_inputs()))
    for it in kb.items:
        if bw_used.get(it.key, False):
            kb.emit_item_read(sub, it, "sp", it.key)
    sub.graph(g_bw, allow_over_m=True)
    outs = g_bw.outputs
    # per-row gradients (inputs that vary over rows)
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
        else:
            idx0 = _elem_off(go.spec, [(0, "b"), (1, "t"), (2, "h")])
            kb.emit_row_vec_store(f"gv{go.index}", go.spec.dt, f"dx{go.index}", idx0, go.spec.st(3),
                                  go.spec.aligned16 and all((go.spec.st(d) * ELT[go.spec.dt]) % 16 == 0 for d in (0, 1, 2)),
                                  atomic=go.atomic)
    # per-column / per-head gradient partials -> exchange buffer
    if redw:
        if red_bufs == 1:
            w("frnn_block_sync();   // single exchange buffer: the previous step's readers must be done")
        w(f"float* rb = red + rpar * {t.RG * redw_pad} + rg * {redw_pad};")
        for vi, go in enumerate(pm_vec):
            val = go.value
            is_pm = sub.partial.get(val, False)
            w(f"float pv{vi}[{t.C}];")
            w("#pragma unroll")
            if is_pm:
                w(f"for (int c = 0; c < {t.C}; c++) pv{vi}[c] = {sub.at(val, '0', 'c')};")
            else:
                # not a sum over rows (e.g. identically zero): only row group 0 contributes
                w(f"for (int c = 0; c < {t.C}; c++) pv{vi}[c] = (rg == 0) ? {sub.at(val, '0', 'c')} : 0.0f;")
            cnt = _pick_cnt(t.V, DT_F32, p.N)
            for j in range(t.NCH):
                for q in range(t.V // cnt):
                    w(f"frnn_stv<0,{cnt}>(rb, {vi * p.N} + cb + {j * t.V * t.L + q * cnt}, &pv{vi}[{j * t.V + q * cnt}]);")
        for si, go in enumerate(pm_sc):
            val = go.value
            is_pm = sub.partial.get(val, False)
            gate = "" if is_pm else "(rg == 0) ? "
            tail = "" if is_pm else " : 0.0f"
            w(f"if (l == 0) rb[{len(pm_vec) * p.N + si}] = {gate}{sub.at(val, '0', '0')}{tail};")
    # d_state for the previous step
    nin_bw = len(p.inputs)
    for k in range(ns):
        o = outs[nin_bw + k]
        sub.loops(stcls, lambda r, c, k=k, o=o: f"{body.at(dnext_names[k], r, c)} = {sub.at(o, r, c)};")
    if redw:
        w("frnn_block_sync();")
        w(f"const float* rr = red + rpar * {t.RG * redw_pad};")
        w("#pragma unroll")
        w.open(f"for (int q = 0; q < {nred_per_thread}; q++)")
        w(f"const int e = tid + q * {t.NT};")
        w.open(f"if (e < {redw})")
        w("float a = 0.0f;")
        w("#pragma unroll 4")
        w(f"for (int gi = 0; gi < {t.RG}; gi++) a += rr[gi * {redw_pad} + e];")
        # dispatch on which gradient element e belongs to
        lo = 0
        for go in pm_vec + pm_sc:
            n_el = p.N if go.cls == N1 else 1
            cond = f"e >= {lo} && e < {lo + n_el}" if len(pm_vec) + len(pm_sc) > 1 else "true"
            w.open(f"if ({cond})")
            j = f"(e - {lo})"
            if go.over_t:
                w("racc[q] += a;")
            else:
                dims = [(0, "b"), (1, "t"), (2, "h")] + ([(4, j)] if go.cls == N1 else [])
                idx = _elem_off(go.spec, dims)
                if go.atomic:
                    w(f"frnn_atomic_add((float*)dx{go.index} + ({idx}), a);")
                else:
                    w(f"frnn_io<{go.spec.dt}>::st(dx{go.index}, {idx}, a);")
            w.close()
            lo += n_el
        w.close()
        w.close()
        if red_bufs == 2:
            w("rpar ^= 1;")
    w.close()   # backward step scope
    w.close()   # i loop
    w.close()   # if j < nseg
    # the highest physical slot of this parity is free now: fetch the next checkpoint into it
    w.open(f"if (j == {nphys - 1} && kc > 0)")
    w("frnn_block_sync();")
    ck_fetch("kc - 1", f"PHYS({nphys - 1})")
    w.close()
    w.close()   # j loop
    if kb.plain_items:
        w("if (kc > 0) {")
        w.ind += 1
        kb.emit_plain_store(f"(stage + (buf ^ 1) * {stage_bytes})")
        w.ind -= 1
        w("}")
    w("frnn_block_sync();")
    if has_tma:
        w.open("if (warp == 0 && kc >= 2)")
        w(f"bw_issue(sp, &full[buf], (kc - 2) * {D}, {D}, lane, b, h, m0{tma_call});")
        w.close()
    w("#undef PHYS")
    w.close()   # chunk loop

    # d_initial_state, laid out like the initial state
    for k in range(ns):
        kb.emit_tile_global(vname(dnext_names[k]), p.states[k], f"ds0_{k}",
                            _elem_off(p.states[k], [(0, "b"), (1, "h")]), 2, 3, load=False)
    # gradients of time-invariant inputs
    for go in grads:
        if not go.over_t:
            continue
        if go.cls == M1:
            idx0 = _elem_off(go.spec, [(0, "b"), (2, "h")])
            kb.emit_row_vec_store(f"gacc{go.index}", DT_F32, f"dx{go.index}", idx0, go.spec.st(3), False, atomic=True)
    if any(go.over_t and go.cls != M1 for go in grads):
        w("#pragma unroll")
        w.open(f"for (int q = 0; q < {nred_per_thread}; q++)")
        w(f"const int e = tid + q * {t.NT};")
        lo = 0
        for go in pm_vec + pm_sc:
            n_el = p.N if go.cls == N1 else 1
            if go.over_t:
                w.open(f"if (e >= {lo} && e < {lo + n_el})")
                dims = [(0, "b"), (2, "h")] + ([(4, f"(e - {lo})")] if go.cls == N1 else [])
                w(f"frnn_atomic_add((float*)dx{go.index} + ({_elem_off(go.spec, dims)}), racc[q]);")
                w.close()
            lo += n_el
        w.close()
    w.close()
    return KernelSource(kname, w.text(), (1, p.H, p.B), t.NT, smem_bytes, kb.params, kb.param_decl,
                        {"stage_bytes": stage_bytes, "slot_bytes": slot_bytes, "red_bytes": red_bytes,
                         "tma_items": len(kb.tma_items), "plain_items": len(kb.plain_items),
                         "nck": nck, "D": D, "ck_tma": ck_tma})
