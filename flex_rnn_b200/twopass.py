"""Planner and host closures of the B200 backend.

Same contract as the reference's ``flex_rnn.twopass`` (flex_rnn/twopass.py:44,
191-192, 224-237, 343-366 in the reference project), which is what the ``jit``
front end calls:

    build_twopass(step, inputs, state, dryrun=False)
        -> (forward, backward, forward_meta, backward_meta)   or, with dryrun,
        -> (forward_meta, backward_meta)

    forward(inputs, state0)  -> (*outputs[B,T,H,M], *final_states, *state_store, aux)
    backward(doutput, dstateT, inputs, state_store, aux) -> (tuple(dinputs), tuple(dstate0))

What differs is everything underneath: the joint graph is sliced into three
sub-graphs (forward step, reduction-free re-step, backward step) instead of
five, two kernels are generated instead of three (``lower.py``), they are
compiled with NVRTC and launched through the C-ABI library on the current
stream, checkpoints are stored untransposed every ``seg * nslots`` steps, and
no dstate checkpoints or ``daux`` buffers exist.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch as th

from . import lower
from .graph import MN, M1, N1, S11, StepGraph
from .lower import (DT_BF16, DT_F16, DT_F32, DT_F64, GradOut, Problem, TensorSpec, choose_tile,
                    emit_backward, emit_forward)
from .trace import as_tuple, run_isolated, trace_joint

_DT = {th.float32: DT_F32, th.bfloat16: DT_BF16, th.float16: DT_F16, th.float64: DT_F64}
_IO_DTYPES = (th.float32, th.bfloat16, th.float16, th.float64)
_PRELUDE: Optional[str] = None


def prelude() -> str:
    global _PRELUDE
    if _PRELUDE is None:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "frnn_device.cuh")) as f:
            _PRELUDE = f.read()
    return _PRELUDE


# -- small helpers with the reference's names (flex_rnn/twopass.py:8-42) -------

def split_list(args, lens):
    """Cut ``args`` into consecutive pieces of the given lengths."""
    out, pos = [], 0
    for n in lens:
        out.append(args[pos:pos + n])
        pos += n
    assert pos == len(args), f"expected {pos} arguments, got {len(args)}"
    return out


def get_meta(tensors):
    return tuple((t.shape, t.stride(), t.dtype) for t in tensors)


def verify_meta(a, b, msg=""):
    """Shapes, dtypes and strides (of dims larger than 1) of ``a`` must equal ``b``'s."""
    for i, (x, y) in enumerate(zip(a, b)):
        assert x.shape == y.shape, msg + f"#{i + 1}: shape {tuple(x.shape)} != {tuple(y.shape)}"
        sx = [s if n > 1 else 0 for s, n in zip(x.stride(), x.shape)]
        sy = [s if n > 1 else 0 for s, n in zip(y.stride(), y.shape)]
        assert sx == sy, msg + f"#{i + 1}: stride {sx} != {sy}"
        assert x.dtype == y.dtype, msg + f"#{i + 1}: dtype {x.dtype} != {y.dtype}"


# -- tunables -------------------------------------------------------------------

@dataclass
class Tuning:
    """Code-generation parameters (defaults picked by ``default_tuning``)."""
    fw_r: int = 4            # forward tile: rows x columns per thread, rows per CTA
    fw_c: int = 32
    fw_mb: int = 128
    fw_stage: int = 16       # timesteps per staged chunk (forward)
    fw_min_blocks: int = 1
    bw_r: int = 8            # backward tile
    bw_c: int = 8
    bw_mb: int = 0           # state rows per backward CTA (0 = all rows of a head, fewer only when they do not fit one CTA)
    seg: int = 4             # generic backward: steps per segment, segments (slots) per checkpoint chunk
    nslots: int = 2
    kflush: int = 8          # steps of gradient partials reduced together (lowered until shared memory fits)
    reverse: int = 1         # use the reverse re-step when the state update is additive
    rev_stage: int = 16      # reverse mode: timesteps per staged chunk
    rev_resync: int = 4      # reverse mode: chunks between exact checkpoints (without helper warps)
    rev_ckpt: int = 64       # reverse mode with helper warps: timesteps between exact checkpoints
    bw_helper: int = 1       # backward helper warps: they stage the inputs and flush the gradient partials while the
                             # tile's warps run the scan; 0 = every warp does everything, with block barriers between
    fw_unroll: int = 4       # unroll factor of the timestep loops
    bw_unroll: int = 4
    slot_search: int = 1     # generic backward: try 4 slots x 2 steps before seg x nslots
    col_major: int = 0       # emit full-tile loops with columns outermost
    bw_min_blocks: int = 0   # backward CTAs per SM the kernel is built for (2: half the registers and shared memory
                             # each); 0 = two when the planned tile gives CTAs of at most 128 threads, else one
    pack2: int = 1           # packed fp32x2 arithmetic (two columns per instruction): bit 0 backward, bit 1 forward
    bw_pack_small: int = 0   # packed arithmetic also in backward kernels built for two CTAs of four compute warps per
                             # SM (a 64x128 state): scalar FMAs measured 9 % faster there, issue slots are not short
    autotune_min_work: int = 1 << 28   # B*T*H*M*N below which the planned tiles are used untimed
    autotune: int = 1        # time alternative forward tiles on the first call and keep the fastest
    fw_variant: int = -1     # >= 0: use this member of forward_variants(plan) untimed (tests, reproducible runs)
    bw_variant: int = -1     # >= 0: use this member of backward_variants(plan) untimed
    bw_split: int = 1        # generic backward: evaluate the part of a step that needs only the post-step state while the
                             # registers still hold it (from the step handled before) instead of recomputing that state
    bw_unroll_seg: int = 1   # generic backward: 1 = the steps of a segment (and their re-steps) form one straight-line
                             # block (measured: Gated Delta 7 %, Mamba-2 4 % faster), 2 = the whole chunk does
    bw_tmem: int = 1         # generic backward: keep the segment bases in Tensor Memory when they fit (more slots than
                             # shared memory holds, hence fewer recomputed steps); needs helper warps
    bw_tmem_slots: int = 0   # set by the planner: slots kept in Tensor Memory (0 = shared-memory slots)
    fw_acc: int = 2          # independent accumulators per kept element of a sum, forward kernel (measured: 2 is 3-6 %
                             # faster than 4 or 1 on the forward, 1 is 3 % faster than 2 or 4 on the backward)
    bw_acc: int = 1          # the same, backward kernel
    bounds: int = 0          # 1 = checked build of both kernels: every access is tested against the extents of the
                             # kernel's buffers, one outside is skipped and reported through the error word (debugging)
    use_tma: bool = True


SMEM_LIMIT = 227 * 1024
B200_SMS = 148      # used only when planning without a device (meta tensors, dry runs); else read from the device


def sm_count(device) -> int:
    """Streaming multiprocessors of ``device`` (a CUDA device), else a B200's."""
    if getattr(device, "type", None) == "cuda" and th.cuda.is_available():
        return th.cuda.get_device_properties(device).multi_processor_count
    return B200_SMS


class _GuardedBuffers:
    """Debugging allocator (environment ``FRNN_GUARD=1``): every buffer a kernel
    writes (outputs, final states, checkpoints, saved row sums, gradients) is
    carved out of a larger allocation with a band of a fixed byte pattern on
    either side, and ``check`` (after the launch has finished) raises if a band
    was touched: a store that left its buffer by up to ``BAND`` bytes shows up
    here instead of silently corrupting a neighbouring tensor."""
    BAND = 4096
    FILL = 0xA5

    def __init__(self):
        self.live: List[Tuple[str, th.Tensor, int]] = []

    def empty(self, what, shape, stride, dtype, device, zero=False):
        esize = th.empty((), dtype=dtype).element_size()
        extent = 0 if any(n == 0 for n in shape) else 1 + sum((n - 1) * s for n, s in zip(shape, stride))
        nbytes = extent * esize
        raw = th.full((2 * self.BAND + (nbytes + 255) // 256 * 256,), self.FILL, dtype=th.uint8, device=device)
        body = raw[self.BAND:self.BAND + nbytes].view(dtype)
        if zero:
            body.zero_()
        self.live.append((what, raw, nbytes))
        return body.as_strided(tuple(shape), tuple(stride))

    def check(self):
        live, self.live = self.live, []
        for what, raw, nbytes in live:
            lo, hi = raw[:self.BAND], raw[self.BAND + nbytes:]
            bad = int((lo != self.FILL).sum()) + int((hi != self.FILL).sum())
            if bad:
                side = "before" if int((lo != self.FILL).sum()) else "after"
                raise RuntimeError(f"flex_rnn_b200: a kernel wrote {bad} byte(s) outside {what} ({side} the buffer)")


class _DeviceStatus:
    """The error word the kernels of one device report through.  It lives in pinned host memory, which the
    device reaches directly (unified addressing): a kernel writes it only when one of its bounded waits ran out,
    and the host looks at it before the next launch, so the report costs the hot path neither a copy nor a
    synchronisation (a device-to-host copy per launch would queue behind a caller's own large transfers)."""

    def __init__(self, device):
        self.device = device
        self.word = th.zeros(1, dtype=th.int32).pin_memory()

    def check(self):
        """Raise if a kernel launched earlier on this device reported a timed-out wait; clears the word."""
        from . import runtime
        runtime.status_check(self.word.data_ptr(), 0, 0)

    def check_now(self, stream: int):
        """Wait for ``stream`` and check."""
        th.cuda.current_stream(self.device).synchronize()
        self.check()


_status: Dict[int, _DeviceStatus] = {}


def device_status(device) -> _DeviceStatus:
    """Status words of a CUDA device (created on first use)."""
    device = th.device(device)
    idx = device.index if device.index is not None else th.cuda.current_device()
    if idx not in _status:
        _status[idx] = _DeviceStatus(th.device("cuda", idx))
    return _status[idx]


def _bw_smem_limit(tu) -> int:
    """Dynamic shared memory a backward CTA may use: all of an SM's, or its share when several CTAs are to be
    resident (228 KB per SM, 1 KB reserved per CTA)."""
    return SMEM_LIMIT if tu.bw_min_blocks <= 1 else (228 * 1024) // tu.bw_min_blocks - 1024


def default_tuning(B, T, H, M, N, nstates) -> Tuning:
    tu = Tuning()
    for k, v in os.environ.items():
        if k.startswith("FRNN_TUNE_"):
            f = k[len("FRNN_TUNE_"):].lower()
            if hasattr(tu, f):
                setattr(tu, f, type(getattr(tu, f))(int(v)))
    slot = M * N * 4 * nstates
    # checkpoint chunk = seg * nslots steps, bounded by T and by shared memory for the slots
    while tu.nslots > 1 and max(tu.nslots, 2) * slot > 160 * 1024:
        tu.nslots -= 1
    while tu.seg * tu.nslots > T and tu.nslots > 1:
        tu.nslots -= 1
    while tu.seg * tu.nslots > T and tu.seg > 1:
        tu.seg -= 1
    tu.fw_stage = max(1, min(tu.fw_stage, T))
    tu.rev_stage = max(1, min(tu.rev_stage, T))
    return tu


# -- the planner -----------------------------------------------------------------

@dataclass
class Plan:
    problem: Problem
    joint: StepGraph
    g_fw: StepGraph
    g_re: StepGraph
    g_bw: StepGraph
    aux: List[str]
    n_out: int
    n_st: int
    grads: List[GradOut]
    tuning: Tuning
    fw_tile: lower.Tile
    bw_tile: lower.Tile
    D: int                  # checkpoint interval (timesteps)
    nck: int                # checkpoints stored per (b,h)
    k_fwd: int
    k_joint: int
    reverse: Optional[lower.Reverse] = None
    post_split: bool = False      # generic backward reads the post-step state from the registers (see lower.emit_backward)
    bw_choice: Tuple[int, int, int] = (4, 1, 2)   # (seg or reverse stage, kflush, ring buffers) that fit shared memory


def _spec(t: th.Tensor) -> TensorSpec:
    ptr_ok = True
    fake = isinstance(t, th._subclasses.fake_tensor.FakeTensor)      # shape propagation only: no address
    if t.device.type != "meta" and not fake:
        try:
            ptr_ok = t.data_ptr() % 16 == 0
        except RuntimeError:
            ptr_ok = True
    return TensorSpec(tuple(t.shape), tuple(t.stride()), _DT[t.dtype], ptr_ok)


def make_plan(step: Callable, inputs: Sequence[th.Tensor], state: Sequence[th.Tensor],
              tuning: Optional[Tuning] = None) -> Tuple[Plan, tuple, tuple]:
    inputs, state = tuple(inputs), tuple(state)
    assert len(state) >= 1, "a step function needs at least one state"
    assert not any(0 in s.shape[-2:] for s in state), f"a state needs at least one row and one column, got {list(state[0].shape)}"
    B, T, H = [max(i.shape[j] for i in inputs) for j in range(3)] if inputs else (state[0].shape[0], 1, state[0].shape[1])
    M = max(i.shape[-2] for i in inputs + state)
    N = max(i.shape[-1] for i in inputs + state)
    full = [B, T, H, M, N]
    for i, x in enumerate(inputs):
        assert x.ndim == 5, f"invalid shape {list(x.shape)} of argument #{i + 1}"
        for j in range(5):
            assert x.shape[j] in (1, full[j]), f"shape {list(x.shape)} of argument #{i + 1} is incompatible with {full}"
        assert 1 in x.shape[-2:] or x.shape[1] == 1, (
            f"shape {list(x.shape)} of argument #{i + 1} is both a matrix for each head, and depends on time. This is not supported")
        assert x.dtype in _IO_DTYPES, f"unsupported dtype {x.dtype} of argument #{i + 1}"
    for i, x in enumerate(state):
        assert list(x.shape) == [B, H, M, N], f"shape {list(x.shape)} of argument #{i + 1 + len(inputs)} != {[B, H, M, N]}"
        assert x.dtype in _IO_DTYPES, f"unsupported dtype {x.dtype} of argument #{i + 1 + len(inputs)}"
    nin, nst = len(inputs), len(state)

    # output arity and dtypes: run the step on meta tensors of the original dtypes
    in_desc = [(tuple(x.shape[-2:]), x.dtype) for x in inputs]
    st_desc = [(tuple(x.shape), x.dtype) for x in state]

    def probe_step():
        metas = [th.empty(B, H, *s, dtype=d, device="meta") for s, d in in_desc] + \
                [th.empty(s, dtype=d, device="meta") for s, d in st_desc]
        y, s = step(*metas)
        return ([(tuple(o.shape), o.dtype) for o in as_tuple(y)], [(tuple(o.shape), o.dtype) for o in as_tuple(s)])

    y_t, s_t = run_isolated(probe_step)
    assert len(s_t) == nst, f"step returns {len(s_t)} states but was given {nst}"
    assert all(a[0] == (B, H, M, N) for a in s_t), "new states must have the shape of the states"
    assert all(list(o[0]) == [B, H, M, 1] for o in y_t), [o[0] for o in y_t]
    assert all(o[1] in _IO_DTYPES for o in y_t)
    nout = len(y_t)
    out_dtypes = [o[1] for o in y_t]

    in_cls = [(int(x.shape[3] > 1), int(x.shape[4] > 1)) for x in inputs]
    st_cls = (int(M > 1), int(N > 1))
    joint, no2, ns2 = trace_joint(step, in_cls + [st_cls] * nst, nin, has_m=M > 1, has_n=N > 1, dims=(M, N))
    assert (no2, ns2) == (nout, nst)
    jin = joint.inputs
    in_names, st_names = jin[:nin], jin[nin:nin + nst]
    dy_names, dnext_names = jin[nin + nst:nin + nst + nout], jin[nin + nst + nout:]
    jout = joint.outputs
    y_names, ns_names = jout[:nout], jout[nout:nout + nst]
    dx_names, ds_names = jout[nout + nst:nout + nst + nin], jout[nout + nst + nin:]

    # forward must not depend on the cotangents
    cot = joint.depends_on(dy_names + dnext_names)
    g_fw0 = joint.pruned(y_names + ns_names, "step")
    assert not any(n.name in cot for n in g_fw0.nodes)
    # aux: forward row sums of [M,N] operands that the backward (or the re-step) reads
    cands = [n.name for n in joint.nodes
             if n.op == "sum" and n.over_n and not n.over_m and joint.shape[n.args[0]] == MN and n.name not in cot]
    probe = joint.pruned(ns_names + dx_names + ds_names, "probe", leaves=cands)
    aux = [c for c in cands if c in probe.inputs]
    g_fw = joint.pruned(y_names + ns_names + aux, "step")
    g_fw.inputs = jin[:nin + nst]
    g_re = joint.pruned(ns_names, "restep", leaves=aux)
    g_bw = joint.pruned(dx_names + ds_names, "dstep", leaves=aux)
    for n in g_fw.nodes:
        if n.op == "sum" and n.over_m:
            raise AssertionError("Only torch.sum(x, dim=-1, keepdim=True) is supported")

    tu = tuning or default_tuning(B, T, H, M, N, nst)
    n_sm = sm_count(inputs[0].device if inputs else state[0].device)
    # register budget: every state (and, in the backward, its gradient) and every matrix-per-head input
    # (and its gradient) is an R x C tile per thread
    n_mat = sum(1 for c in in_cls if c == MN)
    fw_tiles, bw_tiles = nst + n_mat, 2 * nst + 2 * n_mat
    fr, fc, br, bc = tu.fw_r, tu.fw_c, tu.bw_r, tu.bw_c
    while fr * fc * fw_tiles > 160 and fr * fc > 4:
        fr, fc = (fr // 2, fc) if fr >= 4 else (fr, max(1, fc // 2))
    while br * bc * bw_tiles > 160 and br * bc > 4:
        br, bc = (br // 2, bc) if br >= bc else (br, max(1, bc // 2))
    def fitted_tile(want_r, want_c, want_mb, n_tiles, extra_threads):
        """The tile nearest to the wish whose CTA fits an SM's register file: a row needs at least N/32 columns
        per thread, so wide states get fewer rows per thread, and a CTA whose threads' tiles (plus about 96
        working registers each) exceed the 64 K registers gives rows to further CTAs.  Rows are independent
        recurrences; only the gradients summed over rows couple them (accumulated across CTAs, see below)."""
        t = choose_tile(M, N, want_r, want_c, want_mb)
        while t.R * t.C * n_tiles > 160 and t.R > 1:
            t2 = choose_tile(M, N, t.R // 2, want_c, want_mb)
            if t2.R >= t.R:          # fewer rows per thread would need more than 1024 threads at this row count
                break
            t = t2
        mb = t.MB
        while mb % 2 == 0 and mb // 2 >= t.R:
            limit = min(1024 - extra_threads, 65536 // (t.R * t.C * n_tiles + 96) // 32 * 32)
            if t.NT <= max(32, limit):
                break
            try:
                t2 = choose_tile(M, N, t.R, want_c, mb // 2)
            except lower.LoweringError:
                break
            if t2.MB >= mb:
                break
            mb, t = t2.MB, t2
        return t

    fw_tile = fitted_tile(fr, fc, tu.fw_mb, fw_tiles, 0)
    if fw_tile.NT < 128 and fc >= 32:
        # a forward CTA of fewer than four warps leaves schedulers with a single warp: halve the columns per
        # thread instead (Mamba-2's 64x128 state: R4xC16, 128 threads, measured 4 % faster than R4xC32)
        fw_tile = fitted_tile(fr, fc // 2, tu.fw_mb, fw_tiles, 0)
    bw_tile = fitted_tile(br, bc, tu.bw_mb or None, bw_tiles, 128 if tu.bw_helper else 0)
    rows_split = bw_tile.MB < M
    # additive state update S' = S +/- X with X free of the state (given the saved row sums):
    # the backward can step the state backwards instead of recomputing it from checkpoints
    reverse = None
    if tu.reverse:
        dep = g_re.depends_on(st_names)
        prod = g_re.node_map()
        incs, signs = [], []
        for k, nm in enumerate(ns_names):
            n = prod.get(nm)
            if n is None or n.op not in ("add", "sub") or len(n.args) != 2:
                break
            a, b = n.args
            if a == st_names[k] and isinstance(b, str) and b not in dep and b not in st_names:
                incs.append(b)
                signs.append(1 if n.op == "add" else -1)
            elif n.op == "add" and b == st_names[k] and isinstance(a, str) and a not in dep and a not in st_names:
                incs.append(a)
                signs.append(1)
            else:
                break
        if len(incs) == nst:
            g_x = joint.pruned(incs, "unstep", leaves=aux)
            reverse = lower.Reverse(g_x, signs, max(1, tu.rev_resync))
    dy_names, dnext_names = list(dy_names), list(dnext_names)
    prob = Problem(B, T, H, M, N, [_spec(x) for x in inputs], list(in_names), [_spec(s) for s in state],
                   list(st_names), [_DT[d] for d in out_dtypes], len(aux))
    dx_meta = tuple(th.empty_like(x, device="meta") for x in inputs)

    def make_grads(rows_split: bool) -> List[GradOut]:
        """Where each input's gradient goes: its own dtype and layout, or fp32 with atomic accumulation when
        several CTAs or timesteps add to the same element (inputs broadcast over B, T or H; gradients summed
        over rows when the rows of a head are split over CTAs)."""
        out = []
        for i, x in enumerate(inputs):
            cls = in_cls[i]
            atomic = list(x.shape[:3]) != [B, T, H] or (rows_split and cls in (N1, S11))
            over_t = x.shape[1] == 1 and T > 1
            gm = dx_meta[i]
            if atomic:
                spec = TensorSpec(tuple(gm.shape), tuple(th.empty(gm.shape, device="meta").stride()), DT_F32, True)
            else:
                spec = TensorSpec(tuple(gm.shape), tuple(gm.stride()), _DT[gm.dtype], True)
            out.append(GradOut(i, cls, spec, dx_names[i], over_t, atomic))
        return out

    grads = make_grads(rows_split)

    # pick the backward's staging / flush parameters that fit shared memory
    choice = None
    import dataclasses
    tu = dataclasses.replace(tu)
    auto_blocks = tu.bw_min_blocks <= 0
    if auto_blocks:
        # a (b,h) state small enough for a CTA of four warps leaves room for a second CTA on the SM
        # (Mamba-2 64x128: 7 % faster backward than one CTA of eight warps)
        tu.bw_min_blocks = 2 if bw_tile.NT <= 128 and B * H * (M // bw_tile.MB) > n_sm else 1

    def flush_options(helper: int):
        ks, k = [], max(1, tu.kflush)
        while k >= 1:
            ks.append(k)
            k //= 2
        if helper:
            # a second ring half lets the compute warps go on while the helpers flush: worth more than a longer group
            return [(k, 2) for k in ks] + [(k, 1) for k in ks]
        return [(k, b) for k in ks for b in (2, 1)]

    post_split = bool(tu.bw_split) and reverse is None and lower.can_split_post(g_re, g_bw, list(st_names))

    def fits(sg, nsl, kflush, bufs, helper, tmem=0):
        try:
            ks = emit_backward(prob, g_re, g_bw, aux, nout, grads, dy_names, dnext_names, bw_tile, sg, nsl,
                               tu.use_tma, "", kflush=kflush, ring_bufs=bufs, reverse=reverse, helper_warps=helper,
                               min_blocks=max(1, tu.bw_min_blocks), tmem_slots=tmem, post_split=post_split)
        except lower.LoweringError:
            if tmem:
                return False
            raise
        return ks.smem_bytes <= _bw_smem_limit(tu)

    def fit():
        """((steps per segment or staged chunk, flush group, ring buffers), slots, helper warps) that fit
        shared memory, preferring helper warps as long as they do not cost recomputation."""
        helpers = [1, 0] if tu.bw_helper else [0]
        tu.bw_tmem_slots = 0
        if reverse is None and tu.bw_helper and tu.bw_tmem and T >= 8:
            # segment bases in Tensor Memory: as many slots as fit, one step fewer to recompute per slot more
            for nsl in (8, 4):
                for kflush, bufs in flush_options(1):
                    if fits(8 // nsl, nsl, kflush, bufs, 1, tmem=nsl):
                        tu.bw_tmem_slots = nsl
                        return (8 // nsl, kflush, bufs), nsl, 1
        if reverse is not None:
            for helper in helpers:
                # with helper warps a chunk boundary is cheap: prefer a long flush group over a long staged chunk
                stages = [s for s in (16, 8, 4) if s <= tu.rev_stage] if helper else list(range(tu.rev_stage, 0, -1))
                # ... and a staged chunk that is exactly one flush group first (one straight-line block of steps per
                # chunk: measured 6 % faster than two groups per chunk for the Delta Rule)
                order = [(sg, fl) for fl in flush_options(helper) for sg in sorted(stages, key=lambda s: (s != fl[0], -s))] \
                    if helper else [(sg, fl) for sg in stages for fl in flush_options(helper)]
                for sg, (kflush, bufs) in order:
                    if fits(sg, tu.nslots, kflush, bufs, helper):
                        return (sg, kflush, bufs), tu.nslots, helper
            return None, tu.nslots, 0
        # (steps per segment, slots): fewer recomputed steps first, then what the tuning asks for
        pairs = ([(2, 4)] if tu.slot_search and T >= 8 else []) + [(sg, tu.nslots) for sg in range(tu.seg, 0, -1)]
        if tu.nslots > 1:
            pairs += [(sg, 1) for sg in range(tu.seg, 0, -1)]
        for sg, nsl in pairs:
            for helper in helpers:
                for kflush, bufs in flush_options(helper):
                    if fits(sg, nsl, kflush, bufs, helper):
                        return (sg, kflush, bufs), nsl, helper
        return None, tu.nslots, 0

    while choice is None:
        choice, nsl, helper = fit()
        if choice is not None:
            tu.bw_helper, tu.nslots = helper, nsl
            break
        if auto_blocks and tu.bw_min_blocks > 1:
            tu.bw_min_blocks = 1          # half an SM's shared memory is not enough: one CTA per SM after all
            continue
        # fewer rows per CTA: smaller slots and fewer row groups in the ring of gradient partials
        try:
            smaller = choose_tile(M, N, bw_tile.R, bw_tile.C, bw_tile.MB // 2) if bw_tile.MB % 2 == 0 else None
        except lower.LoweringError:
            smaller = None
        if smaller is None or smaller.MB >= bw_tile.MB or smaller.NT < 32:
            break
        bw_tile = smaller
        grads = make_grads(True)
    if reverse is not None and choice is not None and tu.bw_helper:
        reverse.resync = max(1, tu.rev_ckpt // choice[0])
    if choice is None:
        raise lower.LoweringError(f"the backward kernel of a {M}x{N} state does not fit shared memory")
    if reverse is not None:
        D = choice[0] * reverse.resync
        nck = (T + D - 1) // D + 1          # plus the final state
    else:
        D = choice[0] * tu.nslots
        nck = (T + D - 1) // D + (1 if post_split else 0)     # plus the final state

    dev = inputs[0].device if inputs else state[0].device
    # declared outputs (what the fake implementations materialise)
    out_meta = tuple(th.empty(B, T, H, M, dtype=d, device="meta") for d in out_dtypes)
    stT_meta = tuple(th.empty_like(s, device="meta") for s in state)
    store_meta = tuple(th.empty(B, H, nck, M, N, dtype=th.float32, device="meta") for _ in state)
    aux_meta = (th.empty(len(aux), B, H, T, M, dtype=th.float32, device="meta"),)
    fw_meta = get_meta([*out_meta, *stT_meta, *store_meta, *aux_meta])
    bw_meta = get_meta([*dx_meta, *stT_meta])

    plan = Plan(prob, joint, g_fw, g_re, g_bw, aux, nout, nst, grads, tu, fw_tile, bw_tile, D, nck,
                g_fw0.count_mn_ops(), joint.pruned(jout, "all").count_mn_ops(), reverse, post_split, choice)
    plan.dy_names, plan.dnext_names = dy_names, dnext_names   # type: ignore[attr-defined]
    plan.n_sm = n_sm                                            # type: ignore[attr-defined]
    return plan, fw_meta, bw_meta


def generate_forward(plan: Plan, tile: Optional[lower.Tile] = None, pack: Optional[bool] = None,
                     stage: Optional[int] = None, unroll: Optional[int] = None) -> lower.KernelSource:
    """Emit the forward kernel.  The optional arguments replace the plan's
    choices: the tile, packed arithmetic on or off, timesteps staged per chunk
    and the unroll factor of the step loop."""
    p, tu = plan.problem, plan.tuning
    pack2 = bool(tu.pack2 & 2) if pack is None else bool(pack)
    tile = tile or plan.fw_tile
    # keep the per-CTA shared memory small enough for all CTAs of an SM to be resident
    stage = max(1, min(stage or tu.fw_stage, p.T))
    if unroll is None:
        # bound the code size of the unrolled step loop: about 0.55 instructions of 16 bytes per counted [M,N]
        # operation and tile element, plus the per-step overhead (larger bodies measured no faster)
        step_bytes = 16 * (0.55 * plan.k_fwd * tile.R * tile.C * (0.6 if pack2 else 1.0) + 120)
        unroll = tu.fw_unroll
        while unroll > 1 and unroll * step_bytes > 40 * 1024:
            unroll //= 2
    while True:
        fw = emit_forward(p, plan.g_fw, plan.aux, plan.n_out, tile, stage, plan.D, tu.use_tma,
                          tu.fw_min_blocks, prelude(), final_ckpt=plan.reverse is not None or plan.post_split,
                          step_unroll=unroll or tu.fw_unroll, pack2=pack2, col_major=bool(tu.col_major),
                          max_acc=tu.fw_acc)
        ncta = fw.grid[0] * fw.grid[1] * fw.grid[2]
        # CTAs an SM will hold at once: as many as there are per SM, but no more than the register file admits
        # (the state tiles plus about 96 registers of vectors and addresses per thread, unless the launch bounds
        # ask for more CTAs and accept the spills)
        by_regs = 65536 // (fw.block * min(255, tile.R * tile.C * plan.n_st + 96))
        per_sm = min(max(1, -(-ncta // getattr(plan, "n_sm", B200_SMS))), 2048 // fw.block, 32,
                     max(1, by_regs, tu.fw_min_blocks))
        if stage <= 4 or fw.smem_bytes * per_sm <= 200 * 1024:
            break
        stage //= 2
    if fw.smem_bytes > SMEM_LIMIT:
        raise lower.LoweringError(f"kernel {fw.name} needs {fw.smem_bytes} bytes of shared memory (limit {SMEM_LIMIT})")
    return _checked(fw, tu)


def _checked(ks: lower.KernelSource, tu: Tuning) -> lower.KernelSource:
    """The checked build of a kernel when ``Tuning.bounds`` asks for it."""
    if not tu.bounds:
        return ks
    import dataclasses
    return dataclasses.replace(ks, source="#define FRNN_BOUNDS 1\n" + ks.source, info={**ks.info, "bounds": True})


def forward_tile_candidates(plan: Plan) -> List[lower.Tile]:
    """Alternative forward tilings worth timing (the planned one first)."""
    p = plan.problem
    out, seen = [plan.fw_tile], {(plan.fw_tile.R, plan.fw_tile.C, plan.fw_tile.MB)}
    for r, c in ((2, 64), (4, 32), (8, 16), (2, 32), (4, 16)):
        try:
            t = choose_tile(p.M, p.N, r, c, plan.tuning.fw_mb)
        except lower.LoweringError:
            continue
        if (t.R, t.C, t.MB) not in seen and t.R * t.C * plan.n_st <= 128:
            seen.add((t.R, t.C, t.MB))
            out.append(t)
    return out


def forward_variants(plan: Plan) -> List[dict]:
    """Keyword arguments of ``generate_forward`` for every forward kernel the
    autotuner may pick; member 0 is the planned kernel."""
    default_pack = bool(plan.tuning.pack2 & 2)
    out = [dict(tile=t, pack=default_pack, stage=None, unroll=None) for t in forward_tile_candidates(plan)]
    out.append(dict(tile=plan.fw_tile, pack=not default_pack, stage=None, unroll=None))
    out.append(dict(tile=plan.fw_tile, pack=default_pack, stage=None, unroll=1))
    if 2 * plan.tuning.fw_stage <= plan.problem.T:
        # twice the timesteps per staged chunk: half the block barriers and conversions per step
        out.append(dict(tile=plan.fw_tile, pack=default_pack, stage=2 * plan.tuning.fw_stage, unroll=None))
    if plan.reverse is None and plan.D <= 16:
        # one chunk per checkpoint interval, step loop fully unrolled
        out.append(dict(tile=plan.fw_tile, pack=default_pack, stage=plan.D, unroll=plan.D))
    return out


def backward_variants(plan: Plan) -> List[dict]:
    """Keyword arguments of ``generate_backward`` for every backward kernel the
    autotuner may pick; member 0 is the planned kernel."""
    out = [dict(tile=t) for t in backward_tile_candidates(plan)]
    # the planned tile with the other kind of arithmetic (scalar FMAs measured 9 % faster than packed ones on
    # Mamba-2's 64x128 state, 8-24 % slower on the 128x128 workloads)
    out.append(dict(tile=plan.bw_tile, pack=not _bw_packed(plan, plan.bw_tile)))
    return out


def _bw_packed(plan: Plan, tile: lower.Tile) -> bool:
    """Whether a backward kernel with this tile uses packed two-column arithmetic by default."""
    tu = plan.tuning
    two_small_ctas = tile.NT <= 128 and tu.bw_min_blocks >= 2
    return bool(tu.pack2 & 1) and (not two_small_ctas or bool(tu.bw_pack_small))


def generate_backward(plan: Plan, tile: Optional[lower.Tile] = None,
                      pack: Optional[bool] = None) -> Optional[lower.KernelSource]:
    """Emit the backward kernel.  For a ``tile`` other than the planned one the
    checkpoint interval and slot count stay what the forward was built for and
    only the flush parameters are re-fitted; None if it does not fit.  ``pack``
    switches the packed two-column arithmetic on or off (default: the plan's)."""
    p, tu = plan.problem, plan.tuning
    pack2 = _bw_packed(plan, tile or plan.bw_tile) if pack is None else bool(pack)
    sg, kflush, bufs = plan.bw_choice
    cands = [(kflush, bufs)]
    if tile is not None and tile is not plan.bw_tile:
        k = max(1, tu.kflush)
        cands = []
        while k >= 1:
            cands += [(k, 2), (k, 1)]
            k //= 2
    for kf, nb in cands:
        bw = emit_backward(p, plan.g_re, plan.g_bw, plan.aux, plan.n_out, plan.grads, plan.dy_names,   # type: ignore[attr-defined]
                           plan.dnext_names, tile or plan.bw_tile, sg, tu.nslots, tu.use_tma, prelude(),  # type: ignore[attr-defined]
                           kflush=kf, ring_bufs=nb, reverse=plan.reverse, step_unroll=tu.bw_unroll,
                           min_blocks=max(1, tu.bw_min_blocks), pack2=pack2, col_major=bool(tu.col_major),
                           helper_warps=tu.bw_helper, max_acc=tu.bw_acc, tmem_slots=tu.bw_tmem_slots,
                           post_split=plan.post_split, unroll_segment=int(tu.bw_unroll_seg))
        if bw.smem_bytes <= _bw_smem_limit(tu):
            return _checked(bw, tu)
    return None


def backward_tile_candidates(plan: Plan) -> List[lower.Tile]:
    p = plan.problem
    out, seen = [plan.bw_tile], {(plan.bw_tile.R, plan.bw_tile.C)}
    n_tiles = 2 * plan.n_st + 2 * sum(1 for g in plan.grads if g.cls == MN)
    for r, c in ((8, 8), (4, 8), (4, 16), (8, 4)):
        try:
            t = choose_tile(p.M, p.N, r, c, plan.bw_tile.MB if plan.bw_tile.MB < p.M else None)
        except lower.LoweringError:
            continue
        if (t.R, t.C) not in seen and t.R * t.C * n_tiles <= 160:
            seen.add((t.R, t.C))
            out.append(t)
    return out


def generate(plan: Plan) -> Tuple[lower.KernelSource, lower.KernelSource]:
    """Emit the CUDA source of the forward and the backward kernel."""
    fw = generate_forward(plan)
    bw = generate_backward(plan)
    if bw is None:
        raise lower.LoweringError("the backward kernel does not fit shared memory")
    return fw, bw


class _CudaLauncher:
    """Compiles a generated kernel with NVRTC and launches it through the
    C-ABI library on the current stream of the tensors' device."""

    def __init__(self, ks: lower.KernelSource):
        from . import runtime
        self.rt, self.ks = runtime, ks
        self.mods: Dict[int, object] = {}
        self.log = ""
        self._maps: Dict[tuple, object] = {}     # (device, map name, base address) -> encoded tensor map

    def _tensor_maps(self, ptrs, idx):
        """Tensor maps of this launch (they embed the tensors' base addresses)."""
        out = []
        for tm in self.ks.tmaps:
            base = int(ptrs[tm["src_index"]]) + tm["off_bytes"]
            key = (idx, tm["name"], base)
            arg = self._maps.get(key)
            if arg is None:
                if len(self._maps) > 256:
                    self._maps.clear()
                arg = self.rt.encode_tensor_map(base, tm["elt"], tm["dims"], tm["strides_bytes"], tm["box"])
                self._maps[key] = arg
            out.append(arg)
        return out

    def __call__(self, ptrs, device: th.device):
        idx = device.index if device.index is not None else th.cuda.current_device()
        with th.cuda.device(idx):
            if idx not in self.mods:
                cubin, self.log = self.rt.compile_cubin(self.ks.source)
                self.mods[idx] = self.rt.Module(cubin, [self.ks.name], [self.ks.smem_bytes])
            ptrs = list(ptrs) + self._tensor_maps(ptrs, idx)
            self.mods[idx].launch(0, self.ks.grid, self.ks.block, self.ks.smem_bytes,
                                  th.cuda.current_stream(idx).cuda_stream, ptrs)


class _device_ctx:
    def __init__(self, device):
        self.ctx = th.cuda.device(device) if device.type == "cuda" else None

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)


def _padded_rows(inputs, state) -> Optional[int]:
    """Row count a state too small for one warp is padded to, else None.

    A CTA is at least one warp; a row is spread over at most 32 lanes (a power
    of two dividing N), so M x lanes must be a multiple of 32."""
    M = max(i.shape[-2] for i in tuple(inputs) + tuple(state))
    N = max(i.shape[-1] for i in tuple(inputs) + tuple(state))
    if any(0 in s.shape[-2:] for s in state):
        return None                  # refused with a message by make_plan
    lanes = max(L for L in (1, 2, 4, 8, 16, 32) if N % L == 0)
    k = 1
    while (M * k * lanes) % 32:
        k += 1
    return None if k == 1 else M * k


def _build_row_padded(step, inputs, state, Mp, dryrun, tuning, _launcher):
    """build_twopass for a state with fewer elements than one warp has threads
    (the 1x1 gate recurrence of an mLSTM, say).

    The recurrence is run on ``Mp`` rows: the real rows, repeated.  Repeated rows
    compute the same finite values as the rows they copy; their upstream
    gradients are zero, so they add nothing to the gradients summed over rows,
    and their outputs and state rows are dropped.  The copies this costs are of
    the small tensors that carry a row dimension."""
    inputs, state = tuple(inputs), tuple(state)
    M = max(i.shape[-2] for i in inputs + state)

    def rep(x, dim):
        if x.shape[dim] == 1 and M > 1:
            return x                      # broadcast over rows already
        if x.device.type == "meta" or dryrun:
            shape = list(x.shape)
            shape[dim] = Mp
            return th.empty(shape, dtype=x.dtype, device=x.device)
        return x.index_select(dim, th.arange(Mp, device=x.device) % x.shape[dim])

    # an input without a row dimension stays as it is (M == 1: every input is one, the state alone is padded)
    def pad_inputs(xs):
        return tuple(x if x.shape[-2] == 1 else rep(x, -2) for x in xs)

    def pad_state(ss):
        return tuple(rep(s_, -2) for s_ in ss)

    inner = build_twopass(step, pad_inputs(inputs), pad_state(state), dryrun, tuning, _launcher)
    fw_meta_p, bw_meta_p = inner[-2:]
    nst, nin = len(state), len(inputs)
    nout = len(fw_meta_p) - 2 * nst - 1
    B, T, H = fw_meta_p[0][0][:3] if nout else (state[0].shape[0], max(i.shape[1] for i in inputs), state[0].shape[1])
    out_meta = tuple(th.empty(B, T, H, M, dtype=m[2], device="meta") for m in fw_meta_p[:nout])
    stT_meta = tuple(th.empty_like(s_, device="meta") for s_ in state)
    fw_meta = get_meta([*out_meta, *stT_meta]) + tuple(fw_meta_p[nout + nst:])
    dx_meta = tuple(th.empty_like(x, device="meta") for x in inputs)
    bw_meta = get_meta([*dx_meta, *stT_meta])
    if dryrun:
        return fw_meta, bw_meta
    fwd_p, bwd_p = inner[:2]
    in_meta = tuple(th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device="meta") for x in inputs)
    st_meta = tuple(th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device="meta") for x in state)

    def forward(inputs_, state0):
        verify_meta(inputs_, in_meta, "input Tensor metadata doesn't match compilation\n")
        verify_meta(state0, st_meta, "initial state Tensor metadata doesn't match compilation\n")
        res = fwd_p(pad_inputs(inputs_), pad_state(state0))
        outs = tuple(o[..., :M].contiguous() for o in res[:nout])
        stT = tuple(th.empty_like(s0).copy_(sp[:, :, :M]) for s0, sp in zip(state0, res[nout:nout + nst]))
        return (*outs, *stT, *res[nout + nst:])

    def backward(doutput, dstateT, inputs_, state_store, aux_):
        verify_meta(inputs_, in_meta)
        dout_p = tuple(th.nn.functional.pad(d, (0, Mp - M)) for d in doutput)
        dst_p = tuple(th.nn.functional.pad(d, (0, 0, 0, Mp - M)) for d in dstateT)
        dxs_p, ds0_p = bwd_p(dout_p, dst_p, pad_inputs(inputs_), state_store, aux_)
        dxs = tuple(dp if dp.shape == x.shape else th.empty_like(x).copy_(dp.narrow(-2, 0, x.shape[-2]))
                    for dp, x in zip(dxs_p, inputs_))
        ds0 = tuple(th.empty_strided(m.shape, m.stride(), dtype=m.dtype, device=dp.device).copy_(dp[:, :, :M])
                    for m, dp in zip(stT_meta, ds0_p))
        return dxs, ds0

    for name in ("plan", "sources", "launchers", "kernel_status", "tuned"):
        setattr(forward, name, getattr(fwd_p, name))
    forward.padded_rows = Mp                # type: ignore[attr-defined]
    return forward, backward, fw_meta, bw_meta


def _build_empty(plan: Plan, fw_meta, bw_meta, inputs, state):
    """Host closures for a problem without a single timestep, batch row or head:
    there is nothing to scan and no kernel to launch (a grid or a loop of extent
    zero is not something the generated kernels are built for).  Outputs are
    empty, the final state is the initial state (or empty), gradients of the
    inputs are zero and the gradient of the initial state is the upstream
    gradient of the final state."""
    in_meta = tuple(th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device="meta") for x in inputs)
    st_meta = tuple(th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device="meta") for x in state)

    def like(meta, device):
        shape, stride, dtype = meta
        return th.empty_strided(tuple(shape), tuple(stride), dtype=dtype, device=device).zero_()

    def forward(inputs_, state0):
        verify_meta(inputs_, in_meta, "input Tensor metadata doesn't match compilation\n")
        verify_meta(state0, st_meta, "initial state Tensor metadata doesn't match compilation\n")
        device = state0[0].device
        res = [like(m, device) for m in fw_meta]
        for k, s in enumerate(state0):
            res[plan.n_out + k].copy_(s)
        return tuple(res)

    def backward(doutput, dstateT, inputs_, state_store, aux_):
        device = dstateT[0].device
        nin = len(in_meta)
        dxs = tuple(like(m, device) for m in bw_meta[:nin])
        ds0 = tuple(like(m, device).copy_(d) for m, d in zip(bw_meta[nin:], dstateT))
        return dxs, ds0

    forward.plan = plan                      # type: ignore[attr-defined]
    forward.sources = ()                     # type: ignore[attr-defined]
    forward.launchers = ()                   # type: ignore[attr-defined]
    forward.kernel_status = lambda device=None: 0   # type: ignore[attr-defined]
    forward.tuned = {"fw_choice": 0, "bw_choice": 0, "fw_log": [], "bw_log": []}   # type: ignore[attr-defined]
    return forward, backward


def build_twopass(step, inputs, state, dryrun=False, tuning: Optional[Tuning] = None, _launcher=None):
    """See the module docstring.  With ``dryrun`` nothing touches CUDA.

    ``_launcher`` is a seam for the test-suite only: a factory
    ``KernelSource -> callable(ptrs, device)`` that stands in for the NVRTC +
    C-ABI launch (the tests inject a host emulation of the generated source to
    check it without a GPU).  Library code never passes it, and without it
    tensors that are not on a CUDA device are rejected.
    """
    Mp = _padded_rows(inputs, state)
    if Mp is not None:
        return _build_row_padded(step, inputs, state, Mp, dryrun, tuning, _launcher)
    plan, fw_meta, bw_meta = make_plan(step, inputs, state, tuning)
    if dryrun:
        return fw_meta, bw_meta

    inputs, state = tuple(inputs), tuple(state)
    dev = inputs[0].device if inputs else state[0].device
    if dev.type != "cuda" and _launcher is None:
        raise RuntimeError("flex_rnn_b200 runs on CUDA devices only (there is no CPU path); "
                           "use the .naive method for a CPU evaluation of the step function")
    if 0 in (plan.problem.B, plan.problem.T, plan.problem.H):
        return (*_build_empty(plan, fw_meta, bw_meta, inputs, state), fw_meta, bw_meta)
    fw_src, bw_src = generate(plan)
    tu0 = plan.tuning
    forced_fw, forced_bw = tu0.fw_variant >= 0, tu0.bw_variant >= 0
    if forced_fw and tu0.fw_variant > 0:
        fw_src = generate_forward(plan, **forward_variants(plan)[tu0.fw_variant])
    if forced_bw and tu0.bw_variant > 0:
        bw_src = generate_backward(plan, **backward_variants(plan)[tu0.bw_variant])
        if bw_src is None:
            raise lower.LoweringError("the requested backward variant does not fit shared memory")
    p = plan.problem
    nin, nst, nout = len(inputs), plan.n_st, plan.n_out
    make = _launcher or _CudaLauncher
    launch_fw, launch_bw = make(fw_src), make(bw_src)

    in_meta = tuple(th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device="meta") for x in inputs)
    st_meta = tuple(th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device="meta") for x in state)
    in_align = [x.data_ptr() % 16 == 0 for x in inputs]
    st_align = [x.data_ptr() % 16 == 0 for x in state]
    fw_used = plan.g_fw.used_inputs()
    bw_used = [a or b for a, b in zip(plan.g_re.used_inputs(), plan.g_bw.used_inputs())]
    emulated = _launcher is not None
    emu_words: Dict[str, th.Tensor] = {}

    def err_word(device):
        if emulated:          # the test seam runs on host tensors
            if "w" not in emu_words:
                emu_words["w"] = th.zeros(1, dtype=th.int32, device=device)
            return emu_words["w"]
        return device_status(device).word

    strict = os.environ.get("FRNN_CHECK", "0") not in ("", "0")
    guard = _GuardedBuffers() if os.environ.get("FRNN_GUARD", "0") not in ("", "0") else None

    def alloc(what, shape, stride, dtype, device, zero=False):
        """A buffer the kernels write; between guard bands with FRNN_GUARD=1."""
        if guard is not None:
            return guard.empty(what, shape, stride, dtype, device, zero)
        t = th.empty_strided(tuple(shape), tuple(stride), dtype=dtype, device=device)
        return t.zero_() if zero else t

    def alloc_like(what, like, device, dtype=None, zero=False):
        m = th.empty_like(like, device="meta") if dtype is None else th.empty(like.shape, dtype=dtype, device="meta")
        return alloc(what, m.shape, m.stride(), m.dtype, device, zero)

    def check_guard(device):
        """FRNN_GUARD=1: wait for the launch and look at the bands around everything it wrote."""
        if guard is not None:
            if not emulated:
                th.cuda.synchronize(device)
            guard.check()

    def check_before(device):
        """Raise if a kernel launched by an earlier call on this device reported
        a timed-out wait (its outputs were not valid).  No synchronisation."""
        if not emulated:
            device_status(device).check()

    def check_status(device, what):
        """With FRNN_CHECK=1: wait for the launch and raise now if it reported a timed-out wait (off by
        default, it serialises; by default the next call reports it)."""
        if strict and not emulated:
            device_status(device).check_now(th.cuda.current_stream(device).cuda_stream)

    def check_align(ts, flags, what):
        """What the generated index arithmetic relies on: the alignment seen at compilation, and that the
        last element the strides reach lies inside the tensor's storage."""
        for i, (t, f) in enumerate(zip(ts, flags)):
            assert (t.data_ptr() % 16 == 0) or not f, (
                f"{what} #{i + 1} was 16-byte aligned at compilation but is not now")
            reach = 1 + sum((n - 1) * s for n, s in zip(t.shape, t.stride()) if n > 1)
            have = t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()
            assert t.numel() == 0 or reach <= have, f"{what} #{i + 1}: its strides reach past the end of its storage"

    # timing alternative tilings costs a few NVRTC compilations: only worth it for work of benchmark size
    no_tune = (_launcher is not None or not plan.tuning.autotune
               or p.B * p.T * p.H * p.M * p.N < plan.tuning.autotune_min_work)
    tuned = {"fw": no_tune or forced_fw, "launch_fw": launch_fw, "fw_src": fw_src, "bw": no_tune or forced_bw,
             "launch_bw": launch_bw, "bw_src": bw_src,
             "fw_choice": max(0, tu0.fw_variant), "bw_choice": max(0, tu0.bw_variant), "fw_log": [], "bw_log": []}

    def timed(launcher, ptrs, device, reps=5):
        """Median device time of ``reps`` launches after two warm-up launches (the first also compiles, and the
        GPU's clocks have dropped while the compiler ran)."""
        launcher(ptrs, device)
        launcher(ptrs, device)
        ms = []
        for _ in range(reps):
            ev = [th.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            launcher(ptrs, device)
            ev[1].record()
            ev[1].synchronize()
            ms.append(ev[0].elapsed_time(ev[1]))
        return sorted(ms)[len(ms) // 2]

    def autotune_backward(ptrs, device, dxs, ds0):
        """Time the alternative backward kernels once, writing into throw-away
        gradient buffers (the kernel accumulates into some of its outputs)."""
        tuned["bw"] = True
        nouts = len(dxs) + len(ds0)
        first_out = len(ptrs) - 1 - nouts
        scratch = [th.zeros_like(t) for t in list(ds0) + list(dxs)]
        trial = list(ptrs[:first_out]) + [t.data_ptr() for t in scratch] + [ptrs[-1]]
        best, log = None, []
        for k, kw in enumerate(backward_variants(plan)):
            try:
                ks = bw_src if k == 0 else generate_backward(plan, **kw)
                if ks is None:
                    continue
                launcher = launch_bw if k == 0 else make(ks)
                ms = timed(launcher, trial, device)
            except (lower.LoweringError, RuntimeError):
                continue
            log.append((k, ks.info["tile"], bool(ks.info["packed"]), round(ms, 4)))
            if best is None or ms < best[0]:
                best = (ms, launcher, ks, k)
        if best is not None:
            tuned["launch_bw"], tuned["bw_src"] = best[1], best[2]
            tuned["bw_choice"], tuned["bw_log"] = best[3], log
            forward.sources = (tuned["fw_src"], best[2])       # type: ignore[attr-defined]

    def autotune_forward(ptrs, device):
        """Time the alternative forward kernels once on the real arguments (the
        forward kernel only writes its outputs) and keep the fastest."""
        tuned["fw"] = True
        best, log = None, []
        for k, kw in enumerate(forward_variants(plan)):
            try:
                ks = fw_src if k == 0 else generate_forward(plan, **kw)
                launcher = launch_fw if k == 0 else make(ks)
                ms = timed(launcher, ptrs, device)
            except (lower.LoweringError, RuntimeError):
                continue
            log.append((k, ks.info["tile"], bool(ks.info["packed"]), round(ms, 4)))
            if best is None or ms < best[0]:
                best = (ms, launcher, ks, k)
        if best is not None:
            tuned["launch_fw"], tuned["fw_src"] = best[1], best[2]
            tuned["fw_choice"], tuned["fw_log"] = best[3], log
            forward.sources = (best[2], tuned["bw_src"])       # type: ignore[attr-defined]

    def forward(inputs_, state0):
        verify_meta(inputs_, in_meta, "input Tensor metadata doesn't match compilation\n")
        verify_meta(state0, st_meta, "initial state Tensor metadata doesn't match compilation\n")
        check_align(inputs_, in_align, "input")
        check_align(state0, st_align, "initial state")
        device = inputs_[0].device
        with _device_ctx(device):
            check_before(device)
            cont = lambda *shape: (shape, lower._contig(shape))
            outs = tuple(alloc(f"output #{j + 1}", *cont(p.B, p.T, p.H, p.M), o[2], device)
                         for j, o in enumerate(fw_meta[:nout]))
            stT = tuple(alloc_like(f"final state #{k + 1}", s, device) for k, s in enumerate(state0))
            store = tuple(alloc(f"checkpoints of state #{k + 1}", *cont(p.B, p.H, plan.nck, p.M, p.N), th.float32, device)
                          for k, _ in enumerate(state0))
            aux = alloc("saved row sums", *cont(len(plan.aux), p.B, p.H, p.T, p.M), th.float32, device)
            ew = err_word(device)
            ptrs = [x.data_ptr() for x, u in zip(inputs_, fw_used[:nin]) if u]
            ptrs += [s.data_ptr() for s in state0] + [o.data_ptr() for o in outs] + [s.data_ptr() for s in stT]
            ptrs += [s.data_ptr() for s in store] + [aux.data_ptr(), ew.data_ptr()]
            if not tuned["fw"]:
                autotune_forward(ptrs, device)
            tuned["launch_fw"](ptrs, device)
            check_status(device, "forward")
            check_guard(device)
        return (*outs, *stT, *store, aux)

    def backward(doutput, dstateT, inputs_, state_store, aux_):
        doutput = tuple(d.contiguous() for d in doutput)
        dstateT = tuple(d.contiguous() for d in dstateT)
        verify_meta(inputs_, in_meta)
        check_align(inputs_, in_align, "input")
        aux = aux_[0] if isinstance(aux_, (tuple, list)) else aux_
        device = inputs_[0].device
        with _device_ctx(device):
            check_before(device)
            dxs = []
            for i, (go, x) in enumerate(zip(plan.grads, inputs_)):
                if go.atomic:
                    dxs.append(alloc_like(f"gradient of input #{i + 1}", x, device, dtype=th.float32, zero=True))
                else:
                    dxs.append(alloc_like(f"gradient of input #{i + 1}", x, device))
            ds0 = tuple(alloc_like(f"gradient of initial state #{k + 1}", s, device) for k, s in enumerate(st_meta))
            ew = err_word(device)
            ptrs = [x.data_ptr() for x, u in zip(inputs_, bw_used[:nin]) if u]
            ptrs += [d.data_ptr() for d in doutput] + [d.data_ptr() for d in dstateT]
            ptrs += [s.data_ptr() for s in state_store] + [aux.data_ptr()]
            ptrs += [d.data_ptr() for d in ds0] + [d.data_ptr() for d in dxs] + [ew.data_ptr()]
            if not tuned["bw"]:
                autotune_backward(ptrs, device, dxs, ds0)
            tuned["launch_bw"](ptrs, device)
            check_status(device, "backward")
            check_guard(device)
            for i, go in enumerate(plan.grads):
                if go.atomic:          # accumulated in fp32: now in the input's dtype and layout
                    dxs[i] = th.empty_like(inputs_[i]).copy_(dxs[i])
        return tuple(dxs), ds0

    def kernel_status(device=None) -> int:
        """Error word the kernels write on a timed-out wait (0 = none). Synchronises."""
        device = th.device(device) if device is not None else dev
        if emulated:
            return int(emu_words["w"].item()) if "w" in emu_words else 0
        idx = device.index if device.index is not None else th.cuda.current_device()
        if idx not in _status:
            return 0
        th.cuda.synchronize(idx)
        return int(_status[idx].word.item())

    forward.plan = plan                     # type: ignore[attr-defined]
    forward.sources = (fw_src, bw_src)      # type: ignore[attr-defined]
    forward.launchers = (launch_fw, launch_bw)   # type: ignore[attr-defined]
    forward.kernel_status = kernel_status   # type: ignore[attr-defined]
    forward.tuned = tuned                   # type: ignore[attr-defined]  (which variants were timed and kept)
    return forward, backward, fw_meta, bw_meta
