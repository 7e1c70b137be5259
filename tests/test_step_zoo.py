"""Step families beyond the four benchmark ones (the other examples of the
reference's tests/examples.py): several states, states with one column,
time-invariant row / matrix inputs, comparisons, divisions, sums of row
vectors.  CPU: the generated kernels under the host emulation; GPU: the public
API.  Oracle: the naive scan in fp64 + autograd."""
import pytest
import torch

import flex_rnn_b200
from flex_rnn_b200 import examples as X
from flex_rnn_b200 import workloads as W
from flex_rnn_b200.twopass import Tuning, build_twopass
from oracle import naive_oracle as O


def shapes(op):
    if op in ("rwkv4", "hgrn"):
        return 64, 1
    return 16, 16


def oracle(op, ins, sts, dys, dSs):
    return O.fwd_bwd(X.ZOO[op], ins, sts, dys, dSs, dtype=torch.float64)


@pytest.mark.parametrize("op", ["rwkv6", "rwkv4", "s4d", "longhorn"])
def test_emulated(op):
    from emu.emu import EmuLauncher
    M, N = shapes(op)
    ins, sts = X.zoo_case(op, 2, 7, 2, M, N)
    tu = Tuning(fw_r=2, fw_c=4, fw_mb=16, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)
    fwd, bwd, _, _ = build_twopass(X.ZOO[op], tuple(ins), tuple(sts), tuning=tu, _launcher=EmuLauncher)
    res = fwd(tuple(ins), tuple(sts))
    ns = len(sts)
    no = len(res) - 2 * ns - 1
    g = torch.Generator().manual_seed(1)
    dys = [torch.randn(y.shape, generator=g) for y in res[:no]]
    dSs = [torch.randn(s.shape, generator=g) for s in sts]
    dx, ds0 = bwd(tuple(dys), tuple(dSs), tuple(ins), tuple(res[no + ns:no + 2 * ns]), (res[-1],))
    ry, rST, rgx, rgs = oracle(op, ins, sts, dys, dSs)
    for a, b in zip(list(res[:no + ns]) + list(dx) + list(ds0), list(ry) + list(rST) + rgx + rgs):
        assert a.shape == b.shape
        assert O.rel_err(a, b) < 1e-5


@pytest.mark.parametrize("op,M,N", [("mlstm_gates", 1, 1), ("hgrn", 4, 1), ("gla", 2, 4)])
def test_emulated_small_state(op, M, N):
    """States with fewer elements than a warp has threads (the reference runs
    them with one thread per element, twopass.py:154-164) go through the same
    kernels on repeated rows; three outputs for the mLSTM gates."""
    from emu.emu import EmuLauncher
    from flex_rnn_b200.twopass import verify_meta
    ins, sts = X.zoo_case(op, 2, 7, 2, M, N)
    tu = Tuning(fw_r=2, fw_c=4, fw_mb=16, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)
    fwd, bwd, fm, bm = build_twopass(X.ZOO[op], tuple(ins), tuple(sts), tuning=tu, _launcher=EmuLauncher)
    assert fwd.padded_rows % M == 0 and fwd.padded_rows > M
    meta = tuple(x.to("meta") for x in ins), tuple(s.to("meta") for s in sts)
    assert build_twopass(X.ZOO[op], *meta, dryrun=True) == (fm, bm)
    res = fwd(tuple(ins), tuple(sts))
    ns = len(sts)
    no = len(res) - 2 * ns - 1
    assert no == (3 if op == "mlstm_gates" else 1)
    g = torch.Generator().manual_seed(1)
    dys = [torch.randn(y.shape, generator=g) for y in res[:no]]
    dSs = [torch.randn(s.shape, generator=g) for s in sts]
    dx, ds0 = bwd(tuple(dys), tuple(dSs), tuple(ins), tuple(res[no + ns:no + 2 * ns]), (res[-1],))
    verify_meta(res, [torch.empty_strided(a, b, dtype=c) for a, b, c in fm])
    verify_meta(list(dx) + list(ds0), [torch.empty_strided(a, b, dtype=c) for a, b, c in bm])
    ry, rST, rgx, rgs = oracle(op, ins, sts, dys, dSs)
    for a, b in zip(list(res[:no + ns]) + list(dx) + list(ds0), list(ry) + list(rST) + rgx + rgs):
        assert a.shape == b.shape
        assert O.rel_err(a, b) < 1e-5


@pytest.mark.parametrize("M,N", [(1, 32), (1, 64), (32, 1)])
def test_emulated_one_row_or_column_state(M, N):
    """A state of one row ([B,H,1,N]: the mLSTM normaliser) makes the output
    gradient a single value per step and every column input a scalar; a state of
    one column does the same to the row inputs."""
    from emu.emu import EmuLauncher
    step2 = _mlstm_steps()[1]
    B, T, H = 2, 12, 2
    g = torch.Generator().manual_seed(5)
    n = lambda *s: torch.randn(*s, generator=g)
    ins = (n(B, T, H, 1, N), n(B, T, H, 1, N), n(B, T, H, 1, 1), torch.sigmoid(n(B, T, H, 1, 1)))
    for step, xs in ((step2, ins), (W.delta_rule, (ins[0] / N ** .5, ins[1] / N ** .5, n(B, T, H, M, 1), ins[3]))):
        sts = (n(B, H, M, N),)
        fwd, bwd, _, _ = build_twopass(step, xs, sts, _launcher=EmuLauncher)
        res = fwd(xs, sts)
        dys, dSs = [n(*res[0].shape)], [n(*sts[0].shape)]
        dx, ds0 = bwd(tuple(dys), tuple(dSs), xs, (res[2],), (res[3],))
        ry, rST, rgx, rgs = O.fwd_bwd(step, list(xs), list(sts), dys, dSs, dtype=torch.float64)
        for a, b in zip(list(res[:2]) + list(dx) + list(ds0), list(ry) + list(rST) + rgx + rgs):
            assert a.shape == b.shape and O.rel_err(a, b) < 1e-5


LARGE = [("s4d", 256, 128), ("mamba", 256, 256), ("rwkv4", 8192, 1), ("rwkv6", 256, 256)]


@pytest.mark.gpu
@pytest.mark.parametrize("op,M,N", LARGE, ids=[c[0] for c in LARGE])
def test_gpu_states_larger_than_one_cta(op, M, N):
    """Rows of a head split over several CTAs in both kernels: two states plus four
    matrix inputs with their gradients (S4D), a matrix input's gradient across the
    split (Mamba), three one-column states of 8192 rows (RWKV-4), a time-invariant
    row input whose gradient sums over the split rows (RWKV-6)."""
    test_gpu(op, torch.float32, M=M, N=N, T=12, B=1, H=2)
    assert _last["f"].forward_func.sources[1].grid[0] > 1


_last = {}


@pytest.mark.gpu
@pytest.mark.parametrize("op", list(X.ZOO))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gpu(op, dtype, M=None, N=None, T=40, B=2, H=3):
    if M is None:
        M, N = (256, 1) if op in ("rwkv4", "hgrn") else (1, 1) if op == "mlstm_gates" else (64, 64)
    ins, sts = X.zoo_case(op, B, T, H, M, N, dtype)
    dev = "cuda:0"
    leaves = [x.to(dev).requires_grad_() for x in ins + sts]
    f = flex_rnn_b200.jit(X.ZOO[op])
    _last["f"] = f
    outs = f(*leaves)
    g = torch.Generator().manual_seed(1)
    ups = [torch.randn(o.shape, generator=g) for o in outs]
    grads = torch.autograd.grad(list(outs), leaves, [u.to(dev).to(o.dtype) for u, o in zip(ups, outs)], allow_unused=True)
    torch.cuda.synchronize()
    assert f.forward_func.kernel_status(dev) == 0
    no = len(outs) - len(sts)
    ups_r = [u.to(dtype).float() for u in ups]
    ry, rST, rgx, rgs = oracle(op, ins, sts, ups_r[:no], ups_r[no:])
    tol_out, tol_grad = (1e-5, 2e-5) if dtype == torch.float32 else (5e-3, 1e-2)
    for a, b in zip(outs, list(ry) + list(rST)):
        assert O.rel_err(a, b) < tol_out
    for a, b, x in zip(grads, rgx + rgs, ins + sts):
        a = torch.zeros_like(x) if a is None else a
        assert a.shape == x.shape and a.dtype == x.dtype
        if float(b.abs().max()) == 0.0:
            assert float(a.float().abs().max()) == 0.0
        else:
            assert O.rel_err(a, b) < tol_grad, (op, O.rel_err(a, b))


def _mlstm(step1, step2, step3, q, k, v, i, f, sa, sb, sc):
    """The three-kernel mLSTM pipeline of the reference's examples
    (tests/examples.py:396-426): gates on a 1x1 state, the normaliser on a
    one-row state, then the matrix state; layout adaptors are views."""
    C = q.shape[-1]
    i, f, sb, sc = [x.unsqueeze(-1) for x in [i, f, sb, sc]]
    q, k, v, i, f = [x.transpose(1, 2).unsqueeze(-2) for x in [q, k, v, i, f]]
    i, f, sc, scT = step1(i, f, sc)
    i, f = i.unsqueeze(-1), f.unsqueeze(-1)
    sb_q, sbT = step2(k, q, i, f, sb.mT)
    norm = 1 / (torch.maximum(torch.abs(sb_q), (-sc).exp() * C ** .5) + 1e-6 * C ** .5).unsqueeze(-1)
    y, saT = step3(q, k, v.mT, i, f, norm, sa.mT)
    return y.transpose(1, 2), saT.mT, sbT.squeeze(-2), scT.squeeze(-1)


def _mlstm_steps():
    def step2(k, q, i, f, sb):
        sb_ = f * sb + i * k
        return (sb_ * q).sum(-1, True), sb_

    def step3(q, k, v, i, f, norm, sa):
        sa_ = f * sa + i * v * k
        return (norm * q * sa_).sum(-1, True), sa_
    return X.mlstm_gates, step2, step3


def _gsa(step1, step2, q, k, v, x, g, sa, sb):
    """Two chained kernels with a softmax between them (tests/examples.py:356-371)."""
    q, k, v, x, g = [i.unsqueeze(-2) for i in [q, k, v, x, g]]
    qv, sa = step1(q, k, x.mT, g.mT, sa.mT)
    qv = qv.softmax(-1).unsqueeze(-2)
    y, sb = step2(qv.to(q.dtype), x, v.mT, g, sb.mT)
    return y, sa.mT, sb.mT


def _gsa_steps():
    def step1(q, k, x, g, s):
        s = g.exp() * s + x * k
        return (s * q).sum(-1, True), s

    def step2(q, x, v, g, s):
        s = g.exp() * s + v * x
        return (s * q).sum(-1, True), s
    return step1, step2


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mlstm", "gsa"])
def test_gpu_pipelines(name):
    """Multi-kernel callers: every stage compiled by this backend, chained
    through views and ordinary torch ops, differentiated end to end, against
    the same pipeline on the naive scans in fp64."""
    B, T, H, C = 2, 24, 3, 32
    g = torch.Generator().manual_seed(3)
    n = lambda *s: torch.randn(*s, generator=g)
    if name == "mlstm":
        args = [n(B, H, T, C), n(B, H, T, C) / C ** .5, n(B, H, T, C), n(B, H, T), n(B, H, T) + 2,
                n(B, H, C, C), n(B, H, C), n(B, H, 1)]
        steps, pipe = _mlstm_steps(), _mlstm
    else:
        args = [n(B, T, H, C), n(B, T, H, C), n(B, T, H, C), n(B, T, H, C), -torch.sigmoid(n(B, T, H, C)),
                n(B, H, C, C), n(B, H, C, C)]
        steps, pipe = _gsa_steps(), _gsa
    dev = "cuda:0"
    ops = [flex_rnn_b200.jit(s) for s in steps]
    leaves = [a.to(dev).requires_grad_() for a in args]
    outs = pipe(*ops, *leaves)
    ups = [torch.randn(o.shape, generator=g) for o in outs]
    grads = torch.autograd.grad(list(outs), leaves, [u.to(dev) for u in ups])
    torch.cuda.synchronize()
    for o in ops:
        assert o.forward_func.kernel_status(dev) == 0
    ref_leaves = [a.double().requires_grad_() for a in args]
    ref_outs = pipe(*[o.naive_fp64 for o in ops], *ref_leaves)
    ref_grads = torch.autograd.grad(list(ref_outs), ref_leaves, [u.double() for u in ups])
    for a, b in zip(list(outs) + list(grads), list(ref_outs) + list(ref_grads)):
        assert a.shape == b.shape
        assert O.rel_err(a, b) < 5e-5, (name, O.rel_err(a, b))


# ---- operations beyond the reference's table (+ - * / < > exp log sqrt, to_cuda.py:41-42) ----

def _op_relu_mask(q, k, v, w, S):
    S = S * torch.exp(-torch.relu(w)) + v * k * (k > 0)
    return (S * q).sum(-1, True), S


def _op_normalise(q, k, v, S):
    S = S + v * k
    S = S / (1 + (S * S).sum(-1, True))
    return torch.log1p((S * q).sum(-1, True) ** 2), S


def _op_maximum(q, k, v, w, S):
    S = torch.maximum(S * torch.sigmoid(w), v * k)
    return (S * q).sum(-1, True), S


def _op_silu(q, k, v, S):
    S = S * 0.5 + torch.nn.functional.silu(v * k)
    return (S * q).sum(-1, True), S


def _op_sign_clamp(q, k, v, S):
    S = S - 0.1 * torch.sign(S) + v * k
    return (S * q).sum(-1, True).clamp(-2, 2), S


def _op_minimum_reciprocal(q, k, v, S):
    S = torch.minimum(S * 0.9 + v * k, torch.ones_like(S) * 2)
    return (S * q).sum(-1, True).exp().reciprocal(), S


def _op_mean(q, k, v, S):
    S = S * 0.9 + v * k
    return (S * q).sum(-1, True) - (S * q).mean(-1, True), S


def _op_softplus_where(q, k, v, S):
    S = torch.where(S > 1, S * 0.5, S) + torch.nn.functional.softplus(v * k)
    return torch.sqrt(torch.abs((S * q).sum(-1, True)) + 1), S


def _op_gelu_elu(q, k, v, S):
    S = S * 0.9 + torch.nn.functional.gelu(v) * k
    return torch.nn.functional.elu((S * q).sum(-1, True)), S


def _op_tanh_state(q, k, v, S):
    S = torch.tanh(S + v * k)
    y = (S * q).sum(-1, True)
    return y * torch.rsqrt(1 + y * y), S


OPERATION_STEPS = [_op_relu_mask, _op_normalise, _op_maximum, _op_silu, _op_sign_clamp, _op_minimum_reciprocal,
                   _op_mean, _op_softplus_where, _op_gelu_elu, _op_tanh_state]


def _operation_case(step, B=2, T=7, H=2, M=8, N=16):
    import inspect
    g = torch.Generator().manual_seed(0)
    n = lambda *s: torch.randn(*s, generator=g)
    ins = [n(B, T, H, 1, N) * 0.5, n(B, T, H, 1, N) * 0.5, n(B, T, H, M, 1)]
    if len(inspect.signature(step).parameters) == 5:
        ins.append(n(B, T, H, 1, N))
    return ins, [n(B, H, M, N) * 0.5], n(B, T, H, M), n(B, H, M, N)


@pytest.mark.parametrize("step", OPERATION_STEPS, ids=lambda f: f.__name__[4:])
def test_emulated_operations(step):
    """Activations, masks, clamps and means in the state update and in the
    output, forward and backward (autograd's formulas for them are imported
    operation by operation, flex_rnn_b200/graph.py)."""
    from emu.emu import EmuLauncher
    ins, sts, dy, dS = _operation_case(step)
    tu = Tuning(fw_r=2, fw_c=4, fw_mb=8, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)
    fwd, bwd, _, _ = build_twopass(step, tuple(ins), tuple(sts), tuning=tu, _launcher=EmuLauncher)
    res = fwd(tuple(ins), tuple(sts))
    dx, ds0 = bwd((dy,), (dS,), tuple(ins), (res[2],), (res[3],))
    ry, rST, rgx, rgs = O.fwd_bwd(step, ins, sts, [dy], [dS], dtype=torch.float64)
    for a, b in zip(list(res[:2]) + list(dx) + list(ds0), list(ry) + list(rST) + rgx + rgs):
        assert a.shape == b.shape and O.rel_err(a, b) < 3e-5


@pytest.mark.gpu
@pytest.mark.parametrize("step", OPERATION_STEPS, ids=lambda f: f.__name__[4:])
def test_gpu_operations(step):
    ins, sts, dy, dS = _operation_case(step, 2, 40, 3, 64, 64)
    dev = "cuda:0"
    leaves = [x.to(dev).requires_grad_() for x in ins + sts]
    f = flex_rnn_b200.jit(step)
    y, ST = f(*leaves)
    grads = torch.autograd.grad([y, ST], leaves, [dy.to(dev), dS.to(dev)])
    torch.cuda.synchronize()
    assert f.forward_func.kernel_status(dev) == 0
    ry, rST, rgx, rgs = O.fwd_bwd(step, ins, sts, [dy], [dS], dtype=torch.float64)
    for a, b in zip([y, ST] + list(grads), list(ry) + list(rST) + rgx + rgs):
        assert a.shape == b.shape and O.rel_err(a, b) < 3e-5


@pytest.mark.gpu
def test_gpu_pipeline_under_torch_compile():
    """The three-kernel mLSTM pipeline (1x1 gate state padded with repeated
    rows, one-row normaliser, matrix state) compiled as one graph: the custom
    ops stay opaque, their fake implementations plan without touching the GPU,
    and values and gradients equal the eager run."""
    B, T, H, C = 2, 16, 2, 32
    g = torch.Generator().manual_seed(4)
    n = lambda *s: torch.randn(*s, generator=g)
    dev = "cuda:0"
    args = [a.to(dev) for a in [n(B, H, T, C), n(B, H, T, C) / C ** .5, n(B, H, T, C), n(B, H, T), n(B, H, T) + 2,
                                n(B, H, C, C), n(B, H, C), n(B, H, 1)]]
    ops = [flex_rnn_b200.jit(s) for s in _mlstm_steps()]
    fn = lambda *a: _mlstm(*ops, *a)
    compiled = torch.compile(fn, fullgraph=True)
    out = []
    for f in (fn, compiled):
        leaves = [a.clone().requires_grad_() for a in args]
        res = f(*leaves)
        grads = torch.autograd.grad([r.sum() for r in res], leaves)
        out.append(list(res) + list(grads))
    for a, b in zip(*out):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
