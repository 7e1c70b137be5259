"""Step families beyond the four benchmark ones (the other examples of the
reference's tests/examples.py): several states, states with one column,
time-invariant row / matrix inputs, comparisons, divisions, sums of row
vectors.  CPU: the generated kernels under the host emulation; GPU: the public
API.  Oracle: the naive scan in fp64 + autograd."""
import pytest
import torch

import flex_rnn_b200
from flex_rnn_b200 import workloads as W
from flex_rnn_b200.twopass import Tuning, build_twopass
from oracle import naive_oracle as O


def shapes(op):
    if op in ("rwkv4", "hgrn"):
        return 64, 1
    return 16, 16


def oracle(op, ins, sts, dys, dSs):
    return O.fwd_bwd(W.ZOO[op], ins, sts, dys, dSs, dtype=torch.float64)


@pytest.mark.parametrize("op", ["rwkv6", "rwkv4", "s4d", "longhorn"])
def test_emulated(op):
    from emu.emu import EmuLauncher
    M, N = shapes(op)
    ins, sts = W.zoo_case(op, 2, 7, 2, M, N)
    tu = Tuning(fw_r=2, fw_c=4, fw_mb=16, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)
    fwd, bwd, _, _ = build_twopass(W.ZOO[op], tuple(ins), tuple(sts), tuning=tu, _launcher=EmuLauncher)
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


@pytest.mark.gpu
@pytest.mark.parametrize("op", [k for k in W.ZOO if k != "mlstm_gates"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gpu(op, dtype):
    M, N = (256, 1) if op in ("rwkv4", "hgrn") else (64, 64)
    ins, sts = W.zoo_case(op, 2, 40, 3, M, N, dtype)
    dev = "cuda:0"
    leaves = [x.to(dev).requires_grad_() for x in ins + sts]
    f = flex_rnn_b200.jit(W.ZOO[op])
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
