"""The front-end contract of the reference's ``jit`` object, on both sides of
the Python boundary:

* ``jit.naive`` / ``naive_fp64`` of this package reproduce the golden fixtures
  (made by the reference's own ``jit.naive``) bit for bit - two GPU tests use
  them as their reference side;
* upstream gradients that autograd leaves out (``None``) are zeros
  (reference: flex_rnn/jit.py:76-80);
* one ``jit`` object called with states of other strides or dtype
  re-specialises, and each backward finds the kernels of its own forward;
* the reference's UNMODIFIED ``flex_rnn/jit.py`` runs on top of this package's
  ``build_twopass`` (it imports ``build_twopass, split_list, verify_meta`` from
  ``flex_rnn.twopass``, flex_rnn/jit.py:5): the drop-in claim of the Python
  boundary.  The file is taken from an install of the reference under
  ``baseline/_ref`` when one is present (it is not part of this repository).

The CPU variants run the generated kernels under the host emulation, injected
through the test seam of ``build_twopass``; the GPU variants run the real path.
"""
import functools
import importlib.util
import os
import sys
import types

import pytest
import torch

import flex_rnn_b200
from flex_rnn_b200 import twopass
from oracle import naive_oracle as O

jit_mod = sys.modules["flex_rnn_b200.jit"]     # the module (the package re-exports the class under the same name)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
REF_JIT = os.path.join(ROOT, "baseline", "_ref", "flex_rnn", "jit.py")
SMALL = twopass.Tuning(fw_r=2, fw_c=4, fw_mb=8, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)


@pytest.fixture
def emulated(monkeypatch):
    """jit objects built inside this fixture launch through the host emulation."""
    from emu.emu import EmuLauncher
    build = functools.partial(twopass.build_twopass, tuning=SMALL, _launcher=EmuLauncher)

    def build_twopass(step, inputs, state, dryrun=False):
        return build(step, inputs, state, dryrun)
    monkeypatch.setattr(jit_mod, "build_twopass", build_twopass)
    return build_twopass


# ---------------------------------------------------------------- naive vs golden

@pytest.mark.parametrize("op_name", list(O.STEPS))
@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_naive_reproduces_reference_fixtures(op_name, tag):
    fx = torch.load(os.path.join(GOLDEN, f"{op_name}_{tag}.pt"))
    op = flex_rnn_b200.jit(O.STEPS[op_name])
    for ref, fn in ((fx, op.naive), (fx["fp64"], op.naive_fp64)):
        leaves = [x.clone().requires_grad_() for x in fx["inputs"]]
        y, ST = fn(*leaves)
        assert y.dtype == ref["y"].dtype and ST.dtype == ref["ST"].dtype
        assert torch.equal(y, ref["y"]) and torch.equal(ST, ref["ST"])
        grads = torch.autograd.grad([y, ST], leaves, [fx["dy"].to(y.dtype), fx["dS"].to(ST.dtype)])
        for g, r in zip(grads, ref["grads"]):
            assert g.dtype == r.dtype and O.rel_err(g, r) < 1e-6


# ---------------------------------------------------------------- None upstream gradients

def _none_grad_case(dev):
    xs, dy, dS = O.make_case("delta_rule", 2, 9, 2, 16, 16, torch.float32)
    op = flex_rnn_b200.jit(O.delta_rule)
    zero_y, zero_S = torch.zeros_like(dy), torch.zeros_like(dS)
    for up_y, up_S, ref_up in ((dy, None, (dy, zero_S)), (None, dS, (zero_y, dS))):
        leaves = [x.to(dev).requires_grad_() for x in xs]
        y, ST = op(*leaves)
        outs, ups = ([y], [up_y.to(dev)]) if up_S is None else ([ST], [up_S.to(dev)])
        grads = torch.autograd.grad(outs, leaves, ups)
        _, _, rgx, rgs = O.fwd_bwd(O.delta_rule, xs[:-1], xs[-1:], [ref_up[0]], [ref_up[1]], dtype=torch.float64)
        for g, r in zip(grads, rgx + rgs):
            assert O.rel_err(g, r) < 1e-5


def test_none_upstream_gradients_emulated(emulated):
    _none_grad_case("cpu")


@pytest.mark.gpu
def test_none_upstream_gradients_gpu():
    _none_grad_case("cuda:0")


# ---------------------------------------------------------------- one jit object, several state layouts

def _state_layout_case(dev):
    """Contiguous fp32 state, then a transposed (.mT) view, then a bf16 state,
    all with the same inputs; the backward passes run afterwards, in another
    order, so each must find the specialisation of its own forward."""
    B, T, H, M, N = 1, 7, 2, 16, 16
    xs, dy, dS = O.make_case("delta_rule", B, T, H, M, N, torch.float32)
    op = flex_rnn_b200.jit(O.delta_rule)
    ins = [x.to(dev) for x in xs[:-1]]
    S0 = xs[-1].to(dev)
    states = [S0.clone(), S0.transpose(-1, -2).contiguous().mT, S0.bfloat16()]
    runs = []
    for st in states:
        leaves = [x.clone().requires_grad_() for x in ins] + [st.detach().requires_grad_()]
        y, ST = op(*leaves)
        assert ST.stride() == st.stride() and ST.dtype == st.dtype
        runs.append((leaves, y, ST))
    assert len(op._compiled) == 3
    for k in (1, 2, 0):
        leaves, y, ST = runs[k]
        grads = torch.autograd.grad([y, ST], leaves, [dy.to(dev), dS.to(dev).to(ST.dtype)])
        assert grads[-1].stride() == states[k].stride() and grads[-1].dtype == states[k].dtype
        ref_in = [x for x in xs[:-1]] + [states[k].detach().cpu().contiguous()]
        ry, rST, rgx, rgs = O.fwd_bwd(O.delta_rule, ref_in[:-1], ref_in[-1:], [dy], [dS], dtype=torch.float64)
        tol = 1e-5 if k < 2 else 1e-2
        assert O.rel_err(y, ry[0]) < tol and O.rel_err(ST, rST[0]) < tol
        for g, r in zip(grads, rgx + rgs):
            assert O.rel_err(g, r) < tol, k


def test_state_layouts_share_one_jit_object_emulated(emulated):
    _state_layout_case("cpu")


@pytest.mark.gpu
def test_state_layouts_share_one_jit_object_gpu():
    _state_layout_case("cuda:0")


# ---------------------------------------------------------------- the reference's own jit.py on this backend

def _load_reference_jit(build_twopass):
    """Execute the reference's jit.py with ``flex_rnn.twopass`` bound to this
    package's planner.  Nothing else of the reference is imported."""
    if not os.path.exists(REF_JIT):
        pytest.skip("no install of the reference under baseline/_ref (its jit.py is not part of this repository)")
    saved = {k: sys.modules.get(k) for k in ("flex_rnn", "flex_rnn.twopass", "flex_rnn.jit")}
    pkg = types.ModuleType("flex_rnn")
    pkg.__path__ = []
    tp = types.ModuleType("flex_rnn.twopass")
    tp.build_twopass, tp.split_list, tp.verify_meta = build_twopass, twopass.split_list, twopass.verify_meta
    sys.modules["flex_rnn"], sys.modules["flex_rnn.twopass"] = pkg, tp
    try:
        spec = importlib.util.spec_from_file_location("flex_rnn.jit", REF_JIT)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return mod


def _reference_frontend_case(ref_jit, dev, op_name="delta_rule"):
    xs, dy, dS = O.make_case(op_name, 2, 9, 2, 16, 16, torch.float32)
    op = ref_jit.jit(O.STEPS[op_name])
    leaves = [x.to(dev).requires_grad_() for x in xs]
    y, ST = op(*leaves)
    grads = torch.autograd.grad([y, ST], leaves, [dy.to(dev), dS.to(dev)])
    ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op_name], xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < 1e-5 and O.rel_err(ST, rST[0]) < 1e-5
    for g, r in zip(grads, rgx + rgs):
        assert O.rel_err(g, r) < 1e-5
    # its .naive is the reference's own: same numbers as the oracle restatement
    ny, nST = op.naive(*[x.to(dev) for x in xs])
    assert O.rel_err(ny, ry[0]) < 1e-5 and O.rel_err(nST, rST[0]) < 1e-5
    return op


def test_reference_frontend_on_this_backend_emulated(emulated):
    ref_jit = _load_reference_jit(emulated)
    _reference_frontend_case(ref_jit, "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("op_name", ["delta_rule", "rwkv7"])
def test_reference_frontend_on_this_backend_gpu(op_name):
    """flex_rnn/jit.py:5, 46-67 unmodified, kernels from this package, on the GPU."""
    ref_jit = _load_reference_jit(twopass.build_twopass)
    op = _reference_frontend_case(ref_jit, "cuda:0", op_name)
    torch.cuda.synchronize()
    assert op.forward_func.kernel_status("cuda:0") == 0
    # and under torch.compile without a graph break (the reference's fake implementations call dryrun=True)
    xs, _, _ = O.make_case(op_name, 2, 9, 2, 16, 16, torch.float32)
    xs = [x.to("cuda:0") for x in xs]
    op2 = ref_jit.jit(O.STEPS[op_name])
    torch._dynamo.reset()
    # static shapes: the kernels are specialised for them (recompiling one code location for other shapes
    # would otherwise switch Dynamo to symbolic sizes)
    compiled = torch.compile(lambda *z: op2(*z), fullgraph=True, dynamic=False)
    y0, S0 = op(*xs)
    y1, S1 = compiled(*xs)
    assert torch.equal(y0, y1) and torch.equal(S0, S1)
