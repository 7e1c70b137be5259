"""Every kernel variant the autotuner may pick, each checked on its own.

On the first call of a benchmark-sized problem the planner times alternative
forward kernels (tilings, packed or scalar arithmetic, longer staged chunks, one
fully unrolled chunk per checkpoint interval) and backward kernels (tilings,
the other kind of arithmetic), and keeps the fastest; which one
wins depends on the GPU's state at that moment.  So parity must hold for every
member of ``forward_variants`` / ``backward_variants``, not only for the
planned kernel that small test cases run.  Here each member is forced through
``Tuning.fw_variant`` / ``Tuning.bw_variant`` and compared with the oracle:
on the GPU at the benchmark's state sizes (short sequences), and under the
host emulation at a smaller state for the two backward modes.
"""
import dataclasses

import pytest
import torch

from flex_rnn_b200 import twopass
from flex_rnn_b200.twopass import backward_variants, build_twopass, default_tuning, forward_variants, make_plan
from oracle import naive_oracle as O


def _variant_counts(op, xs, tu):
    plan, _, _ = make_plan(O.STEPS[op], tuple(xs[:-1]), (xs[-1],), tu)
    return plan, len(forward_variants(plan)), len(backward_variants(plan))


def _run_variant(op, xs, dy, dS, tu, launcher=None):
    fwd, bwd, _, _ = build_twopass(O.STEPS[op], tuple(xs[:-1]), (xs[-1],), tuning=tu, _launcher=launcher)
    y, ST, store, aux = fwd(tuple(xs[:-1]), (xs[-1],))
    dx, ds0 = bwd((dy.to(y.dtype),), (dS.to(ST.dtype),), tuple(xs[:-1]), (store,), (aux,))
    return y, ST, list(dx) + list(ds0), fwd


def _check(op, k, xs, dy, dS, got, tol_out, tol_grad):
    y, ST, grads = got
    ref_in = [x.detach().cpu() for x in xs]
    ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op], ref_in[:-1], ref_in[-1:], [dy.cpu().to(y.dtype).float()],
                                  [dS.cpu().to(ST.dtype).float()], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < tol_out and O.rel_err(ST, rST[0]) < tol_out, (op, "variant", k)
    for g, r in zip(grads, rgx + rgs):
        assert O.rel_err(g, r) < tol_grad, (op, "variant", k, O.rel_err(g, r))


@pytest.mark.parametrize("op", ["delta_rule", "gated_delta_rule"])
def test_every_variant_emulated(op):
    """Reverse re-step (Delta Rule) and recomputing (Gated Delta Rule) backward,
    32x64 state: the candidate lists hold several distinct tilings there."""
    from emu.emu import EmuLauncher
    B, T, H, M, N = 1, 10, 1, 32, 64
    xs, dy, dS = O.make_case(op, B, T, H, M, N, torch.float32)
    tu = dataclasses.replace(default_tuning(B, T, H, M, N, 1), autotune=0)
    plan, nf, nb = _variant_counts(op, xs, tu)
    assert nf >= 3 and nb >= 2
    tiles = set()
    for k in range(max(nf, nb)):
        tk = dataclasses.replace(tu, fw_variant=min(k, nf - 1), bw_variant=min(k, nb - 1))
        y, ST, grads, fwd = _run_variant(op, xs, dy, dS, tk, EmuLauncher)
        tiles.add((hash(fwd.sources[0].source), hash(fwd.sources[1].source)))
        assert fwd.tuned["fw_choice"] == min(k, nf - 1) and fwd.tuned["bw_choice"] == min(k, nb - 1)
        _check(op, k, xs, dy, dS, (y, ST, grads), 1e-5, 1e-5)
    assert len(tiles) == max(nf, nb)          # the variants really are different kernels


GPU_SHAPES = {"delta_rule": (128, 128), "rwkv7": (128, 128), "mamba2": (64, 128), "gated_delta_rule": (128, 128)}


@pytest.mark.gpu
@pytest.mark.parametrize("op", list(GPU_SHAPES))
def test_every_variant_gpu(op):
    """The benchmark's state sizes and dtype (bf16), B1 H2, 40 steps (several
    checkpoint chunks and a ragged last chunk)."""
    M, N = GPU_SHAPES[op]
    B, T, H = 1, 40, 2
    xs, dy, dS = O.make_case(op, B, T, H, M, N, torch.bfloat16)
    xs = [x.to("cuda:0") for x in xs]
    dy, dS = dy.to("cuda:0"), dS.to("cuda:0")
    tu = dataclasses.replace(default_tuning(B, T, H, M, N, 1), autotune=0)
    plan, nf, nb = _variant_counts(op, xs, tu)
    assert nf >= 4 and nb >= 2
    seen = []
    for k in range(max(nf, nb)):
        tk = dataclasses.replace(tu, fw_variant=min(k, nf - 1), bw_variant=min(k, nb - 1))
        y, ST, grads, fwd = _run_variant(op, xs, dy, dS, tk)
        torch.cuda.synchronize()
        assert fwd.kernel_status("cuda:0") == 0
        seen.append((fwd.sources[0].info["tile"], fwd.sources[0].info["packed"], fwd.sources[1].info["tile"]))
        _check(op, k, xs, dy, dS, (y.cpu(), ST.cpu(), [g.cpu() for g in grads]), 5e-3, 1e-2)
    print(f"[variants] {op}: {seen}")
