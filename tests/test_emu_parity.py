"""The generated CUDA source itself, compiled with g++ against a host emulation
of the few CUDA facilities it uses (tests/emu/frnn_emu.h) and run on CPU
tensors, against the oracle.  This checks index arithmetic, the graph lowering,
both reductions, TMA/plain staging and the checkpoint/recompute schedule of
both kernels without a GPU.  The emulation is injected through the test seam
of build_twopass; the library itself has no CPU path."""
import pytest
import torch

from emu.emu import EmuLauncher
from flex_rnn_b200 import workloads as W
from flex_rnn_b200.twopass import Tuning, build_twopass
from oracle import naive_oracle as O


def run_emu(op, xs, dy, dS, tu):
    fwd, bwd, fw_meta, bw_meta = build_twopass(W.STEPS[op], tuple(xs[:-1]), (xs[-1],), tuning=tu, _launcher=EmuLauncher)
    y, ST, store, aux = fwd(tuple(xs[:-1]), (xs[-1],))
    dx, ds0 = bwd((dy.to(y.dtype),), (dS.to(ST.dtype),), tuple(xs[:-1]), (store,), (aux,))
    return y, ST, list(dx) + list(ds0), fwd


def check(op, xs, dy, dS, got, tol_out, tol_grad):
    y, ST, grads = got
    ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op], xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < tol_out and O.rel_err(ST, rST[0]) < tol_out
    for g, r, x in zip(grads, rgx + rgs, xs):
        assert g.shape == x.shape and g.dtype == x.dtype
        assert O.rel_err(g, r) < tol_grad, (op, O.rel_err(g, r))


SMALL = Tuning(fw_r=2, fw_c=4, fw_mb=8, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)


@pytest.mark.parametrize("op", list(W.STEPS))
def test_fp32_ragged_T(op):
    """T is not a multiple of the stage length nor of the checkpoint chunk."""
    xs, dy, dS = O.make_case(op, 2, 9, 2, 16, 16, torch.float32)
    y, ST, grads, fwd = run_emu(op, xs, dy, dS, SMALL)
    check(op, xs, dy, dS, (y, ST, grads), 1e-5, 1e-5)
    assert fwd.sources[0].info["tma_items"] > 0       # rows of 16 fp32 = 64 B go through the bulk-copy path


@pytest.mark.parametrize("op", list(W.STEPS))
@pytest.mark.parametrize("pack2", [0, 3])
def test_packed_and_scalar_arithmetic(op, pack2):
    """The scan loops written with two-column packed operations in both
    kernels (products folded into packed fused multiply-adds), and without
    them, give the same results."""
    import dataclasses
    xs, dy, dS = O.make_case(op, 1, 6, 2, 8, 16, torch.float32)
    y, ST, grads, fwd = run_emu(op, xs, dy, dS, dataclasses.replace(SMALL, pack2=pack2))
    check(op, xs, dy, dS, (y, ST, grads), 1e-5, 1e-5)
    packed = ["frnn_fma2(" in ks.source.split('extern "C"')[-1] for ks in fwd.sources]
    assert packed == [bool(pack2), bool(pack2)]


@pytest.mark.parametrize("op,M,N,tu", [
    ("mamba2", 8, 16, Tuning(fw_r=1, fw_c=8, fw_mb=8, fw_stage=3, bw_r=1, bw_c=4, seg=3, nslots=1)),
    ("rwkv7", 16, 32, Tuning(fw_r=2, fw_c=8, fw_mb=16, fw_stage=8, bw_r=4, bw_c=8, seg=2, nslots=3)),
    ("gated_delta_rule", 16, 16, Tuning(fw_r=4, fw_c=2, fw_mb=16, fw_stage=5, bw_r=2, bw_c=2, seg=1, nslots=2)),
    ("mamba2", 16, 32, Tuning(fw_r=2, fw_c=8, fw_mb=16, fw_stage=4, bw_r=4, bw_c=4, seg=2, nslots=2, bw_min_blocks=2)),
])
def test_bf16_tilings(op, M, N, tu):
    xs, dy, dS = O.make_case(op, 1, 8, 2, M, N, torch.bfloat16)
    y, ST, grads, _ = run_emu(op, xs, dy, dS, tu)
    assert y.dtype == torch.bfloat16
    check(op, xs, dy.bfloat16().float(), dS.bfloat16().float(), (y, ST, grads), 5e-3, 1e-2)


def test_fp16_and_single_step():
    xs, dy, dS = O.make_case("delta_rule", 1, 1, 2, 16, 32, torch.float16)
    y, ST, grads, _ = run_emu("delta_rule", xs, dy, dS, Tuning(fw_r=2, fw_c=8, fw_mb=16, fw_stage=8, bw_r=8, bw_c=8, seg=1, nslots=1))
    check("delta_rule", xs, dy.half().float(), dS.half().float(), (y, ST, grads), 2e-3, 5e-3)


def test_plain_staging_and_strided_views():
    """No TMA (use_tma off), q/k as halves of one fused tensor, v and the state
    as .mT views: everything goes through the strided plain-load path."""
    B, T, H, M, N = 1, 7, 2, 16, 16
    xs, dy, dS = O.make_case("delta_rule", B, T, H, M, N, torch.float32)
    q, k, v, beta, S0 = xs
    qk = torch.cat([q, k], dim=-1)
    vT = v.transpose(-1, -2).contiguous()
    S0T = S0.transpose(-1, -2).contiguous()
    views = [qk[..., :N], qk[..., N:], vT.mT, beta, S0T.mT]
    tu = Tuning(fw_r=2, fw_c=4, fw_mb=8, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2, use_tma=False)
    y, ST, grads, fwd = run_emu("delta_rule", views, dy, dS, tu)
    assert fwd.sources[0].info["tma_items"] == 0
    assert ST.stride() == views[-1].stride() and grads[-1].stride() == views[-1].stride()
    check("delta_rule", xs, dy, dS, (y, ST, grads), 1e-5, 1e-5)


def test_unused_and_time_invariant_inputs():
    """An input the step ignores gets a zero gradient; an input without a time
    dimension gets its gradient summed over time (and over the batch)."""
    def step(k, v, w, unused, S):
        S = S * w + v * k
        return (S * k).sum(-1, True), S
    B, T, H, M, N = 2, 6, 2, 16, 16
    g = torch.Generator().manual_seed(3)
    k = torch.randn(B, T, H, 1, N, generator=g)
    v = torch.randn(B, T, H, M, 1, generator=g)
    w = torch.rand(1, 1, H, 1, N, generator=g)
    unused = torch.randn(B, T, H, 1, N, generator=g)
    S0 = torch.randn(B, H, M, N, generator=g)
    dy, dS = torch.randn(B, T, H, M, generator=g), torch.randn(B, H, M, N, generator=g)
    xs = [k, v, w, unused, S0]
    fwd, bwd, _, _ = build_twopass(step, tuple(xs[:-1]), (S0,), tuning=SMALL, _launcher=EmuLauncher)
    y, ST, store, aux = fwd(tuple(xs[:-1]), (S0,))
    dx, ds0 = bwd((dy,), (dS,), tuple(xs[:-1]), (store,), (aux,))
    ry, rST, rgx, rgs = O.fwd_bwd(step, xs[:-1], [S0], [dy], [dS], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < 1e-5
    for a, r in zip(list(dx) + list(ds0), rgx + rgs):
        assert a.shape == r.shape
        assert O.rel_err(a, r) < 1e-5 or float(r.abs().max()) == 0.0 and float(a.abs().max()) == 0.0


@pytest.mark.parametrize("op,M,N", [("delta_rule", 48, 96), ("rwkv7", 24, 40)])
def test_sizes_that_are_not_powers_of_two(op, M, N):
    """96 = 32 lanes x 3 columns, 40 = 8 lanes x 5 columns: any N with a
    power-of-two divisor <= 32 that leaves whole warps is accepted."""
    xs, dy, dS = O.make_case(op, 1, 6, 1, M, N, torch.float32)
    fwd, bwd, _, _ = build_twopass(W.STEPS[op], tuple(xs[:-1]), (xs[-1],), _launcher=EmuLauncher)
    y, ST, store, aux = fwd(tuple(xs[:-1]), (xs[-1],))
    dx, ds0 = bwd((dy,), (dS,), tuple(xs[:-1]), (store,), (aux,))
    check(op, xs, dy, dS, (y, ST, list(dx) + list(ds0)), 1e-5, 1e-5)


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_expanded_input(dim):
    """An input expanded (stride 0) over the batch, time or head dimension is
    read with its own strides: no tiled tensor map is built for it (a map would
    need a real byte stride for that dimension), it takes the per-timestep bulk
    copies instead, and its gradient has the full shape."""
    B, T, H, M, N = 2, 6, 2, 16, 16
    xs, dy, dS = O.make_case("delta_rule", B, T, H, M, N, torch.float32)
    shape = list(xs[0].shape)
    shape[dim] = 1
    g = torch.Generator().manual_seed(11)
    small = torch.nn.functional.normalize(torch.randn(shape, generator=g), dim=-1)
    xs[0] = small.expand(B, T, H, 1, N)
    assert xs[0].stride(dim) == 0
    fwd, bwd, _, _ = build_twopass(W.delta_rule, tuple(xs[:-1]), (xs[-1],), tuning=SMALL, _launcher=EmuLauncher)
    for ks in fwd.sources:
        assert all(tm["src"] != "in0" for tm in ks.tmaps)
        assert ks.info["tma_items"] > 0
    y, ST, store, aux = fwd(tuple(xs[:-1]), (xs[-1],))
    dx, ds0 = bwd((dy,), (dS,), tuple(xs[:-1]), (store,), (aux,))
    dense = [x.contiguous() for x in xs]
    check("delta_rule", dense, dy, dS, (y, ST, list(dx) + list(ds0)), 1e-5, 1e-5)


def test_mixed_io_dtypes():
    """bf16, fp16, fp64 and fp32 tensors in one call: the output takes the dtype
    torch's promotion gives the step (fp64 here), the final state its initial
    state's, each gradient its input's; arithmetic in fp32."""
    xs, dy, dS = O.make_case("delta_rule", 1, 9, 2, 16, 16, torch.float32)
    dts = [torch.bfloat16, torch.float16, torch.float64, torch.float32, torch.float32]
    xs = [x.to(d) for x, d in zip(xs, dts)]
    y, ST, grads, _ = run_emu("delta_rule", xs, dy, dS, SMALL)
    assert y.dtype == torch.float64 and ST.dtype == torch.float32
    check("delta_rule", xs, dy, dS, (y, ST, grads), 1e-5, 1e-2)


@pytest.mark.parametrize("op", list(W.STEPS))
def test_backward_rows_split_over_ctas(op):
    """A state too large for one CTA has its rows split over several backward
    CTAs; the gradients summed over rows (per-column and per-head ones) are then
    accumulated across CTAs in fp32.  Forced here on a 16x16 state (8 rows per
    CTA), both backward modes, ragged T."""
    import dataclasses
    xs, dy, dS = O.make_case(op, 2, 9, 2, 16, 16, torch.float32)
    y, ST, grads, fwd = run_emu(op, xs, dy, dS, dataclasses.replace(SMALL, bw_mb=8))
    assert fwd.sources[1].grid[0] == 2 and fwd.sources[1].info["tile"][2] == 8
    assert all(go.atomic for go in fwd.plan.grads if go.cls != (1, 0))
    check(op, xs, dy, dS, (y, ST, grads), 1e-5, 1e-5)
