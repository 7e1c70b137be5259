"""The CPU oracle against the fixtures produced by the reference's own
``jit.naive`` (tests/golden/make_golden.py) and the known-answer norms."""
import json
import os

import pytest
import torch

from oracle import naive_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("op", list(O.STEPS))
@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_oracle_matches_reference_naive(op, tag):
    fx = torch.load(os.path.join(GOLDEN, f"{op}_{tag}.pt"))
    dtype = torch.float32 if tag == "fp32" else torch.bfloat16
    xs, dy, dS = O.make_case(op, dtype=dtype, **fx["shape"])
    for a, b in zip(xs, fx["inputs"]):
        assert torch.equal(a, b), "seeded inputs differ from the fixture"
    assert torch.equal(dy, fx["dy"]) and torch.equal(dS, fx["dS"])
    y, ST, gx, gs = O.fwd_bwd(O.STEPS[op], xs[:-1], xs[-1:], [dy], [dS])
    assert y[0].dtype == fx["y"].dtype and ST[0].dtype == fx["ST"].dtype
    assert torch.equal(y[0], fx["y"])
    assert torch.equal(ST[0], fx["ST"])
    for g, r in zip(gx + gs, fx["grads"]):
        assert g.dtype == r.dtype
        assert O.rel_err(g, r) < 1e-6
    # fp64 variant
    y, ST, gx, gs = O.fwd_bwd(O.STEPS[op], xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    assert O.rel_err(y[0], fx["fp64"]["y"]) < 1e-12
    for g, r in zip(gx + gs, fx["fp64"]["grads"]):
        assert O.rel_err(g, r) < 1e-6


def test_known_answer_norms():
    """L2 norms of [y, S_T, *grads] at seed 0, B2 T64 H4 (64x64; Mamba-2 32x64),
    fp32, recorded from the reference's naive on torch's CPU generator."""
    norms = json.load(open(os.path.join(GOLDEN, "norms_c0.json")))
    expect_delta = [62.648118, 82.242255, 502.915756, 893.832979, 101.341143, 208.305696, 198.106522]
    assert all(abs(a - b) < 1e-4 for a, b in zip(norms["delta_rule"]["norms"], expect_delta))
    for op, rec in norms.items():
        xs, dy, dS = O.make_case(op, dtype=torch.float32, **rec["shape"])
        y, ST, gx, gs = O.fwd_bwd(O.STEPS[op], xs[:-1], xs[-1:], [dy], [dS])
        got = [float(t.double().norm()) for t in [y[0], ST[0], *gx, *gs]]
        for a, b in zip(got, rec["norms"]):
            assert abs(a - b) <= 1e-5 * max(1.0, abs(b)), (op, got, rec["norms"])


def test_scan_semantics_edge_cases():
    """Broadcast over T and B, dtype of the final state, single step."""
    xs, dy, dS = O.make_case("mamba2", 2, 5, 3, 4, 8, torch.float32)
    assert xs[2].shape == (1, 1, 3, 1, 1)
    outs, fin = O.scan(O.mamba2, xs[:-1], xs[-1:])
    assert outs[0].shape == (2, 5, 3, 4) and fin[0].shape == (2, 3, 4, 8)
    xs16 = [x.bfloat16() for x in xs]
    outs, fin = O.scan(O.mamba2, xs16[:-1], xs16[-1:])
    assert outs[0].dtype == torch.float32 and fin[0].dtype == torch.bfloat16   # as jit.naive does
    # one timestep equals one direct call of the step
    xs1, _, _ = O.make_case("delta_rule", 1, 1, 1, 4, 4, torch.float32)
    outs, fin = O.scan(O.delta_rule, xs1[:-1], xs1[-1:])
    y, S = O.delta_rule(*[x[:, 0] for x in xs1[:-1]], xs1[-1])
    assert torch.allclose(outs[0][:, 0], y.squeeze(-1)) and torch.allclose(fin[0], S)
    # a transposed (dense, non-contiguous) initial state keeps its strides in the result
    S0 = torch.randn(1, 1, 4, 4).mT
    outs, fin = O.scan(O.delta_rule, xs1[:-1], [S0])
    assert fin[0].stride() == S0.stride()
