"""GPU parity: the compiled op (public ``jit`` API -> custom op -> C-ABI launch)
against the CPU oracle and the golden fixtures made by the reference's own
``jit.naive``.  Tolerances (relative L2, the metric of the reference's
check_grad): fp32 I/O 1e-5; bf16/fp16 I/O 5e-3 on outputs and final state,
1e-2 on gradients."""
import os

import pytest
import torch

import flex_rnn_b200
from oracle import naive_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DEV = "cuda:0"


def run_gpu(op_name, xs, dy, dS, wrap=None):
    op = flex_rnn_b200.jit(O.STEPS[op_name])
    leaves = [x.to(DEV).requires_grad_() for x in xs]
    args = wrap(leaves) if wrap else leaves
    y, ST = op(*args)
    grads = torch.autograd.grad([y, ST], leaves, [dy.to(DEV).to(y.dtype), dS.to(DEV).to(ST.dtype)])
    torch.cuda.synchronize()
    assert op.forward_func.kernel_status(DEV) == 0
    return y.cpu(), ST.cpu(), [g.cpu() for g in grads], op


def tolerances(dtype):
    return (1e-5, 1e-5) if dtype == torch.float32 else (5e-3, 1e-2)


@pytest.mark.parametrize("op_name", list(O.STEPS))
@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_golden_fixture(op_name, tag):
    """Inputs and results stored from the reference's jit.naive / naive_fp64."""
    fx = torch.load(os.path.join(GOLDEN, f"{op_name}_{tag}.pt"))
    dtype = torch.float32 if tag == "fp32" else torch.bfloat16
    y, ST, grads, _ = run_gpu(op_name, fx["inputs"], fx["dy"], fx["dS"])
    tol_out, tol_grad = tolerances(dtype)
    ref = fx["fp64"]
    assert O.rel_err(y, ref["y"]) < tol_out
    assert O.rel_err(ST, ref["ST"]) < tol_out
    for g, r in zip(grads, ref["grads"]):
        assert O.rel_err(g, r) < tol_grad


CASES = [
    ("delta_rule", 2, 64, 4, 64, 64, torch.float32),       # the CPU-runnable benchmark configuration
    ("delta_rule", 1, 40, 2, 128, 128, torch.bfloat16),
    ("gated_delta_rule", 2, 33, 2, 128, 128, torch.bfloat16),
    ("rwkv7", 1, 48, 2, 128, 128, torch.bfloat16),
    ("rwkv7", 2, 17, 3, 64, 64, torch.float32),
    ("mamba2", 2, 64, 4, 64, 128, torch.bfloat16),
    ("mamba2", 2, 19, 2, 32, 64, torch.float32),
    ("delta_rule", 1, 24, 2, 64, 64, torch.float16),
    ("delta_rule", 1, 1, 1, 32, 32, torch.float32),         # a single timestep
    ("delta_rule", 2, 21, 2, 48, 96, torch.float32),        # sizes that are not powers of two
    ("rwkv7", 1, 10, 2, 24, 40, torch.bfloat16),
    ("gated_delta_rule", 1, 70, 1, 256, 64, torch.float32),  # tall state, several checkpoint chunks
]


@pytest.mark.parametrize("op_name,B,T,H,M,N,dtype", CASES)
def test_against_oracle(op_name, B, T, H, M, N, dtype):
    xs, dy, dS = O.make_case(op_name, B, T, H, M, N, dtype)
    y, ST, grads, _ = run_gpu(op_name, xs, dy, dS)
    ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op_name], xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    tol_out, tol_grad = tolerances(dtype)
    assert y.dtype == dtype and ST.dtype == dtype
    assert O.rel_err(y, ry[0]) < tol_out
    assert O.rel_err(ST, rST[0]) < tol_out
    for g, r, x in zip(grads, rgx + rgs, xs):
        assert g.shape == x.shape and g.dtype == x.dtype
        assert O.rel_err(g, r) < tol_grad


def test_known_answer_norms():
    """L2 norms of every result at seed 0, B2 T64 H4 64x64, fp32 (recorded from
    the reference's naive; they depend on torch's CPU generator)."""
    import json
    norms = json.load(open(os.path.join(GOLDEN, "norms_c0.json")))
    for op_name, rec in norms.items():
        xs, dy, dS = O.make_case(op_name, dtype=torch.float32, **rec["shape"])
        y, ST, grads, _ = run_gpu(op_name, xs, dy, dS)
        got = [float(t.double().norm()) for t in [y, ST, *grads]]
        for a, b in zip(got, rec["norms"]):
            assert abs(a - b) <= 2e-5 * max(1.0, abs(b)), (op_name, got, rec["norms"])


def test_strided_views():
    """Non-contiguous inputs are read in place: q, k as slices of a fused
    projection, v and the state as .mT views (as the reference's examples pass
    them), beta expanded from a per-head value."""
    B, T, H, M, N = 2, 20, 2, 64, 64
    xs, dy, dS = O.make_case("delta_rule", B, T, H, M, N, torch.float32)
    q, k, v, beta, S0 = xs
    qk = torch.cat([q, k], dim=-1).to(DEV)                       # [B,T,H,1,2N]
    vT = v.transpose(-1, -2).contiguous().to(DEV)                # [B,T,H,1,M]
    S0T = S0.transpose(-1, -2).contiguous().to(DEV)              # [B,H,N,M]
    beta_d = beta.to(DEV)
    leaves = [qk.requires_grad_(), vT.requires_grad_(), beta_d.requires_grad_(), S0T.requires_grad_()]
    op = flex_rnn_b200.jit(O.delta_rule)
    y, ST = op(leaves[0][..., :N], leaves[0][..., N:], leaves[1].mT, leaves[2], leaves[3].mT)
    assert ST.stride() == leaves[3].mT.stride()
    grads = torch.autograd.grad([y, ST], leaves, [dy.to(DEV), dS.to(DEV)])
    ry, rST, rgx, rgs = O.fwd_bwd(O.delta_rule, xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < 1e-5 and O.rel_err(ST, rST[0]) < 1e-5
    assert O.rel_err(grads[0][..., :N], rgx[0]) < 1e-5
    assert O.rel_err(grads[0][..., N:], rgx[1]) < 1e-5
    assert O.rel_err(grads[1].mT, rgx[2]) < 1e-5
    assert O.rel_err(grads[2], rgx[3]) < 1e-5
    assert O.rel_err(grads[3].mT, rgs[0]) < 1e-5


def test_full_size_slices_and_split():
    """Benchmark configuration (Delta Rule, bf16, B8 T1024 H32 128x128): each
    (b,h) pair is an independent recurrence, so single (b,h) slices of the full
    result are checked against the oracle run on that slice alone; and running
    the two halves of the sequence back to back (state carried, upstream state
    gradient chained) must reproduce the one-pass results."""
    B, T, H, M, N = 8, 1024, 32, 128, 128
    g = torch.Generator().manual_seed(0)
    xs = [x.to(DEV) for x in O.make_inputs("delta_rule", B, T, H, M, N, torch.bfloat16, generator=g)]
    dy = torch.randn(B, T, H, M, generator=g).to(DEV).bfloat16()
    dS = torch.randn(B, H, M, N, generator=g).to(DEV).bfloat16()
    op = flex_rnn_b200.jit(O.delta_rule)
    leaves = [x.requires_grad_() for x in xs]
    y, ST = op(*leaves)
    grads = torch.autograd.grad([y, ST], leaves, [dy, dS])
    torch.cuda.synchronize()
    assert op.forward_func.kernel_status(DEV) == 0
    for (b, h) in [(0, 0), (3, 17), (7, 31)]:
        sl = [x.detach()[b:b + 1, :, h:h + 1].cpu() for x in xs[:-1]] + [xs[-1].detach()[b:b + 1, h:h + 1].cpu()]
        ry, rST, rgx, rgs = O.fwd_bwd(O.delta_rule, sl[:-1], sl[-1:], [dy[b:b + 1, :, h:h + 1].cpu().float()],
                                      [dS[b:b + 1, h:h + 1].cpu().float()], dtype=torch.float64)
        assert O.rel_err(y[b:b + 1, :, h:h + 1], ry[0]) < 5e-3
        assert O.rel_err(ST[b:b + 1, h:h + 1], rST[0]) < 5e-3
        for gi, r in zip(grads[:-1], rgx):
            assert O.rel_err(gi[b:b + 1, :, h:h + 1], r) < 1e-2
        assert O.rel_err(grads[-1][b:b + 1, h:h + 1], rgs[0]) < 1e-2
    # two halves chained == one pass (fp32 I/O so that the carried state is not re-rounded)
    B2, H2 = 2, 4
    xs32 = [x.detach()[:B2, :, :H2].float().contiguous() for x in xs[:-1]] + [xs[-1].detach()[:B2, :H2].float().contiguous()]
    dy32, dS32 = dy[:B2, :, :H2].float().contiguous(), dS[:B2, :H2].float().contiguous()
    l1 = [x.clone().requires_grad_() for x in xs32]
    y1, ST1 = op(*l1)
    g1 = torch.autograd.grad([y1, ST1], l1, [dy32, dS32])
    half = T // 2
    la = [x[:, :half].clone().requires_grad_() for x in xs32[:-1]] + [xs32[-1].clone().requires_grad_()]
    lb = [x[:, half:].clone().requires_grad_() for x in xs32[:-1]]
    ya, Sa = op(*la)
    yb, Sb = op(*lb, Sa)
    gall = torch.autograd.grad([ya, yb, Sb], la + lb, [dy32[:, :half], dy32[:, half:], dS32])
    assert O.rel_err(torch.cat([ya, yb], 1), y1) < 1e-5 and O.rel_err(Sb, ST1) < 1e-5
    n = len(xs32) - 1
    for i in range(n):
        assert O.rel_err(torch.cat([gall[i], gall[n + 1 + i]], 1), g1[i]) < 2e-5
    assert O.rel_err(gall[n], g1[n]) < 2e-5


def test_check_grad_and_torch_compile():
    """The user-facing check (compiled vs naive_fp64, tolerance 1e-2 as in the
    reference's check_grad) and the same op under torch.compile without a
    graph break."""
    xs, _, _ = O.make_case("rwkv7", 2, 32, 2, 64, 64, torch.float32)
    xs = [x.to(DEV) for x in xs]
    op = flex_rnn_b200.jit(O.rwkv7)
    err = flex_rnn_b200.check_grad(op, op.naive_fp64, xs, verbose=False)
    assert err < 1e-4
    compiled = torch.compile(lambda *z: op(*z), fullgraph=True)
    y0, S0 = op(*xs)
    y1, S1 = compiled(*xs)
    assert torch.equal(y0, y1) and torch.equal(S0, S1)
    leaves = [x.clone().requires_grad_() for x in xs]
    y, S = compiled(*leaves)
    g = torch.autograd.grad([y.sum(), S.sum()], leaves)
    leaves2 = [x.clone().requires_grad_() for x in xs]
    y2, S2 = op(*leaves2)
    g2 = torch.autograd.grad([y2.sum(), S2.sum()], leaves2)
    for a, b in zip(g, g2):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("op_name", ["delta_rule", "mamba2"])
def test_more_ctas_than_sms_small_state(op_name):
    """With more (b,h) pairs than SMs and a state small enough for a CTA of four
    warps the backward is built for two CTAs per SM (half the shared memory
    each); reverse re-step and recomputing mode.  Checked on a few (b,h) slices."""
    B, T, H, M, N = 5, 24, 32, 64, 64
    xs, dy, dS = O.make_case(op_name, B, T, H, M, N, torch.float32)
    y, ST, grads, op = run_gpu(op_name, xs, dy, dS)
    assert op.forward_func.plan.tuning.bw_min_blocks == 2
    for b, h in ((0, 0), (2, 17), (4, 31)):
        sl = [x[b:b + 1, :, h:h + 1] if x.shape[0] > 1 else x[:, :, h:h + 1] for x in xs[:-1]]
        ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op_name], sl, [xs[-1][b:b + 1, h:h + 1]], [dy[b:b + 1, :, h:h + 1]],
                                      [dS[b:b + 1, h:h + 1]], dtype=torch.float64)
        assert O.rel_err(y[b:b + 1, :, h:h + 1], ry[0]) < 1e-5 and O.rel_err(ST[b:b + 1, h:h + 1], rST[0]) < 1e-5
        for g, r, x in zip(grads, rgx + rgs, xs):
            if x.dim() == 5 and x.shape[0] == 1:
                continue                        # summed over the batch: not a per-slice quantity
            gs = g[b:b + 1, :, h:h + 1] if x.dim() == 5 else g[b:b + 1, h:h + 1]
            assert O.rel_err(gs, r) < 1e-5, (op_name, b, h)


def test_examples_cli_and_benchmark(capsys):
    """The user-facing tooling runs: the examples command line (as a fresh
    process, check mode: compiled op against naive_fp64 with the reference's
    1e-2 acceptance), its benchmark mode, and one direct ``benchmark()`` call."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "flex_rnn_b200.examples", "--op", "delta_rule", "--check-flex", "--seqlen", "64"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Verifying flex compiled kernel" in r.stdout and "Gradient rel. errors" in r.stdout
    from flex_rnn_b200 import examples
    examples.main(["--op", "hgrn", "--benchmark-flex", "--seqlen", "64", "--batchsz", "2", "--modeldim", "256"])
    out = capsys.readouterr().out
    assert "Benchmarking flex compiled kernel" in out and " ms (" in out and "memory" in out
    xs, _, _ = O.make_case("mamba2", 2, 32, 2, 64, 64, torch.float32)
    op = flex_rnn_b200.jit(O.mamba2)
    ms = flex_rnn_b200.benchmark(op, [x.to(DEV) for x in xs], warmup=2, rep=5, verbose=False)
    assert 0.0 < ms < 1e3


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,H", [(2, 0, 3), (0, 5, 3), (2, 5, 0)])
def test_empty_problems_launch_nothing(B, T, H):
    """No timestep, no batch row or no head: outputs are empty, the final state
    is the initial state, input gradients are zero (empty) and the gradient of
    the initial state is the upstream gradient of the final state; through the
    public API and autograd, without a kernel launch."""
    M, N = 64, 64
    op = flex_rnn_b200.jit(O.STEPS["gated_delta_rule"])
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g).to("cuda:0").requires_grad_()
    q, k, v, gate, beta, S = mk(B, T, H, 1, N), mk(B, T, H, 1, N), mk(B, T, H, M, 1), mk(B, T, H, 1, 1), mk(B, T, H, 1, 1), mk(B, H, M, N)
    y, ST = op(q, k, v, gate, beta, S)
    assert y.shape == (B, T, H, M) and ST.shape == S.shape and torch.equal(ST, S)
    dS = torch.randn(B, H, M, N, generator=g).to("cuda:0")
    grads = torch.autograd.grad([y, ST], [q, k, v, gate, beta, S], [torch.zeros_like(y), dS])
    assert all(gr.shape == x.shape and not gr.any() for gr, x in zip(grads[:-1], [q, k, v, gate, beta]))
    assert torch.equal(grads[-1], dS)
    assert op.forward_func.sources == () and op.forward_func.kernel_status("cuda:0") == 0


@pytest.mark.gpu
def test_mixed_and_fp64_io_dtypes():
    """Every tensor in its own I/O dtype (bf16, fp16, fp32 and fp64 in one call): the
    output takes the dtype torch's promotion gives the step, each gradient its
    input's, the arithmetic stays fp32 (the reference's contract, twopass.py:54-58,
    74-76, 175-180 of the reference project)."""
    B, T, H, M, N = 2, 37, 2, 64, 128
    xs, dy, dS = O.make_case("delta_rule", B, T, H, M, N, torch.float32)
    dts = [torch.bfloat16, torch.float16, torch.float64, torch.float32, torch.float32]     # q, k, v, beta, S
    xs = [x.to(d) for x, d in zip(xs, dts)]
    y, ST, grads, _ = run_gpu("delta_rule", xs, dy, dS)
    ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS["delta_rule"], xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    assert y.dtype == torch.float64 and ST.dtype == torch.float32          # v is fp64: the row sums promote to it
    assert O.rel_err(y, ry[0]) < 1e-5 and O.rel_err(ST, rST[0]) < 1e-5
    for g, r, x in zip(grads, rgx + rgs, xs):
        assert g.dtype == x.dtype and g.shape == x.shape
        assert O.rel_err(g, r) < (1e-2 if x.dtype in (torch.bfloat16, torch.float16) else 1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("op_name,M,N", [("delta_rule", 256, 256), ("gated_delta_rule", 256, 256), ("rwkv7", 256, 256),
                                         ("mamba2", 512, 128), ("delta_rule", 1024, 64), ("rwkv7", 128, 512),
                                         ("gated_delta_rule", 64, 1024)])
def test_states_larger_than_one_cta(op_name, M, N):
    """65 536 state elements per head: S and dS do not fit the registers of one SM,
    so the backward splits the rows of a head over several CTAs (the forward
    already tiles rows) and accumulates the per-column gradients across them."""
    B, T, H = 1, 20, 2
    xs, dy, dS = O.make_case(op_name, B, T, H, M, N, torch.float32)
    y, ST, grads, op = run_gpu(op_name, xs, dy, dS)
    assert op.forward_func.sources[1].grid[0] > 1
    ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op_name], xs[:-1], xs[-1:], [dy], [dS], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < 1e-5 and O.rel_err(ST, rST[0]) < 1e-5
    for g, r, x in zip(grads, rgx + rgs, xs):
        assert g.shape == x.shape and g.dtype == x.dtype
        assert O.rel_err(g, r) < 1e-5, (op_name, O.rel_err(g, r))
