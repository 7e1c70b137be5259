"""Tracing, graph slicing, planner metadata and the front-end wiring (CPU only)."""
import pytest
import torch

import flex_rnn_b200
from flex_rnn_b200 import examples as X
from flex_rnn_b200 import workloads as W
from flex_rnn_b200.graph import MN, M1, N1, S11, UnsupportedStepOp
from flex_rnn_b200.lower import LoweringError, choose_tile
from flex_rnn_b200.trace import trace_joint
from flex_rnn_b200.twopass import build_twopass, generate, make_plan, split_list, verify_meta


def metas(op, B, T, H, M, N, dtype=torch.bfloat16):
    xs, _, _ = W.synthetic(op, 2, 2, H, 4, 8, dtype)
    ins = []
    for x in xs[:-1]:
        shape = [B if x.shape[0] > 1 else 1, T if x.shape[1] > 1 else 1, H, M if x.shape[3] > 1 else 1, N if x.shape[4] > 1 else 1]
        ins.append(torch.empty(shape, dtype=dtype, device="meta"))
    return tuple(ins), (torch.empty(B, H, M, N, dtype=dtype, device="meta"),)


# per-element op counts of the joint graph ([M,N]-sized ops and sums of [M,N] operands)
@pytest.mark.parametrize("op,k_fwd,k_joint", [("delta_rule", 6, 18), ("gated_delta_rule", 7, 22), ("rwkv7", 9, 28),
                                              ("mamba2", 5, 16)])
def test_op_counts_and_slices(op, k_fwd, k_joint):
    ins, st = metas(op, 2, 16, 2, 32, 32)
    plan, fw_meta, bw_meta = make_plan(W.STEPS[op], ins, st)
    assert plan.k_fwd == k_fwd and plan.k_joint == k_joint
    # the re-step is reduction free, the forward has only sums over n, aux are row sums
    assert all(n.op != "sum" for n in plan.g_re.nodes)
    assert all(not n.over_m for n in plan.g_fw.nodes if n.op == "sum")
    assert len(plan.aux) == (0 if op == "mamba2" else 1)
    assert all(plan.joint.shape[a] == M1 for a in plan.aux)
    # declared metadata: y [B,T,H,M] in the step's dtype, states like S0, fp32 checkpoints and aux
    assert tuple(fw_meta[0][0]) == (2, 16, 2, 32) and fw_meta[0][2] == torch.bfloat16
    assert tuple(fw_meta[1][0]) == (2, 2, 32, 32)
    assert fw_meta[2][2] == torch.float32 and tuple(fw_meta[2][0]) == (2, 2, plan.nck, 32, 32)
    assert tuple(fw_meta[3][0]) == (len(plan.aux), 2, 2, 16, 32)
    assert [tuple(m[0]) for m in bw_meta[:-1]] == [tuple(i.shape) for i in ins]


def test_shape_classes():
    g, no, ns = trace_joint(W.mamba2, [M1, S11, S11, N1, N1, MN], 5)
    assert (no, ns) == (1, 1)
    assert [g.shape[i] for i in g.inputs[:6]] == [M1, S11, S11, N1, N1, MN]
    sums = [n for n in g.nodes if n.op == "sum"]
    assert any(n.over_m and n.over_n for n in sums)          # d(dt*A) sums over the whole tile
    assert any(n.over_m and not n.over_n for n in sums) and any(n.over_n and not n.over_m for n in sums)


def test_state_with_one_column():
    def hgrn(x, g, s):
        s = g.exp() * s + x
        return s, s
    B, T, H, M = 2, 8, 1, 64
    ins = (torch.empty(B, T, H, M, 1, device="meta"), torch.empty(B, T, H, M, 1, device="meta"))
    plan, fw_meta, _ = make_plan(hgrn, ins, (torch.empty(B, H, M, 1, device="meta"),))
    assert plan.problem.N == 1 and plan.aux == []
    fw, bw = generate(plan)
    assert "frnn_fw" in fw.source and "frnn_bw" in bw.source


def test_input_validation_messages():
    ins, st = metas("delta_rule", 2, 8, 2, 32, 32)
    bad = list(ins)
    bad[0] = torch.empty(2, 8, 2, 32, 32, dtype=torch.bfloat16, device="meta")
    with pytest.raises(AssertionError, match="both a matrix for each head, and depends on time"):
        make_plan(W.delta_rule, tuple(bad), st)
    with pytest.raises(AssertionError, match="incompatible"):
        make_plan(W.delta_rule, (torch.empty(2, 8, 2, 1, 7, device="meta"),) + ins[1:], st)
    with pytest.raises(AssertionError, match="invalid shape"):
        make_plan(W.delta_rule, (torch.empty(2, 8, 2, 32, device="meta"),) + ins[1:], st)
    with pytest.raises(AssertionError, match="!="):
        make_plan(W.delta_rule, ins, (torch.empty(2, 2, 32, 16, device="meta"),))

    def col_sum(q, S):
        S = S + q * S.sum(-2, True)
        return (S * q).sum(-1, True), S
    with pytest.raises(AssertionError, match="Only torch.sum"):
        make_plan(col_sum, (ins[0],), st)

    def unsupported(q, S):
        S = S + torch.cumsum(q, -1)
        return (S * q).sum(-1, True), S
    with pytest.raises(UnsupportedStepOp):
        make_plan(unsupported, (ins[0],), st)


def test_cpu_tensors_are_rejected_not_emulated():
    xs, _, _ = W.synthetic("delta_rule", 1, 4, 1, 32, 32, torch.float32)
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        build_twopass(W.delta_rule, tuple(xs[:-1]), (xs[-1],))
    op = flex_rnn_b200.jit(W.delta_rule)
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        op(*xs)


def test_dryrun_under_fake_mode():
    """What torch.compile does: the fake implementation asks for output
    metadata while a FakeTensorMode is active; nothing may touch CUDA."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    op = flex_rnn_b200.jit(W.rwkv7)
    assert (op.ninputs, op.nstates, op.noutputs) == (6, 1, 1)
    with FakeTensorMode():
        B, T, H, M, N = 2, 16, 2, 32, 32
        xs = [torch.empty(B, T, H, 1, N, dtype=torch.bfloat16) for _ in range(3)] + \
             [torch.empty(B, T, H, M, 1, dtype=torch.bfloat16)] + \
             [torch.empty(B, T, H, 1, N, dtype=torch.bfloat16) for _ in range(2)]
        xs = [xs[0], xs[1], xs[2], xs[3], xs[4], xs[5]]
        S0 = torch.empty(B, H, N, M, dtype=torch.bfloat16).mT
        y, ST = op(*xs, S0)
        assert y.shape == (B, T, H, M) and y.dtype == torch.bfloat16
        assert ST.shape == (B, H, M, N) and ST.stride() == S0.stride()


def test_naive_matches_simplified_naive():
    xs, _, _ = W.synthetic("gated_delta_rule", 2, 6, 2, 8, 8, torch.float32)
    op = flex_rnn_b200.jit(W.gated_delta_rule)
    y, ST = op.naive(*xs)
    y2, ST2 = flex_rnn_b200.simplified_naive(W.gated_delta_rule, *xs)
    assert torch.allclose(y, y2) and torch.allclose(ST, ST2)
    y64, _ = op.naive_fp64(*xs)
    assert y64.dtype == torch.float64 and torch.allclose(y64.float(), y, atol=1e-5)
    # the tests of the reference swap .apply for the naive callable; keep that working
    op.apply = op.naive_fp64
    assert op(*xs)[0].dtype == torch.float64


def test_helpers():
    assert split_list([1, 2, 3, 4], [1, 3]) == [[1], [2, 3, 4]]
    with pytest.raises(AssertionError):
        split_list([1, 2, 3], [1, 1])
    a = torch.empty(2, 1, 3)
    verify_meta([a], [torch.empty_strided((2, 1, 3), (3, 99, 1))])      # stride of a size-1 dim is ignored
    with pytest.raises(AssertionError):
        verify_meta([a], [torch.empty(2, 1, 3, dtype=torch.float64)])
    with pytest.raises(AssertionError):
        verify_meta([a], [torch.empty(3, 1, 2).transpose(0, 2)])


def test_tile_chooser():
    t = choose_tile(128, 128, 8, 8)
    assert (t.R, t.C, t.L, t.G, t.NT, t.RG) == (8, 8, 16, 2, 256, 16)
    t = choose_tile(128, 128, 4, 16, 32)
    assert (t.MB, t.NT) == (32, 64)
    t = choose_tile(64, 1, 4, 8)
    assert t.C == 1 and t.L == 1 and t.NT % 32 == 0
    with pytest.raises(LoweringError):
        choose_tile(4, 4, 1, 1)


def test_sizes_read_inside_the_step_are_the_real_ones():
    """A step that scales by its state's width must see the real width (the
    reference traces on the real per-head sizes, twopass.py:86-90)."""
    from emu.emu import EmuLauncher
    from flex_rnn_b200.twopass import Tuning, build_twopass
    from oracle import naive_oracle as O

    def step(q, k, v, S):
        S = S * 0.9 + v * k
        return (S * q).sum(-1, True) * S.shape[-1] ** -0.5 + S.shape[-2], S

    g = torch.Generator().manual_seed(0)
    n = lambda *s: torch.randn(*s, generator=g)
    B, T, H, M, N = 1, 5, 2, 8, 16
    ins, sts = (n(B, T, H, 1, N), n(B, T, H, 1, N), n(B, T, H, M, 1)), (n(B, H, M, N),)
    tu = Tuning(fw_r=2, fw_c=4, fw_mb=8, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2)
    fwd, _, _, _ = build_twopass(step, ins, sts, tuning=tu, _launcher=EmuLauncher)
    y = fwd(ins, sts)[0]
    ry, _, _, _ = O.fwd_bwd(step, list(ins), list(sts), [torch.zeros_like(y)], [torch.zeros_like(sts[0])], dtype=torch.float64)
    assert O.rel_err(y, ry[0]) < 1e-5


def test_dry_run_under_fake_tensors():
    """What a custom op's fake implementation does under torch.compile: plan on
    fake CUDA tensors (no GPU, no addresses), for an ordinary state and for one
    that is padded with repeated rows."""
    import warnings
    from torch._subclasses.fake_tensor import FakeTensorMode
    from flex_rnn_b200.twopass import build_twopass
    with FakeTensorMode(), warnings.catch_warnings():
        warnings.simplefilter("error")
        bf = dict(device="cuda", dtype=torch.bfloat16)
        q, v, b = torch.empty(2, 7, 3, 1, 16, **bf), torch.empty(2, 7, 3, 8, 1, **bf), torch.empty(2, 7, 3, 1, 1, **bf)
        fm, bm = build_twopass(W.delta_rule, (q, q, v, b), (torch.empty(2, 3, 8, 16, **bf),), dryrun=True)
        assert tuple(fm[0][0]) == (2, 7, 3, 8) and fm[0][2] == torch.bfloat16 and tuple(bm[-1][0]) == (2, 3, 8, 16)
        i = torch.empty(2, 7, 3, 1, 1, device="cuda")
        fm, bm = build_twopass(X.mlstm_gates, (i, i), (torch.empty(2, 3, 1, 1, device="cuda"),), dryrun=True)
        assert [tuple(m[0]) for m in fm[:4]] == [(2, 7, 3, 1)] * 3 + [(2, 3, 1, 1)]
        assert [tuple(m[0]) for m in bm] == [(2, 7, 3, 1, 1)] * 2 + [(2, 3, 1, 1)]


def test_backward_structure_at_benchmark_shapes():
    """What the planner builds for the benchmark workloads: helper warps (a warpgroup beside the tile's
    threads, registers rebalanced between the two), segment bases in Tensor Memory for the recomputing
    backward (four of them: 10 re-steps per 8 steps), the post-step state taken from the registers, and the
    reverse re-step without any of the recomputing machinery for the Delta Rule."""
    for op, (M, N) in (("delta_rule", (128, 128)), ("gated_delta_rule", (128, 128)), ("rwkv7", (128, 128)), ("mamba2", (64, 128))):
        ins, st = metas(op, 8, 1024, 32, M, N)
        plan, fw_meta, _ = make_plan(W.STEPS[op], ins, st)
        fw, bw = generate(plan)
        src = bw.source.split('extern "C"')[-1]
        assert bw.info["helper_warps"] == 4 and bw.block == bw.info["tile"][2] // bw.info["tile"][0] * (N // bw.info["tile"][1]) + 128
        assert "frnn_regs_release<" in src and "frnn_regs_acquire<" in src and "frnn_mbar_arrive(" in src
        assert "frnn_block_sync" not in src.split("frnn_block_sync();", 2)[-1]      # one block barrier, before the roles split
        if op == "delta_rule":
            assert plan.reverse is not None and bw.info["tmem_cols"] == 0 and not bw.info["post_split"]
            assert plan.D == 64 and plan.nck == 1024 // 64 + 1
        else:
            assert plan.reverse is None and bw.info["post_split"] and plan.post_split
            assert bw.info["tmem_cols"] == (512 if M == 128 else 256) and (bw.info["seg"], bw.info["nslots"]) == (2, 4)
            assert "frnn_tmem_alloc(" in src and "frnn_tmem_dealloc(" in src and "frnn_tmem_st<64>" in src
            assert plan.D == 8 and plan.nck == 1024 // 8 + 1                          # plus the final state
            assert tuple(fw_meta[2][0]) == (8, 32, plan.nck, M, N)
        assert bw.smem_bytes <= 227 * 1024


def test_product_reassociation():
    """(T * s) * y -> T * (s * y) and sum(a[M,1] * b[1,N]) -> vector * sum: same values, fewer full-tile ops."""
    from flex_rnn_b200.graph import Node, StepGraph
    g = StepGraph("t", ["T", "s", "y", "a", "b"], [
        Node("m1", "mul", ["T", "s"], MN), Node("m2", "mul", ["m1", "y"], MN), Node("r", "sum", ["m2"], N1, True, False),
        Node("o", "mul", ["a", "b"], MN), Node("q", "sum", ["o"], N1, True, False), Node("z", "add", ["r", "q"], N1)],
        ["z"], {"T": MN, "s": S11, "y": M1, "a": M1, "b": N1, "m1": MN, "m2": MN, "r": N1, "o": MN, "q": N1, "z": N1})
    h = g.simplified_products()
    assert g.count_mn_ops() == 5 and h.count_mn_ops() == 2
    vals = {"T": torch.randn(6, 5), "s": torch.randn(1, 1), "y": torch.randn(6, 1), "a": torch.randn(6, 1), "b": torch.randn(1, 5)}

    def run(graph):
        v = dict(vals)
        for n in graph.nodes:
            x = [v[a] for a in n.args]
            if n.op == "mul":
                v[n.name] = x[0] * x[1]
            elif n.op == "add":
                v[n.name] = x[0] + x[1]
            else:
                dims = [d for d, on in ((0, n.over_m), (1, n.over_n)) if on]
                v[n.name] = x[0].sum(dims, keepdim=True)
        return v[graph.outputs[0]]
    assert torch.allclose(run(g), run(h), rtol=1e-5, atol=1e-6)
    # a product with another use is left alone
    g2 = StepGraph("t", ["T", "s", "y"], [Node("m1", "mul", ["T", "s"], MN), Node("m2", "mul", ["m1", "y"], MN),
                                          Node("k", "add", ["m1", "m2"], MN)], ["k"],
                   {"T": MN, "s": S11, "y": M1, "m1": MN, "m2": MN, "k": MN})
    assert [n.name for n in g2.simplified_products().nodes] == ["m1", "m2", "k"]


@pytest.mark.parametrize("B,T,H", [(1, 0, 2), (0, 4, 2), (2, 3, 0)])
def test_empty_problems_build_no_kernel(B, T, H):
    """A problem without a timestep, a batch row or a head gets host closures that launch nothing (the launcher
    seam given here would raise if it were ever constructed)."""
    import torch
    from flex_rnn_b200.twopass import build_twopass
    from oracle import naive_oracle as O

    def never(ks):
        raise AssertionError("a kernel was built for an empty problem")

    q, k = torch.randn(B, T, H, 1, 16), torch.randn(B, T, H, 1, 16)
    v, beta, S = torch.randn(B, T, H, 16, 1), torch.rand(B, T, H, 1, 1), torch.randn(B, H, 16, 16)
    fwd, bwd, fm, bm = build_twopass(O.STEPS["delta_rule"], (q, k, v, beta), (S,), _launcher=never)
    y, ST, store, aux = fwd((q, k, v, beta), (S,))
    assert tuple(y.shape) == (B, T, H, 16) and torch.equal(ST, S)
    assert [tuple(m[0]) for m in fm] == [tuple(t.shape) for t in (y, ST, store, aux)]
    dS = torch.randn(B, H, 16, 16)
    dx, ds0 = bwd((torch.zeros_like(y),), (dS,), (q, k, v, beta), (store,), (aux,))
    assert [tuple(d.shape) for d in dx] == [tuple(x.shape) for x in (q, k, v, beta)] and torch.equal(ds0[0], dS)
