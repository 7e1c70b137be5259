"""Parity at the benchmark's full sizes, through the public ``jit`` API, so that
the kernels under test are the ones the benchmark times: at these sizes the
first call autotunes (alternative tilings are timed and the fastest kept).

Each (batch, head) pair is an independent recurrence, so single (b,h) slices of
the full result are compared with the CPU oracle run in fp64 on that slice
alone (relative L2 as in the reference's check_grad; bf16 I/O: 5e-3 on outputs
and final state, 1e-2 on gradients).  The reference's own acceptance is the
same comparison at its check size (tests/examples.py:447-454 of the reference
project).  Gradients of inputs shared by several slices (Mamba-2's per-head
``A``) are compared on a whole head.
"""
import pytest
import torch

import flex_rnn_b200
from oracle import naive_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

FULL = [
    # op, B, T, H, M, N, (b,h) slices
    ("rwkv7", 8, 1024, 32, 128, 128, [(0, 0), (3, 17), (7, 31)]),
    ("mamba2", 8, 1024, 32, 64, 128, [(0, 0), (4, 9), (7, 31)]),
    ("gated_delta_rule", 8, 1024, 32, 128, 128, [(0, 0), (5, 20), (7, 31)]),
    # one GPU's share of the scaling configuration (global batch 64 over 8 GPUs)
    ("gated_delta_rule", 8, 4096, 32, 128, 128, [(0, 0), (6, 13), (7, 31)]),
]


def _slice(x, b, h):
    if x.dim() == 4:
        return x[b:b + 1, h:h + 1]
    bs = slice(b, b + 1) if x.shape[0] > 1 else slice(None)
    hs = slice(h, h + 1) if x.shape[2] > 1 else slice(None)
    return x[bs, :, hs]


@pytest.mark.parametrize("op_name,B,T,H,M,N,slices", FULL, ids=[f"{c[0]}-T{c[2]}" for c in FULL])
def test_full_size_slices(op_name, B, T, H, M, N, slices):
    g = torch.Generator().manual_seed(0)
    xs_cpu = O.make_inputs(op_name, B, T, H, M, N, torch.bfloat16, generator=g)
    dy_cpu = torch.randn(B, T, H, M, generator=g).bfloat16()
    dS_cpu = torch.randn(B, H, M, N, generator=g).bfloat16()
    op = flex_rnn_b200.jit(O.STEPS[op_name])
    leaves = [x.to(DEV).requires_grad_() for x in xs_cpu]
    y, ST = op(*leaves)
    grads = torch.autograd.grad([y, ST], leaves, [dy_cpu.to(DEV), dS_cpu.to(DEV)])
    torch.cuda.synchronize()
    fwd = op.forward_func
    assert fwd.kernel_status(DEV) == 0
    # the kernels that ran are the autotuner's picks; say which, and that they were picked by timing
    tuned = fwd.tuned
    assert len(tuned["fw_log"]) >= 2 and len(tuned["bw_log"]) >= 2, "autotuning did not run at benchmark size"
    print(f"[full size] {op_name} T={T}: forward variant {tuned['fw_choice']} {fwd.sources[0].info['tile']} "
          f"packed={fwd.sources[0].info['packed']} of {tuned['fw_log']}; backward variant {tuned['bw_choice']} "
          f"{fwd.sources[1].info['tile']} of {tuned['bw_log']}")
    y, ST, grads = y.cpu(), ST.cpu(), [gr.cpu() for gr in grads]
    for (b, h) in slices:
        sl = [_slice(x, b, h) for x in xs_cpu]
        ry, rST, rgx, rgs = O.fwd_bwd(O.STEPS[op_name], sl[:-1], sl[-1:], [_slice(dy_cpu.unsqueeze(-1), b, h).squeeze(-1).float()],
                                      [_slice(dS_cpu, b, h).float()], dtype=torch.float64)
        assert O.rel_err(_slice(y.unsqueeze(-1), b, h).squeeze(-1), ry[0]) < 5e-3, (op_name, b, h)
        assert O.rel_err(_slice(ST, b, h), rST[0]) < 5e-3, (op_name, b, h)
        for gi, r, x in zip(grads, rgx + rgs, xs_cpu):
            if x.dim() == 5 and (x.shape[0] == 1 or x.shape[1] == 1):
                continue                       # summed over the batch or over time: checked on a whole head below
            assert O.rel_err(_slice(gi, b, h), r) < 1e-2, (op_name, b, h, O.rel_err(_slice(gi, b, h), r))
    shared = [i for i, x in enumerate(xs_cpu[:-1]) if x.shape[0] == 1 or x.shape[1] == 1]
    if shared:
        # all batch elements of one head: the gradient of a per-head input sums over them
        # (fp64 leaves holding the same bf16 values: autograd would otherwise add the per-step contributions
        # to a bf16 leaf in bf16, which is good to a few per cent only over 8192 terms)
        h = slices[1][1]
        sl = [(x[:, :, h:h + 1] if x.dim() == 5 else x[:, h:h + 1]).double() for x in xs_cpu]
        _, _, rgx, _ = O.fwd_bwd(O.STEPS[op_name], sl[:-1], sl[-1:], [dy_cpu[:, :, h:h + 1].double()],
                                 [dS_cpu[:, h:h + 1].double()], dtype=torch.float64)
        for i in shared:
            assert O.rel_err(grads[i][:, :, h:h + 1], rgx[i]) < 1e-2, (op_name, "shared input", i)
