"""CPU oracle for the recurrent hot path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module; the library
(``flex_rnn_b200/``) never does.

It restates, in plain PyTorch on the CPU, the semantics the reference defines
for a compiled step function:

* ``scan``        - the time loop of ``jit.naive`` (reference project,
                    flex_rnn/jit.py:23-36): inputs ``[B,T,H,M|1,N|1]`` are
                    expanded over T, sliced per step, cast to the compute
                    dtype, fed to the step with the running state(s); outputs
                    are stacked to ``[B,T,H,M]``; the final state is copied
                    into a tensor shaped and typed like the initial state.
* ``fwd_bwd``     - forward plus ``torch.autograd.grad`` with given upstream
                    gradients, which is how the reference's own check compares
                    implementations (flex_rnn/check_grad.py:12-44).
* ``rel_err``     - the relative L2 error of flex_rnn/check_grad.py:20.
* the four step functions of the benchmark configurations, written out
  explicitly (Delta Rule, Gated Delta Rule, RWKV-7, Mamba-2), and the seeded
  input generators for them.

Parity pin: ``tests/golden/*.pt`` hold outputs and gradients produced by the
reference's own ``flex_rnn.jit(step).naive`` (imported from the reference
checkout by ``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks
this restatement against them and against the known-answer norms recorded for
the seed-0 configuration.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# step functions (one timestep; per-head tiles broadcast as [B,H,M|1,N|1])
# --------------------------------------------------------------------------

def delta_rule(q, k, v, beta, S):
    S = S + beta * k * (v - (S * k).sum(-1, True))
    return (S * q).sum(-1, True), S


def gated_delta_rule(q, k, v, g, beta, S):
    S = S * g
    S = S + beta * k * (v - (S * k).sum(-1, True))
    return (S * q).sum(-1, True), S


def rwkv7(q, w, k, v, a, b, S):
    S = S * w + (S * a).sum(-1, True) * b + v * k
    return (S * q).sum(-1, True), S


def mamba2(x, dt, A, Bm, C, S):
    S = S * torch.exp(dt * A) + dt * x * Bm
    return (S * C).sum(-1, True), S


STEPS: Dict[str, Callable] = {"delta_rule": delta_rule, "gated_delta_rule": gated_delta_rule,
                              "rwkv7": rwkv7, "mamba2": mamba2}
N_STATES = 1


# --------------------------------------------------------------------------
# seeded inputs (CPU generator, fp32 draws in a fixed order, then cast)
# --------------------------------------------------------------------------

def make_inputs(op: str, B: int, T: int, H: int, M: int, N: int, dtype=torch.float32, seed: int = 0,
                generator: torch.Generator = None) -> List[torch.Tensor]:
    """Inputs followed by the initial state, distributions as the benchmark
    configurations state them (N(a,b) = mean a, std b)."""
    g = generator or torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    if op == "delta_rule":
        q = F.normalize(r(B, T, H, 1, N), dim=-1)
        k = F.normalize(r(B, T, H, 1, N), dim=-1)
        v = r(B, T, H, M, 1)
        beta = torch.sigmoid(r(B, T, H, 1, 1))
        S0 = r(B, H, M, N) * 0.1
        xs = [q, k, v, beta, S0]
    elif op == "gated_delta_rule":
        q = F.normalize(r(B, T, H, 1, N), dim=-1)
        k = F.normalize(r(B, T, H, 1, N), dim=-1)
        v = r(B, T, H, M, 1)
        gate = torch.exp(-F.softplus(r(B, T, H, 1, 1)))
        beta = torch.sigmoid(r(B, T, H, 1, 1))
        S0 = r(B, H, M, N) * 0.1
        xs = [q, k, v, gate, beta, S0]
    elif op == "rwkv7":
        q = r(B, T, H, 1, N) / N ** 0.5
        w = torch.exp(-torch.exp(-0.5 + 0.5 * r(B, T, H, 1, N)))
        k = r(B, T, H, 1, N) / N ** 0.5
        v = r(B, T, H, M, 1)
        kk = F.normalize(r(B, T, H, 1, N), dim=-1)
        a = -kk
        b = kk * torch.sigmoid(r(B, T, H, 1, N))
        S0 = r(B, H, M, N) * 0.1
        xs = [q, w, k, v, a, b, S0]
    elif op == "mamba2":
        x = r(B, T, H, M, 1)
        dt = F.softplus(-1 + r(B, T, H, 1, 1))
        A = -torch.exp(r(1, 1, H, 1, 1))
        Bm = r(B, T, H, 1, N) / N ** 0.5
        C = r(B, T, H, 1, N) / N ** 0.5
        S0 = torch.zeros(B, H, M, N)
        xs = [x, dt, A, Bm, C, S0]
    else:
        raise KeyError(op)
    return [t.to(dtype) for t in xs]


def make_case(op: str, B: int, T: int, H: int, M: int, N: int, dtype=torch.float32, seed: int = 0):
    """(inputs + [S0], dy[B,T,H,M], dS[B,H,M,N]) drawn, in this order, from one
    CPU generator seeded with ``seed``: the inputs, then the upstream gradient
    of the output, then that of the final state (both N(0,1), kept in fp32)."""
    g = torch.Generator().manual_seed(seed)
    xs = make_inputs(op, B, T, H, M, N, dtype, generator=g)
    dy = torch.randn(B, T, H, M, generator=g)
    dS = torch.randn(B, H, M, N, generator=g)
    return xs, dy, dS


# --------------------------------------------------------------------------
# the scan and its gradients
# --------------------------------------------------------------------------

def scan(step: Callable, inputs: Sequence[torch.Tensor], states: Sequence[torch.Tensor],
         dtype=torch.float32) -> Tuple[Tuple[torch.Tensor, ...], Tuple[torch.Tensor, ...]]:
    T = max(x.shape[1] for x in inputs)
    cur = tuple(states)
    ys = None
    for t in range(T):
        x_t = [x.expand(-1, T, -1, -1, -1)[:, t].to(dtype) for x in inputs]
        y, cur = step(*x_t, *cur)
        y = y if isinstance(y, tuple) else (y,)
        cur = cur if isinstance(cur, tuple) else (cur,)
        if ys is None:
            ys = [[] for _ in y]
        for acc, v in zip(ys, y):
            acc.append(v.squeeze(-1))
    outs = tuple(torch.stack(a, dim=1) for a in ys)
    finals = tuple(torch.empty_like(s0).copy_(s) for s0, s in zip(states, cur))
    return outs, finals


def fwd_bwd(step: Callable, inputs, states, d_outs, d_states, dtype=torch.float32):
    """Returns (outputs, final_states, input_grads, state_grads)."""
    xs = [x.detach().clone().requires_grad_() for x in inputs]
    ss = [s.detach().clone().requires_grad_() for s in states]
    outs, finals = scan(step, xs, ss, dtype)
    ups = [d.to(o.dtype) for d, o in zip(d_outs, outs)] + [d.to(f.dtype) for d, f in zip(d_states, finals)]
    grads = torch.autograd.grad(list(outs) + list(finals), xs + ss, ups, allow_unused=True)
    grads = [g if g is not None else torch.zeros_like(p) for g, p in zip(grads, xs + ss)]
    return ([o.detach() for o in outs], [f.detach() for f in finals],
            grads[:len(xs)], grads[len(xs):])


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / max(float(b.norm()), 1e-30))
