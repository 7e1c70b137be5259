"""Bundled example step functions and a command line driver over them, in the
spirit of the reference's tests/examples.py (modes --check-flex,
--benchmark-flex, --torch-compile, --forward; the comparisons with third-party
kernels are not reproduced).

    python -m flex_rnn_b200.examples --op rwkv7 --check-flex
    python -m flex_rnn_b200.examples --op delta_rule --benchmark-flex

Besides the four benchmark steps (``workloads.py``) it carries the other step
families of the reference's example script, written on ``[B,T,H,M|1,N|1]``
inputs directly: a step function *is* the workload's definition, so these
follow the reference's expressions (tests/examples.py of the reference
project: RWKV-6 :73-77, GLA :96-99, Retention :117-121, Longhorn :215-220,
RWKV-4 :241-255, HGRN :274-277, Mamba :298-301, S4D :324-329, the mLSTM gate
recurrence :398-404).  ``zoo_case`` draws small synthetic arguments for each of
them; the parity tests use it.
"""
import argparse

import torch
import torch as th

import flex_rnn_b200
from flex_rnn_b200 import workloads as W


def rwkv6(q, k, v, w, u, S):
    y = ((S + v * (u * k)) * q).sum(-1, True)
    S = S * w.exp() + v * k
    return y, S


def gla(q, k, v, g, S):
    S = S * g.exp() + v * k
    return (S * q).sum(-1, True), S


def retention(w, q, k, v, S):
    S = w * S + v * k
    return (S * q).sum(-1, True), S


def longhorn(u, q, k, dt, S):
    k2 = k * k
    dt = 1 / (1 + (-dt).exp() + k2.sum(-1, True))
    S = S - dt * S * k2 + dt * u * k
    return (S * q).sum(-1, True), S


def rwkv4(w, u, k, v, sa, sb, sc):
    x = k + u - sc
    A = (-x * (x > 0)).exp()
    B = (x * (x < 0)).exp()
    y = (A * sa + B * v) / (A * sb + B)
    w = -w.exp()
    x = k - w - sc
    A = (-x * (x > 0)).exp()
    B = (x * (x < 0)).exp()
    return y, (A * sa + B * v, A * sb + B, k - x * (x < 0))


def hgrn(x, g, s):
    s = g.exp() * s + x
    return s, s


def mamba(u, dt, A, b, c, S):
    S = (dt * A).exp() * S + (dt * u) * b
    return (S * c).sum(-1, True), S


def s4d(u, Ar, Ai, Qr, Qi, D, Sr, Si):
    Sr_ = Ar * Sr - Ai * Si + u
    Si_ = Ar * Si + Ai * Sr
    y = torch.sum(Sr_ * Qr - Si_ * Qi, dim=-1, keepdim=True) + D * u
    return y, (Sr_, Si_)


def mlstm_gates(i, f, sc):
    f = -torch.log(1 + torch.exp(-f))
    m = f + sc
    sc_ = m + (i - m) * (i > m).float()
    return ((i - sc_).exp(), (f + sc - sc_).exp(), sc_), sc_


ZOO = {"rwkv6": rwkv6, "gla": gla, "retention": retention, "longhorn": longhorn, "rwkv4": rwkv4, "hgrn": hgrn,
       "mamba": mamba, "s4d": s4d, "mlstm_gates": mlstm_gates}


def zoo_case(op: str, B: int, T: int, H: int, M: int, N: int, dtype=torch.float32, seed: int = 0):
    """(inputs, states) of a step family of ``ZOO`` at the given sizes."""
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g)
    row, col, sc = (lambda: n(B, T, H, 1, N)), (lambda: n(B, T, H, M, 1)), (lambda: n(B, T, H, 1, 1))
    if op == "rwkv6":
        ins = [row(), row(), col(), -torch.sigmoid(row()), n(1, 1, H, 1, N)]
        sts = [n(B, H, M, N)]
    elif op == "gla":
        ins = [row(), row(), col(), -torch.sigmoid(row())]
        sts = [n(B, H, M, N)]
    elif op == "retention":
        w = (1 - 2.0 ** (-5 - torch.arange(H).float())).view(1, 1, H, 1, 1).expand(B, T, H, 1, 1).contiguous()
        ins = [w, row(), row(), col()]
        sts = [n(B, H, M, N)]
    elif op == "longhorn":
        ins = [col(), row(), row(), col()]
        sts = [torch.zeros(B, H, M, N)]
    elif op == "rwkv4":
        s = n(B, 3, H, M, 1)
        s[:, 2] = -1e30
        ins = [n(1, 1, H, M, 1), n(1, 1, H, M, 1), col(), col()]
        sts = [s[:, 0].contiguous(), s[:, 1].contiguous(), s[:, 2].contiguous()]
    elif op == "hgrn":
        ins = [col(), -torch.sigmoid(col())]
        sts = [torch.zeros(B, H, M, 1)]
    elif op == "mamba":
        ins = [col(), torch.sigmoid(col()), -torch.sigmoid(n(1, 1, H, M, N)), row(), row()]
        sts = [torch.zeros(B, H, M, N)]
    elif op == "s4d":
        # |Ar + i Ai| < 1: a stable (decaying) diagonal system
        ins = [col(), 0.65 * torch.rand(1, 1, H, M, N, generator=g), 0.65 * torch.rand(1, 1, H, M, N, generator=g),
               n(1, 1, H, M, N), n(1, 1, H, M, N), n(1, 1, H, M, 1)]
        sts = [torch.zeros(B, H, M, N), torch.zeros(B, H, M, N)]
    elif op == "mlstm_gates":
        ins = [sc(), sc()]
        sts = [n(B, H, 1, 1)]
    else:
        raise KeyError(op)
    return [x.to(dtype) for x in ins], [s.to(dtype) for s in sts]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ops = list(W.STEPS) + list(ZOO)
    ap.add_argument("--op", default="rwkv7", choices=ops)
    ap.add_argument("--batchsz", type=int, default=8)
    ap.add_argument("--modeldim", type=int, default=None)
    ap.add_argument("--headsz", type=int, default=128)
    ap.add_argument("--seqlen", type=int, default=None)
    ap.add_argument("--benchmark-flex", action="store_true")
    ap.add_argument("--check-flex", action="store_true")
    ap.add_argument("--torch-compile", action="store_true")
    ap.add_argument("--forward", action="store_true")
    a = ap.parse_args(argv)
    check = a.check_flex or not a.benchmark_flex
    modeldim = a.modeldim or (256 if check else 4096)
    T = a.seqlen or (256 if check else 1024)
    B, C = a.batchsz, a.headsz
    H = modeldim // C
    dev = "cuda"
    print("Testing", a.op)
    print(f"Input sizes B={B}, T={T}, H={H}, C={C}")
    dtype = th.float32 if check or a.op in ("s4d", "mamba") else th.bfloat16
    if a.op in W.STEPS:
        xs, _, _ = W.synthetic(a.op, B, T, H, 64 if a.op == "mamba2" else C, C, dtype)
        step_fn, nst = W.STEPS[a.op], 1
    else:
        M, N = (modeldim, 1) if a.op in ("rwkv4", "hgrn") else (1, 1) if a.op == "mlstm_gates" else (C, 16 if a.op == "mamba" else C)
        Hh = 1 if a.op in ("rwkv4", "hgrn") else H
        ins, sts = zoo_case(a.op, B, T, Hh, M, N, dtype)
        xs, step_fn, nst = ins + sts, ZOO[a.op], len(sts)
    xs = [x.to(dev) for x in xs]
    op = flex_rnn_b200.jit(step_fn)
    flex = th.compile(lambda *z: op(*z)) if a.torch_compile else op
    if check:
        print("Verifying flex compiled kernel")
        flex_rnn_b200.check_grad(flex, op.naive_fp64, xs, backward=not a.forward)
    else:
        print("Benchmarking flex compiled kernel")
        flex_rnn_b200.benchmark(flex, xs, backward=not a.forward)


if __name__ == "__main__":
    main()
