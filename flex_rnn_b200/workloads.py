"""The benchmark step functions and their synthetic inputs.

Step functions are written the way a user of ``@jit`` writes them (compare the
examples of the reference project, tests/examples.py:50-53, 141-144, 165-169,
191-194); the input distributions are the ones the benchmark configurations
state, drawn on a CPU generator so that every device sees identical values.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


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


STEPS = {"delta_rule": delta_rule, "gated_delta_rule": gated_delta_rule, "rwkv7": rwkv7, "mamba2": mamba2}

#: name -> (B, T, H, M, N) of the benchmark configurations
CONFIGS = {
    "delta_rule": (8, 1024, 32, 128, 128),
    "rwkv7": (8, 1024, 32, 128, 128),
    "mamba2": (8, 1024, 32, 64, 128),
    "gated_delta_rule": (64, 4096, 32, 128, 128),
}


def synthetic(op: str, B: int, T: int, H: int, M: int, N: int, dtype=torch.bfloat16, seed: int = 0):
    """(inputs + [initial state], d_output [B,T,H,M], d_final_state [B,H,M,N])."""
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g)
    unit = lambda x: F.normalize(x, dim=-1)
    if op == "delta_rule":
        xs = [unit(n(B, T, H, 1, N)), unit(n(B, T, H, 1, N)), n(B, T, H, M, 1), torch.sigmoid(n(B, T, H, 1, 1)),
              0.1 * n(B, H, M, N)]
    elif op == "gated_delta_rule":
        xs = [unit(n(B, T, H, 1, N)), unit(n(B, T, H, 1, N)), n(B, T, H, M, 1), torch.exp(-F.softplus(n(B, T, H, 1, 1))),
              torch.sigmoid(n(B, T, H, 1, 1)), 0.1 * n(B, H, M, N)]
    elif op == "rwkv7":
        q = n(B, T, H, 1, N) * N ** -0.5
        w = torch.exp(-torch.exp(0.5 * n(B, T, H, 1, N) - 0.5))
        k = n(B, T, H, 1, N) * N ** -0.5
        v = n(B, T, H, M, 1)
        kk = unit(n(B, T, H, 1, N))
        xs = [q, w, k, v, -kk, kk * torch.sigmoid(n(B, T, H, 1, N)), 0.1 * n(B, H, M, N)]
    elif op == "mamba2":
        xs = [n(B, T, H, M, 1), F.softplus(n(B, T, H, 1, 1) - 1.0), -torch.exp(n(1, 1, H, 1, 1)),
              n(B, T, H, 1, N) * N ** -0.5, n(B, T, H, 1, N) * N ** -0.5, torch.zeros(B, H, M, N)]
    else:
        raise KeyError(op)
    dy = n(B, T, H, M)
    dS = n(B, H, M, N)
    return [x.to(dtype) for x in xs], dy.to(dtype), dS.to(dtype)


# ---------------------------------------------------------------------------
# Further step families (the other examples of the reference's tests/examples.py,
# written on [B,T,H,M|1,N|1] inputs directly).  ``zoo_case`` draws small
# synthetic arguments for each of them; used by the parity tests.
# ---------------------------------------------------------------------------

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
