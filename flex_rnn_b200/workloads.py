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


def synthetic(op: str, B: int, T: int, H: int, M: int, N: int, dtype=torch.bfloat16, seed: int = 0, device="cpu"):
    """(inputs + [initial state], d_output [B,T,H,M], d_final_state [B,H,M,N]).

    Drawn on the CPU generator by default (every device then sees identical
    values); ``device`` draws on that device's generator instead, for sizes
    that are too large to draw on the host (the scaling configuration)."""
    g = torch.Generator(device=device).manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g, device=device)
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
              n(B, T, H, 1, N) * N ** -0.5, n(B, T, H, 1, N) * N ** -0.5, torch.zeros(B, H, M, N, device=device)]
    else:
        raise KeyError(op)
    dy = n(B, T, H, M)
    dS = n(B, H, M, N)
    return [x.to(dtype) for x in xs], dy.to(dtype), dS.to(dtype)
