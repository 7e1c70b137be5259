"""Parity and timing helpers for users of ``@jit`` (the counterparts of the
reference's flex_rnn/check_grad.py:12-67: same relative-L2 metric, same
acceptance threshold, same "median of many runs" timing — measured here with
CUDA events instead of triton's ``do_bench``)."""
from __future__ import annotations

from typing import Callable, Sequence

import torch as th


def _detached_like(x: th.Tensor) -> th.Tensor:
    out = th.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    out.copy_(x)
    return out


def rel(a: th.Tensor, b: th.Tensor) -> float:
    """||a - b|| / max(||b||, 1e-30), the metric of the reference's check_grad."""
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / max(float(b.norm()), 1e-30))


def check_grad(f1: Callable, f2: Callable, inputs: Sequence[th.Tensor], backward: bool = True, aux=(),
               tol: float = 1e-2, verbose: bool = True):
    """Compare outputs and input gradients of ``f1`` and ``f2`` on the same
    arguments and shared random upstream gradients; raises if any relative
    error reaches ``tol``.  Returns the largest error."""
    xs = [_detached_like(p) for p in inputs]
    if backward:
        xs = [p.requires_grad_() for p in xs]
    y1, y2 = f1(*xs, *aux), f2(*xs, *aux)
    y1 = y1 if isinstance(y1, tuple) else (y1,)
    y2 = y2 if isinstance(y2, tuple) else (y2,)
    worst = 0.0
    if verbose:
        print("Forward rel. errors")
    for a, b in zip(y1, y2):
        assert a.shape == b.shape, f"shape mismatch {tuple(a.shape)} vs {tuple(b.shape)}"
        e = rel(a, b)
        worst = max(worst, e)
        if verbose:
            print(f"{e:.2e}  ({float(b.detach().double().norm()):.0e})")
    if not backward:
        assert worst < tol, f"Large check error: {worst * 100:.1f}%!"
        return worst
    ups = tuple(th.randn_like(o) for o in y1)
    g1 = th.autograd.grad(y1, xs, grad_outputs=tuple(_detached_like(u) for u in ups), allow_unused=True)
    g2 = th.autograd.grad(y2, xs, grad_outputs=tuple(u.to(o.dtype) for u, o in zip(ups, y2)), allow_unused=True)
    if verbose:
        print("Gradient rel. errors")
    for a, b, x in zip(g1, g2, xs):
        a = th.zeros_like(x) if a is None else a
        b = th.zeros_like(x) if b is None else b
        e = rel(a, b)
        worst = max(worst, e)
        if verbose:
            print(f"{e:.2e}  ({float(b.detach().double().norm()):.0e})")
    assert worst < tol, f"Large grad_check error: {worst * 100:.1f}%!"
    return worst


def benchmark(f: Callable, params: Sequence[th.Tensor], backward: bool = True, aux=(), warmup: int = 10,
              rep: int = 50, verbose: bool = True) -> float:
    """Median milliseconds of ``f`` (plus backward) and its peak memory."""
    if backward:
        for p in params:
            p.requires_grad_()
    ups = None

    def once():
        nonlocal ups
        y = f(*params, *aux)
        if not backward:
            return
        y = y if isinstance(y, tuple) else (y,)
        if ups is None:
            ups = tuple(th.randn_like(o) for o in y)
        th.autograd.grad(y, params, grad_outputs=ups, allow_unused=True)

    once()
    th.cuda.synchronize()
    th.cuda.reset_peak_memory_stats()
    once()
    th.cuda.synchronize()
    mem = th.cuda.max_memory_allocated() / 2 ** 30
    for _ in range(warmup):
        once()
    times = []
    for _ in range(rep):
        e0, e1 = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        e0.record()
        once()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    med, lo, hi = times[len(times) // 2], times[len(times) // 5], times[4 * len(times) // 5]
    if verbose:
        print(f"memory {mem:.2f} GB")
        print(f"{med:.2f} ms ({lo:.2f} - {hi:.2f})")
    return med
