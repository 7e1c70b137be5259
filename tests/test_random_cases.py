"""Randomised cases for the code generator, run on the CPU through the host
emulation of the generated kernels and checked against the naive scan in fp64.

Each seed draws a step family, state sizes (including one-row, one-column,
1x1 and non-power-of-two states), B/T/H (T not a multiple of any stage
length), broadcasting over batch / time / heads, I/O dtype (fp32, bf16, fp16,
fp64; the arithmetic is fp32 throughout), memory layouts
(strided last dimension, odd storage offsets, time-major inputs, transposed
states) and tiling parameters.  The emulation aborts on any vector access or
bulk copy that the GPU would reject as misaligned, so a pass also means that
the alignment guards of the planner hold for that layout.
"""
import random

import pytest
import torch

from flex_rnn_b200 import lower
from flex_rnn_b200 import examples as X
from flex_rnn_b200 import workloads as W
from flex_rnn_b200.twopass import Tuning, build_twopass
from oracle import naive_oracle as O


def two_outputs(q, k, v, w, S):
    S = S * w + v * k
    return ((S * q).sum(-1, True), (S * k).sum(-1, True) * v), S


def two_states(q, k, v, w, S, Z):
    S = S * w + v * k
    Z = Z * w + k
    return (S * q).sum(-1, True) / (1 + (Z * q).sum(-1, True) ** 2), (S, Z)


def column_gate(q, k, v, S):
    S = S * torch.sigmoid(v) + k
    return (S * q).sum(-1, True), S


FAMILIES = ["delta", "gated", "rwkv7", "mamba2", "gla", "retention", "hgrn", "two_outputs", "two_states", "column_gate"]


def draw_case(rng: random.Random):
    fam = rng.choice(FAMILIES)
    M = rng.choice([1, 2, 4, 8, 16, 32, 64])
    N = rng.choice([1, 2, 4, 8, 16, 32, 64, 12, 24])
    B, H, T = rng.choice([1, 2, 3]), rng.choice([1, 2, 3]), rng.choice([1, 2, 3, 5, 8, 9, 16, 17, 23])
    g = torch.Generator().manual_seed(rng.randrange(1 << 30))
    n = lambda *s: torch.randn(*s, generator=g)

    def bc(shape):                      # broadcast some of batch / time / heads
        return [1 if d < 3 and rng.random() < 0.15 else s for d, s in enumerate(shape)]
    row, col, sc = (lambda: n(*bc([B, T, H, 1, N]))), (lambda: n(*bc([B, T, H, M, 1]))), (lambda: n(*bc([B, T, H, 1, 1])))
    unit = lambda x: x / (x.norm(dim=-1, keepdim=True) + 1e-3)
    if fam == "delta":
        step, ins, sts = W.delta_rule, [unit(row()), unit(row()), col(), torch.sigmoid(sc())], [n(B, H, M, N) * 0.1]
    elif fam == "gated":
        step = W.gated_delta_rule
        ins, sts = [unit(row()), unit(row()), col(), torch.sigmoid(sc()), torch.sigmoid(sc())], [n(B, H, M, N) * 0.1]
    elif fam == "rwkv7":
        kk = unit(row())
        step = W.rwkv7
        ins = [row() / N ** .5, torch.exp(-torch.exp(-0.5 + 0.5 * row())), row() / N ** .5, col(), -kk,
               kk * torch.sigmoid(n(*kk.shape))]
        sts = [n(B, H, M, N) * 0.1]
    elif fam == "mamba2":
        step = W.mamba2
        ins = [col(), torch.nn.functional.softplus(-1 + sc()), -torch.exp(n(1, 1, H, 1, 1)), row() / N ** .5, row() / N ** .5]
        sts = [torch.zeros(B, H, M, N)]
    elif fam == "gla":
        step, ins, sts = X.gla, [row(), row(), col(), -torch.sigmoid(row())], [n(B, H, M, N)]
    elif fam == "retention":
        step, ins, sts = X.retention, [torch.sigmoid(sc()), row(), row(), col()], [n(B, H, M, N)]
    elif fam == "hgrn":
        N = 1
        step, ins, sts = X.hgrn, [n(*bc([B, T, H, M, 1])), -torch.sigmoid(n(*bc([B, T, H, M, 1])))], [n(B, H, M, 1)]
    elif fam == "two_outputs":
        step, ins, sts = two_outputs, [row(), row(), col(), torch.sigmoid(row())], [n(B, H, M, N)]
    elif fam == "two_states":
        step, ins, sts = two_states, [row(), row(), col(), torch.sigmoid(sc())], [n(B, H, M, N), n(B, H, M, N)]
    else:
        step, ins, sts = column_gate, [row(), row(), col()], [n(B, H, M, N)]
    for d, full in enumerate((B, T, H)):         # every extent must appear in some input
        if all(x.shape[d] == 1 for x in ins):
            s = list(ins[0].shape)
            s[d] = full
            ins[0] = ins[0].expand(*s).contiguous()
    dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16, torch.bfloat16, torch.float16, torch.float64])
    ins, sts = [x.to(dtype) for x in ins], [x.to(dtype) for x in sts]
    # layouts
    if rng.random() < 0.3:                        # every second element of a wider last dimension
        i = rng.randrange(len(ins))
        x = ins[i]
        big = torch.zeros(*x.shape[:-1], x.shape[-1] * 2, dtype=dtype)
        big[..., ::2] = x
        ins[i] = big[..., ::2]
    if rng.random() < 0.3:
        sts[0] = sts[0].mT.contiguous().mT
    if rng.random() < 0.35:                       # odd storage offset
        i, off = rng.randrange(len(ins)), rng.choice([1, 2, 3])
        x = ins[i]
        big = torch.zeros(*x.shape[:-1], x.shape[-1] + off + 1, dtype=dtype)
        big[..., off:off + x.shape[-1]] = x
        ins[i] = big[..., off:off + x.shape[-1]]
    if rng.random() < 0.2:
        x = sts[0]
        big = torch.zeros(x.numel() + 3, dtype=dtype)
        v = big[1:1 + x.numel()].view(x.shape)
        v.copy_(x)
        sts[0] = v
    if rng.random() < 0.2:                        # time-major input
        i = rng.randrange(len(ins))
        ins[i] = ins[i].transpose(0, 1).contiguous().transpose(0, 1)
    tu = Tuning(fw_r=rng.choice([1, 2, 4]), fw_c=rng.choice([1, 2, 4, 8]), fw_mb=rng.choice([8, 16, 64]),
                fw_stage=rng.choice([2, 4, 16]), bw_r=rng.choice([1, 2, 4, 8]), bw_c=rng.choice([1, 2, 4, 8]),
                seg=rng.choice([2, 4]), nslots=rng.choice([2, 4]), kflush=rng.choice([1, 2, 8]),
                rev_stage=rng.choice([2, 4, 16]), rev_resync=rng.choice([1, 2, 4]), use_tma=rng.random() < 0.7,
                pack2=rng.choice([0, 1, 3]))
    return fam, step, ins, sts, dtype, tu


def on_device(x, dev):
    """Copy to ``dev`` keeping the strides and the storage offset modulo 16 bytes."""
    if dev is None:
        return x
    span = 1 + sum((n - 1) * st for n, st in zip(x.shape, x.stride()))
    lead = x.storage_offset() % (16 // x.element_size())
    buf = torch.zeros(lead + span, dtype=x.dtype, device=dev)
    out = buf.as_strided(x.shape, x.stride(), lead)
    out.copy_(x)
    return out


SEEDS = range(2000, 2016)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_case(seed):
    from emu.emu import EmuLauncher
    run_case(seed, None, EmuLauncher)


@pytest.mark.gpu
@pytest.mark.parametrize("seed", SEEDS)
def test_random_case_gpu(seed):
    """The same seeds through NVRTC and the C-ABI launch on the GPU (each has
    passed the emulation's alignment checks in the CPU test)."""
    run_case(seed, "cuda:0", None)


def run_case(seed, dev, launcher):
    rng = random.Random(seed)
    fam, step, ins, sts, dtype, tu = draw_case(rng)
    ins, sts = [on_device(x, dev) for x in ins], [on_device(x, dev) for x in sts]
    try:
        fwd, bwd, _, _ = build_twopass(step, tuple(ins), tuple(sts), tuning=tu, _launcher=launcher)
    except lower.LoweringError as e:
        pytest.skip(f"{fam}: {e}")
    res = fwd(tuple(ins), tuple(sts))
    ns = len(sts)
    no = len(res) - 2 * ns - 1
    g = torch.Generator().manual_seed(seed)
    dys = [torch.randn(y.shape, generator=g).to(dtype) for y in res[:no]]
    dSs = [torch.randn(s.shape, generator=g).to(dtype) for s in sts]
    dx, ds0 = bwd(tuple(d.to(ins[0].device) for d in dys), tuple(d.to(ins[0].device) for d in dSs), tuple(ins),
                  tuple(res[no + ns:no + 2 * ns]), (res[-1],))
    if dev is not None:
        torch.cuda.synchronize()
        assert fwd.kernel_status(dev) == 0
        res, dx, ds0 = [r.cpu() for r in res], [d.cpu() for d in dx], [d.cpu() for d in ds0]
        ins, sts = [x.cpu() for x in ins], [x.cpu() for x in sts]
    ry, rST, rgx, rgs = O.fwd_bwd(step, ins, sts, dys, dSs, dtype=torch.float64)
    tol_out, tol_grad = (1e-5, 3e-5) if dtype in (torch.float32, torch.float64) else (8e-3, 2e-2)
    got = list(res[:no + ns]) + list(dx) + list(ds0)
    want = list(ry) + list(rST) + rgx + rgs
    for k, (a, b, like) in enumerate(zip(got, want, [None] * (no + ns) + ins + sts)):
        b = torch.zeros_like(a, dtype=torch.float64) if b is None else b
        assert a.shape == b.shape, (fam, k)
        if like is not None:
            assert a.dtype == like.dtype
        if b.numel() < 16 and dtype in (torch.bfloat16, torch.float16):
            continue                              # a handful of bf16 values: one rounding step dominates the norm
        err = O.rel_err(a, b) if float(b.abs().max()) > 0 else float(a.float().abs().max())
        assert err < (tol_out if k < no + ns else tol_grad), (fam, k, err, tu)
