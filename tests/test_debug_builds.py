"""The two debugging aids that stand in for a memory checker on the GPU.

``Tuning.bounds`` (``FRNN_TUNE_BOUNDS=1``) builds both kernels with every load,
store, atomic add and bulk copy tested against the byte extents of the kernel's
buffers; an access outside is skipped and reported through the error word
(code 64).  ``FRNN_GUARD=1`` places every buffer the kernels write between two
bands of a byte pattern and checks the bands after each launch.

CPU tests run the checked build under the host emulation and provoke both
reports on the host (a registered extent made too small in the source text, a
launcher that writes one byte past an output); the GPU tests only run correct
kernels with both aids switched on and expect silence and parity.
"""
import ctypes
import dataclasses
import re

import pytest
import torch

from flex_rnn_b200 import examples as X
from flex_rnn_b200.twopass import Tuning, build_twopass, default_tuning
from oracle import naive_oracle as O

ERR_BOUNDS = 64
SMALL = Tuning(fw_r=2, fw_c=4, fw_mb=8, fw_stage=4, bw_r=2, bw_c=4, seg=2, nslots=2, bounds=1)


def _run(step, ins, sts, tu, launcher=None, dev="cpu"):
    fwd, bwd, _, _ = build_twopass(step, tuple(ins), tuple(sts), tuning=tu, _launcher=launcher)
    res = fwd(tuple(ins), tuple(sts))
    ns = len(sts)
    no = len(res) - 2 * ns - 1
    g = torch.Generator().manual_seed(1)
    dys = [torch.randn(y.shape, generator=g).to(dev) for y in res[:no]]
    dSs = [torch.randn(s.shape, generator=g).to(dev) for s in sts]
    dx, ds0 = bwd(tuple(d.to(y.dtype) for d, y in zip(dys, res[:no])), tuple(d.to(s.dtype) for d, s in zip(dSs, sts)),
                  tuple(ins), tuple(res[no + ns:no + 2 * ns]), (res[-1],))
    return fwd, list(res[:no + ns]) + list(dx) + list(ds0), dys, dSs


def _parity(step, ins, sts, got, dys, dSs, tol_out, tol_grad):
    cpu = lambda ts: [t.detach().cpu() for t in ts]
    ry, rST, rgx, rgs = O.fwd_bwd(step, cpu(ins), cpu(sts), [d.cpu().float() for d in dys], [d.cpu().float() for d in dSs],
                                  dtype=torch.float64)
    n_fw = len(ry) + len(rST)
    for i, (a, b) in enumerate(zip(got, list(ry) + list(rST) + rgx + rgs)):
        assert O.rel_err(a.cpu(), b) < (tol_out if i < n_fw else tol_grad), i


CASES = [("delta_rule", 16, 16), ("gated_delta_rule", 16, 16), ("rwkv7", 16, 16), ("mamba2", 8, 16),
         ("rwkv4", 64, 1), ("mamba", 16, 16), ("s4d", 16, 16)]


def _case(op, B, T, H, M, N, dtype=torch.float32):
    if op in O.STEPS:
        xs = O.make_inputs(op, B, T, H, M, N, dtype)
        return O.STEPS[op], xs[:-1], xs[-1:]
    ins, sts = X.zoo_case(op, B, T, H, M, N, dtype)
    return X.ZOO[op], list(ins), list(sts)


@pytest.mark.parametrize("op,M,N", CASES, ids=[c[0] for c in CASES])
def test_checked_build_and_guard_bands_emulated(op, M, N, monkeypatch):
    """Ragged T (9 steps: stage 4, checkpoint chunk 4), two heads, two batch
    rows: every kind of access the two kernels make passes its check and stays
    inside its buffer."""
    from emu.emu import EmuLauncher
    monkeypatch.setenv("FRNN_GUARD", "1")
    step, ins, sts = _case(op, 2, 9, 2, M, N)
    fwd, got, dys, dSs = _run(step, ins, sts, SMALL, EmuLauncher)
    assert all(ks.source.startswith("#define FRNN_BOUNDS 1") and ks.info["bounds"] for ks in fwd.sources)
    assert fwd.kernel_status() == 0
    _parity(step, ins, sts, got, dys, dSs, 1e-5, 1e-5)


def test_checked_build_refuses_and_reports_emulated(monkeypatch):
    """The checkpoint buffer registered with no extent at all: the checked build
    must drop every checkpoint store (the buffer keeps the guard's byte
    pattern), report code 64, and touch nothing outside its buffers."""
    from emu.emu import EmuLauncher
    monkeypatch.setenv("FRNN_GUARD", "1")

    def shrunk(ks):
        src, n = re.subn(r"frnn_bounds_add\(ck0, \d+L\);", "frnn_bounds_add(ck0, 0L);", ks.source)
        assert n == 1
        return EmuLauncher(dataclasses.replace(ks, source=src))

    step, ins, sts = _case("gated_delta_rule", 1, 8, 1, 16, 16)
    fwd, _, _, _ = build_twopass(step, tuple(ins), tuple(sts), tuning=SMALL, _launcher=shrunk)
    y, ST, store, aux = fwd(tuple(ins), tuple(sts))
    assert fwd.kernel_status() == ERR_BOUNDS
    assert store.numel() > 0 and bool((store.view(torch.uint8) == 0xA5).all())
    ry, rST = O.scan(step, ins, sts)           # everything else was computed as usual
    assert O.rel_err(y, ry[0]) < 1e-5 and O.rel_err(ST, rST[0]) < 1e-5


def test_guard_band_detects_a_stray_store(monkeypatch):
    """A launcher that, after the real kernel, writes one byte just past the
    first output (on the host): the next check names the buffer."""
    from emu.emu import EmuLauncher
    monkeypatch.setenv("FRNN_GUARD", "1")
    B, T, H, M, N = 1, 5, 1, 16, 16

    class Stray(EmuLauncher):
        def __call__(self, ptrs, device=None):
            super().__call__(ptrs, device)
            if "out0" in self.ks.params:
                ctypes.memset(int(ptrs[self.ks.params.index("out0")]) + B * T * H * M * 4, 0, 1)

    step, ins, sts = _case("delta_rule", B, T, H, M, N)
    fwd, _, _, _ = build_twopass(step, tuple(ins), tuple(sts), tuning=SMALL, _launcher=Stray)
    with pytest.raises(RuntimeError, match=r"outside output #1 \(after the buffer\)"):
        fwd(tuple(ins), tuple(sts))


GPU_CASES = [("delta_rule", 128, 128, torch.bfloat16), ("gated_delta_rule", 128, 128, torch.bfloat16),
             ("rwkv7", 128, 128, torch.bfloat16), ("mamba2", 64, 128, torch.bfloat16),
             ("rwkv4", 256, 1, torch.float32), ("mamba", 64, 64, torch.float32), ("s4d", 64, 64, torch.float32),
             ("hgrn", 256, 1, torch.float32)]


@pytest.mark.gpu
@pytest.mark.parametrize("op,M,N,dtype", GPU_CASES, ids=[c[0] for c in GPU_CASES])
def test_checked_build_and_guard_bands_gpu(op, M, N, dtype, monkeypatch):
    """The kernels the benchmark shapes get (state sizes and dtypes of the four
    workloads; three more step families), 40 steps, checked build and guard
    bands on: no report, no touched band, parity as usual."""
    monkeypatch.setenv("FRNN_GUARD", "1")
    B, T, H = 2, 40, 2
    step, ins, sts = _case(op, B, T, H, M, N, dtype)
    ins, sts = [x.to("cuda:0") for x in ins], [s.to("cuda:0") for s in sts]
    tu = dataclasses.replace(default_tuning(B, T, H, M, N, len(sts)), bounds=1, autotune=0)
    fwd, got, dys, dSs = _run(step, ins, sts, tu, dev="cuda:0")
    torch.cuda.synchronize()
    assert all(ks.info.get("bounds") for ks in fwd.sources)
    assert fwd.kernel_status("cuda:0") == 0
    tol = (5e-3, 1e-2) if dtype == torch.bfloat16 else (1e-5, 1e-5)
    _parity(step, ins, sts, got, dys, dSs, *tol)
