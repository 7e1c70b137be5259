"""The C-ABI library: it loads without a GPU, exports every function that
include/frnn.h declares, compiles with NVRTC for sm_100a, and reports errors
through return codes."""
import ctypes
import os
import re

import pytest

from flex_rnn_b200 import runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "frnn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(frnn_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    lib = runtime.lib()
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/frnn.h but not exported"
    assert sorted(runtime.SYMBOLS) == names
    assert lib.frnn_abi_version() == 1


def test_nvrtc_compiles_for_sm100a_without_gpu():
    src = 'extern "C" __global__ void k(float* p) { p[threadIdx.x] = 1.0f; }'
    cubin, log = runtime.compile_cubin(src)
    assert cubin[:4] == b"\x7fELF" and len(cubin) > 500
    assert "registers" in log


def test_compile_error_is_reported_not_thrown():
    lib = runtime.lib()
    with pytest.raises(runtime.FrnnError, match="NVRTC compilation failed"):
        runtime.compile_cubin('extern "C" __global__ void k() { this is not CUDA; }')
    assert b"NVRTC" in lib.frnn_last_error()
    cub, size = ctypes.c_void_p(), ctypes.c_size_t()
    assert lib.frnn_compile(None, None, 0, ctypes.byref(cub), ctypes.byref(size), None, 0) == 1   # FRNN_E_ARG


def test_launch_argument_checks():
    lib = runtime.lib()
    g = (ctypes.c_uint * 3)(1, 1, 1)
    assert lib.frnn_launch(None, 0, g, g, 0, None, None, 0) == 1
    assert lib.frnn_module_load(None, 0, None, None, 0, None) == 1
    assert lib.frnn_l2_flush(None, 0, None) == 1
    assert lib.frnn_module_unload(None) == 0


def test_generated_kernels_compile_without_spills():
    """Benchmark-shape kernels of every benchmark step function: NVRTC accepts
    the generated source and ptxas reports (next to) no register spills."""
    import torch
    from flex_rnn_b200 import workloads as W
    from flex_rnn_b200.twopass import generate, make_plan
    for op in ("delta_rule", "mamba2"):
        B, T, H, M, N = W.CONFIGS[op]
        xs, _, _ = W.synthetic(op, 2, 2, H, 2, 2)
        ins = tuple(torch.empty([B if x.shape[0] > 1 else 1, T if x.shape[1] > 1 else 1, H,
                                 M if x.shape[3] > 1 else 1, N if x.shape[4] > 1 else 1], dtype=torch.bfloat16, device="meta")
                    for x in xs[:-1])
        plan, _, _ = make_plan(W.STEPS[op], ins, (torch.empty(B, H, M, N, dtype=torch.bfloat16, device="meta"),))
        for ks in generate(plan):
            cubin, log = runtime.compile_cubin(ks.source)
            assert "cp.async.bulk" in ks.source and "mbarrier" in ks.source
            spills = [int(x) for x in re.findall(r"(\d+) bytes spill stores", log)]
            assert spills and max(spills) <= 64, log[-600:]      # state tiles stay in registers
