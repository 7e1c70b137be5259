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
    assert lib.frnn_abi_version() == 2


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
    for op in ("delta_rule", "mamba2", "rwkv7", "gated_delta_rule"):
        B, T, H, M, N = W.CONFIGS[op]
        B, T = min(B, 8), min(T, 1024)
        xs, _, _ = W.synthetic(op, 2, 2, H, 2, 2)
        ins = tuple(torch.empty([B if x.shape[0] > 1 else 1, T if x.shape[1] > 1 else 1, H,
                                 M if x.shape[3] > 1 else 1, N if x.shape[4] > 1 else 1], dtype=torch.bfloat16, device="meta")
                    for x in xs[:-1])
        plan, _, _ = make_plan(W.STEPS[op], ins, (torch.empty(B, H, M, N, dtype=torch.bfloat16, device="meta"),))
        for ks in generate(plan):
            cubin, log = runtime.compile_cubin(ks.source)
            assert "cp.async.bulk" in ks.source and "mbarrier" in ks.source
            if ks.name == "frnn_bw":
                assert "setmaxnreg" in ks.source and ("tcgen05.st" in ks.source) and "Used 168 registers" in log or op == "mamba2"
            spills = [int(x) for x in re.findall(r"(\d+) bytes spill stores", log)]
            assert spills and max(spills) < 256, log[-600:]      # a few scalars at most: no state tile (256 bytes) is spilled


def test_static_scratch_refuses_bad_scratch_lists():
    """frnn_launch_static_scratch refuses, before it touches the device, more
    scratch parameters than kernel parameters (its index tables live on the
    stack) and a parameter index listed twice."""
    lib = runtime.lib()
    # never dereferenced for these refusals; zeroed, it would read as a module without kernels
    fake_module = ctypes.create_string_buffer(128)
    g = (ctypes.c_uint * 3)(1, 1, 1)
    vals = (ctypes.c_void_p * 4)()
    args = (ctypes.c_void_p * 4)(*[ctypes.addressof(vals) + 8 * i for i in range(4)])

    def call(idx, sizes, nargs=4):
        sa = (ctypes.c_int * len(idx))(*idx)
        sb = (ctypes.c_size_t * len(idx))(*sizes)
        return lib.frnn_launch_static_scratch(fake_module, 0, g, g, 0, None, args, nargs, sa, sb, len(idx))

    assert call(list(range(80)), [16] * 80) == 1                      # nscratch > nargs (and > 64)
    assert b"no more scratch" in lib.frnn_last_error()
    assert call([0, 1, 2, 3, 0], [16] * 5) == 1                       # nscratch > nargs
    assert call([1, 1], [16, 16]) == 1                                # duplicate
    assert b"listed twice" in lib.frnn_last_error()
    assert call([4], [16]) == 1                                       # index out of range
    assert call([0], [lib.frnn_static_scratch_capacity() + 1]) == 1   # too large
    assert b"more scratch than" in lib.frnn_last_error()
    assert call([0], [16]) == 1                                       # passes the list checks; the empty module is refused
    assert b"bad kernel index" in lib.frnn_last_error()


def test_status_check_reports_and_clears_a_host_word():
    """frnn_status_check looks at the host mirror of a kernel error word: zero
    is OK, anything else is FRNN_E_KERNEL once, after which the mirror is
    clear again.  (No device is involved when no device word is given.)"""
    lib = runtime.lib()
    word = ctypes.c_int(0)
    assert lib.frnn_status_check(ctypes.byref(word), None, None) == 0
    word.value = 2
    assert lib.frnn_status_check(ctypes.byref(word), None, None) == 5     # FRNN_E_KERNEL
    assert b"checkpoint copy" in lib.frnn_last_error()
    assert word.value == 0
    assert lib.frnn_status_check(ctypes.byref(word), None, None) == 0
    assert lib.frnn_status_check(None, None, None) == 1
    assert lib.frnn_status(None, None) == 1 and lib.frnn_status_post(None, None, None) == 1


def test_disk_cache_round_trip(tmp_path, monkeypatch):
    """With FRNN_CACHE_DIR a second compilation of the same source (in a fresh
    process: here the in-memory cache is emptied) is served from disk with
    identical bytes; the key names the NVRTC and ABI versions, so another
    toolchain does not reuse the entry."""
    monkeypatch.setenv("FRNN_CACHE_DIR", str(tmp_path))
    src = 'extern "C" __global__ void cached_k(float* p) { p[threadIdx.x] = 2.0f; }'
    monkeypatch.setattr(runtime, "_cubin_cache", {})
    cubin, log = runtime.compile_cubin(src)
    assert log != "(cached)"
    files = os.listdir(tmp_path)
    assert files == [runtime.cache_key(src) + ".cubin"]
    monkeypatch.setattr(runtime, "_cubin_cache", {})
    cubin2, log2 = runtime.compile_cubin(src)
    assert log2 == "(cached)" and cubin2 == cubin
    assert re.fullmatch(r"nvrtc\d+\.\d+-abi\d+-sm_100a", runtime.toolchain_tag())
    # another NVRTC or ABI version gives another key, hence a miss
    monkeypatch.setattr(runtime, "_toolchain_tag", "nvrtc99.0-abi2-sm_100a")
    assert runtime.cache_key(src) + ".cubin" not in files
    monkeypatch.setattr(runtime, "_cubin_cache", {})
    _, log3 = runtime.compile_cubin(src)
    assert log3 != "(cached)" and len(os.listdir(tmp_path)) == 2
