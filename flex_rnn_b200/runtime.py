"""ctypes binding of libfrnn_b200.so (see include/frnn.h) and a compile cache.

The PyTorch custom op built in ``twopass.py`` reaches the GPU only through
this module: NVRTC compilation of the generated source, module load on the
tensors' device, and launches on ``torch.cuda.current_stream()``.  There is no
other execution path: if the library is missing or the driver cannot be
reached the calls raise.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import threading
from typing import Dict, List, Optional, Sequence, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfrnn_b200.so")

SYMBOLS = ["frnn_abi_version", "frnn_last_error", "frnn_compile", "frnn_free", "frnn_module_load",
           "frnn_module_unload", "frnn_launch", "frnn_kernel_attrs", "frnn_l2_flush", "frnn_fp32_peak_probe",
           "frnn_launch_static_scratch", "frnn_static_scratch_capacity", "frnn_tensor_map_encode",
           "frnn_nvrtc_version", "frnn_status", "frnn_status_post", "frnn_status_check", "frnn_fp32_mix_probe"]


class FrnnError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """Load the C-ABI library (building it first if the .so is absent)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            from . import build as _build
            _build.build()
        L = ctypes.CDLL(LIB_PATH)
        vp, cp, sz, ci, cu = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_uint
        L.frnn_abi_version.restype = ci
        L.frnn_last_error.restype = cp
        L.frnn_compile.argtypes = [cp, ctypes.POINTER(cp), ci, ctypes.POINTER(vp), ctypes.POINTER(sz), cp, sz]
        L.frnn_free.argtypes = [vp]
        L.frnn_free.restype = None
        L.frnn_module_load.argtypes = [vp, sz, ctypes.POINTER(cp), ctypes.POINTER(cu), ci, ctypes.POINTER(vp)]
        L.frnn_module_unload.argtypes = [vp]
        L.frnn_launch.argtypes = [vp, ci, ctypes.POINTER(cu), ctypes.POINTER(cu), cu, vp, ctypes.POINTER(vp), ci]
        L.frnn_kernel_attrs.argtypes = [vp, ci, ctypes.POINTER(ci), ctypes.POINTER(ci), ctypes.POINTER(ci)]
        L.frnn_launch_static_scratch.argtypes = [vp, ci, ctypes.POINTER(cu), ctypes.POINTER(cu), cu, vp,
                                                 ctypes.POINTER(vp), ci, ctypes.POINTER(ci), ctypes.POINTER(sz), ci]
        L.frnn_static_scratch_capacity.restype = sz
        L.frnn_tensor_map_encode.argtypes = [vp, vp, cu, cu, ctypes.POINTER(ctypes.c_uint64),
                                             ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint32)]
        L.frnn_nvrtc_version.argtypes = [ctypes.POINTER(ci), ctypes.POINTER(ci)]
        L.frnn_status.argtypes = [vp, vp]
        L.frnn_status_post.argtypes = [vp, vp, vp]
        L.frnn_status_check.argtypes = [vp, vp, vp]
        L.frnn_l2_flush.argtypes = [vp, sz, vp]
        L.frnn_fp32_peak_probe.argtypes = [vp, ci, vp, ctypes.POINTER(ctypes.c_double)]
        L.frnn_fp32_mix_probe.argtypes = [ci, vp, vp, ci, vp, ctypes.POINTER(ctypes.c_double)]
        _lib = L
    return _lib


def _check(rc: int, what: str):
    if rc != 0:
        raise FrnnError(f"{what} failed (code {rc}): {lib().frnn_last_error().decode(errors='replace')}")


_cubin_cache: Dict[str, Tuple[bytes, str]] = {}
_toolchain_tag: Optional[str] = None


def toolchain_tag() -> str:
    """What a cached cubin depends on besides its source: the NVRTC that
    compiled it and the ABI of the library whose prelude it was generated for."""
    global _toolchain_tag
    if _toolchain_tag is None:
        L = lib()
        major, minor = ctypes.c_int(), ctypes.c_int()
        _check(L.frnn_nvrtc_version(ctypes.byref(major), ctypes.byref(minor)), "frnn_nvrtc_version")
        _toolchain_tag = f"nvrtc{major.value}.{minor.value}-abi{L.frnn_abi_version()}-sm_100a"
    return _toolchain_tag


def cache_key(src: str, opts: Sequence[str] = ()) -> str:
    return hashlib.sha256("\0".join([toolchain_tag(), src, *opts]).encode()).hexdigest()


def compile_cubin(src: str, opts: Sequence[str] = ()) -> Tuple[bytes, str]:
    """NVRTC-compile ``src`` for sm_100a.  Returns (cubin, compiler log).
    Needs no GPU.  Results are cached in memory and, when ``FRNN_CACHE_DIR`` is
    set, on disk, keyed by the source, the options, the NVRTC version and the
    library's ABI version (the reference keys on the source hash alone,
    flex_rnn/to_cuda.py:264).  A cached entry's log reads "(cached)"."""
    key = cache_key(src, opts)
    if key in _cubin_cache:
        return _cubin_cache[key]
    cdir = os.environ.get("FRNN_CACHE_DIR")
    if cdir:
        fn = os.path.join(cdir, key + ".cubin")
        if os.path.exists(fn):
            with open(fn, "rb") as f:
                out = (f.read(), "(cached)")
            _cubin_cache[key] = out
            return out
    L = lib()
    arr = (ctypes.c_char_p * max(1, len(opts)))(*[o.encode() for o in opts])
    cub = ctypes.c_void_p()
    size = ctypes.c_size_t()
    log = ctypes.create_string_buffer(1 << 16)
    rc = L.frnn_compile(src.encode(), arr, len(opts), ctypes.byref(cub), ctypes.byref(size), log, len(log))
    logtxt = log.value.decode(errors="replace")
    if rc != 0:
        raise FrnnError(f"frnn_compile failed (code {rc}): {L.frnn_last_error().decode(errors='replace')}\n{logtxt}")
    data = ctypes.string_at(cub.value, size.value)
    L.frnn_free(cub)
    if cdir:
        os.makedirs(cdir, exist_ok=True)
        tmp = os.path.join(cdir, f"{key}.{os.getpid()}.tmp")
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, os.path.join(cdir, key + ".cubin"))     # atomic: several ranks may fill one cache
    _cubin_cache[key] = (data, logtxt)
    return data, logtxt


class StructArg:
    """A by-value kernel parameter of 128 bytes, 64-byte aligned (a TMA tensor map)."""

    def __init__(self):
        self._raw = ctypes.create_string_buffer(256)
        self.addr = (ctypes.addressof(self._raw) + 63) // 64 * 64


def encode_tensor_map(base_ptr: int, elt_bytes: int, dims: Sequence[int], strides_bytes: Sequence[int],
                      box: Sequence[int]) -> StructArg:
    """Tensor map for a tiled TMA load (dims fastest first; strides for dims 1..)."""
    arg = StructArg()
    r = len(dims)
    d = (ctypes.c_uint64 * r)(*[int(x) for x in dims])
    st = (ctypes.c_uint64 * max(1, r - 1))(*[int(x) for x in strides_bytes])
    bx = (ctypes.c_uint32 * r)(*[int(x) for x in box])
    _check(lib().frnn_tensor_map_encode(ctypes.c_void_p(arg.addr), ctypes.c_void_p(int(base_ptr)), int(elt_bytes), r, d, st, bx),
           "frnn_tensor_map_encode")
    return arg


class Module:
    """A loaded cubin with its kernels, bound to the device current at load."""

    def __init__(self, cubin: bytes, names: Sequence[str], smem: Sequence[int]):
        L = lib()
        self._names = list(names)
        n = len(names)
        arr = (ctypes.c_char_p * n)(*[s.encode() for s in names])
        sm = (ctypes.c_uint * n)(*[int(s) for s in smem])
        h = ctypes.c_void_p()
        self._buf = ctypes.create_string_buffer(cubin, len(cubin))
        _check(L.frnn_module_load(self._buf, len(cubin), arr, sm, n, ctypes.byref(h)), "frnn_module_load")
        self._h = h

    def launch(self, kernel: int, grid: Sequence[int], block: int, smem: int, stream: int, ptrs: Sequence[int]):
        """Launch with the kernel parameters ``ptrs``: ints are device pointers
        (or integers of at most 8 bytes), :class:`StructArg` objects are
        by-value struct parameters."""
        n = len(ptrs)
        vals = (ctypes.c_void_p * n)(*[ctypes.c_void_p(0 if isinstance(p, StructArg) else int(p)) for p in ptrs])
        args = (ctypes.c_void_p * n)(*[p.addr if isinstance(p, StructArg) else
                                       ctypes.addressof(vals) + i * ctypes.sizeof(ctypes.c_void_p)
                                       for i, p in enumerate(ptrs)])
        g = (ctypes.c_uint * 3)(*[int(x) for x in grid])
        b = (ctypes.c_uint * 3)(int(block), 1, 1)
        _check(lib().frnn_launch(self._h, kernel, g, b, int(smem), ctypes.c_void_p(int(stream)), args, n),
               f"frnn_launch({self._names[kernel]})")

    def launch_static_scratch(self, kernel: int, grid: Sequence[int], block: int, smem: int, stream: int,
                              ptrs: Sequence[int], scratch: Dict[int, int]):
        """Like :meth:`launch`, for callers that cannot allocate device memory:
        the parameters listed in ``scratch`` (parameter index -> bytes) are
        pointed at the library's static scratch array; the entries of ``ptrs``
        at those indices are ignored.  Fails if the sizes exceed the array."""
        n = len(ptrs)
        vals = (ctypes.c_void_p * n)(*[ctypes.c_void_p(0 if isinstance(p, StructArg) else int(p)) for p in ptrs])
        args = (ctypes.c_void_p * n)(*[p.addr if isinstance(p, StructArg) else
                                       ctypes.addressof(vals) + i * ctypes.sizeof(ctypes.c_void_p)
                                       for i, p in enumerate(ptrs)])
        g = (ctypes.c_uint * 3)(*[int(x) for x in grid])
        b = (ctypes.c_uint * 3)(int(block), 1, 1)
        idx = sorted(scratch)
        sa = (ctypes.c_int * len(idx))(*idx)
        sb = (ctypes.c_size_t * len(idx))(*[int(scratch[i]) for i in idx])
        _check(lib().frnn_launch_static_scratch(self._h, kernel, g, b, int(smem), ctypes.c_void_p(int(stream)), args, n,
                                                sa, sb, len(idx)),
               f"frnn_launch_static_scratch({self._names[kernel]})")

    def attrs(self, kernel: int) -> Dict[str, int]:
        r, s, l = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _check(lib().frnn_kernel_attrs(self._h, kernel, ctypes.byref(r), ctypes.byref(s), ctypes.byref(l)), "frnn_kernel_attrs")
        return {"regs": r.value, "static_smem": s.value, "local_bytes": l.value}

    def close(self):
        if getattr(self, "_h", None):
            lib().frnn_module_unload(self._h)
            self._h = None


def status(err_word_ptr: int, stream: int):
    """Synchronous check of a kernel error word; raises FrnnError if a kernel reported a timed-out wait."""
    _check(lib().frnn_status(ctypes.c_void_p(err_word_ptr), ctypes.c_void_p(stream)), "kernel status")


def status_post(err_word_ptr: int, host_word_ptr: int, stream: int):
    _check(lib().frnn_status_post(ctypes.c_void_p(err_word_ptr), ctypes.c_void_p(host_word_ptr), ctypes.c_void_p(stream)),
           "frnn_status_post")


def status_check(host_word_ptr: int, err_word_ptr: int, stream: int):
    _check(lib().frnn_status_check(ctypes.c_void_p(host_word_ptr), ctypes.c_void_p(err_word_ptr), ctypes.c_void_p(stream)),
           "kernel status")


def l2_flush(buf_ptr: int, nbytes: int, stream: int):
    _check(lib().frnn_l2_flush(ctypes.c_void_p(buf_ptr), nbytes, ctypes.c_void_p(stream)), "frnn_l2_flush")


MIX_PROBES = {0: "ffma_three_distinct_operands", 1: "ffma_one_operand_kept", 2: "ffma2_three_distinct_pairs",
              3: "ffma2_one_pair_kept", 4: "delta_rule_backward_mix_packed", 5: "delta_rule_forward_mix_scalar"}


def fp32_mix_probe(kind: int, sink_ptr: int, in_ptr: int, iters: int, stream: int) -> float:
    fl = ctypes.c_double()
    _check(lib().frnn_fp32_mix_probe(int(kind), ctypes.c_void_p(sink_ptr), ctypes.c_void_p(in_ptr), iters,
                                     ctypes.c_void_p(stream), ctypes.byref(fl)), "frnn_fp32_mix_probe")
    return fl.value


def fp32_peak_probe(sink_ptr: int, iters: int, stream: int) -> float:
    fl = ctypes.c_double()
    _check(lib().frnn_fp32_peak_probe(ctypes.c_void_p(sink_ptr), iters, ctypes.c_void_p(stream), ctypes.byref(fl)),
           "frnn_fp32_peak_probe")
    return fl.value
