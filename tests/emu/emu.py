"""Compile a generated kernel with g++ against frnn_emu.h and run it on CPU tensors.

Used by the CPU tests to check the generated source itself (index arithmetic,
graph lowering, reductions, staging, checkpoint/recompute schedule) against the
oracle without a GPU.  Test infrastructure only.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE = os.path.join(tempfile.gettempdir(), "frnn_emu_cache")


def _wrapper(ks) -> str:
    casts = []
    for i, d in enumerate(ks.param_decl):
        if d.startswith("FRNN_TMAP_PARAM"):
            casts.append(f"*(const frnn_tmap*)args[{i}]")
            continue
        ctype = d.rsplit(" ", 1)[0].replace("__restrict__", "")
        casts.append(f"({ctype})args[{i}]")
    return (f'\nextern "C" void emu_run_{ks.name}(const unsigned* grid, unsigned nthreads, unsigned smem, void** args) {{\n'
            f"  emu_launch([](void** args) {{ {ks.name}({', '.join(casts)}); }}, grid, nthreads, smem, args);\n}}\n")


_FLAGS = ["-std=c++20", "-O1", "-fPIC", "-pthread", "-Wno-unknown-pragmas", "-Wno-attributes"]
_pch_dir = None


def _precompiled_header() -> str:
    """Directory holding a copy of frnn_emu.h and its precompiled form (parsing <barrier>, <thread> and friends is
    most of a kernel's build time otherwise).  Keyed by the header's contents; built once per cache."""
    global _pch_dir
    if _pch_dir is None:
        text = open(os.path.join(HERE, "frnn_emu.h")).read()
        d = os.path.join(_CACHE, "pch_" + hashlib.sha256((text + " ".join(_FLAGS)).encode()).hexdigest()[:16])
        gch = os.path.join(d, "frnn_emu.h.gch")
        if not os.path.exists(gch):
            os.makedirs(d, exist_ok=True)
            with open(os.path.join(d, "frnn_emu.h"), "w") as f:
                f.write(text)
            tmp = gch + f".{os.getpid()}.tmp"
            r = subprocess.run(["g++", *_FLAGS, "-x", "c++-header", "-o", tmp, os.path.join(d, "frnn_emu.h")],
                               capture_output=True, text=True)
            if r.returncode:
                raise RuntimeError("emulation header build failed:\n" + r.stderr[-4000:])
            os.replace(tmp, gch)
        _pch_dir = d
    return _pch_dir


def compile_emu(ks):
    os.makedirs(_CACHE, exist_ok=True)
    src = '#include "frnn_emu.h"\n' + ks.source + _wrapper(ks)
    key = hashlib.sha256((src + open(os.path.join(HERE, "frnn_emu.h")).read()).encode()).hexdigest()[:24]
    so = os.path.join(_CACHE, f"emu_{key}.so")
    if not os.path.exists(so):
        cpp = os.path.join(_CACHE, f"emu_{key}.cpp")
        with open(cpp, "w") as f:
            f.write(src)
        cmd = ["g++", *_FLAGS, "-shared", "-I", _precompiled_header(), "-o", so + ".tmp", cpp]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError("emulation build failed:\n" + r.stderr[-4000:])
        os.replace(so + ".tmp", so)
    return ctypes.CDLL(so)


class EmuLauncher:
    """Drop-in for the CUDA launcher of ``build_twopass`` (its ``_launcher`` seam)."""

    def __init__(self, ks):
        self.ks = ks
        self.lib = compile_emu(ks)
        self.fn = getattr(self.lib, f"emu_run_{ks.name}")
        self.fn.argtypes = [ctypes.POINTER(ctypes.c_uint), ctypes.c_uint, ctypes.c_uint, ctypes.POINTER(ctypes.c_void_p)]
        self.fn.restype = None

    def __call__(self, ptrs, device=None):
        ptrs = list(ptrs)
        keep = []
        for tm in self.ks.tmaps:      # emulated tensor maps (layout of frnn_tmap in frnn_emu.h)
            raw = ctypes.create_string_buffer(256)
            addr = (ctypes.addressof(raw) + 63) // 64 * 64
            vals = [int(ptrs[tm["src_index"]]) + tm["off_bytes"]] + list(tm["dims"]) + list(tm["strides_bytes"])
            ctypes.memmove(addr, (ctypes.c_uint64 * 8)(*vals), 64)
            ctypes.memmove(addr + 64, (ctypes.c_uint32 * 5)(*(list(tm["box"]) + [tm["elt"]])), 20)
            keep.append(raw)
            ptrs.append(addr)
        n = len(ptrs)
        args = (ctypes.c_void_p * n)(*[ctypes.c_void_p(int(p)) for p in ptrs])
        grid = (ctypes.c_uint * 3)(*self.ks.grid)
        self.fn(grid, self.ks.block, self.ks.smem_bytes, args)
