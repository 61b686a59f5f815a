"""Loader of the native kernel library (plain C ABI, ctypes).

On a machine with a GPU the library must be present: ops raise instead of silently falling back to PyTorch,
so a missing or stale build is noticed at once. On a CPU-only machine the ops use their PyTorch reference
implementations (the same code that the numerics tests compare the kernels against).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

from . import _counters

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_KERNELS = None
_RUNTIME = None


class NativeLibraryError(RuntimeError):
    pass


def kernels_path() -> Path:
    return _LIB_DIR / "libmstar_kernels.so"


def runtime_path() -> Path:
    return _LIB_DIR / "libmstar_runtime.so"


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library. Raises NativeLibraryError if it has not been built."""
    global _KERNELS
    if _KERNELS is None:
        p = kernels_path()
        if not p.exists():
            raise NativeLibraryError(
                f"{p} is missing: build it with `python -m mstar_b200.build` (needs nvcc, no GPU required)")
        lib = ctypes.CDLL(str(p))
        lib.mstar_last_error.restype = ctypes.c_char_p
        lib.mstar_read_status.restype = ctypes.c_uint
        lib.mstar_read_status.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.mstar_set_wait_limit_ns.argtypes = [ctypes.c_ulonglong]
        lib.mstar_get_wait_limit_ns.restype = ctypes.c_ulonglong
        _KERNELS = lib
    return _KERNELS


def runtime() -> ctypes.CDLL:
    """The C++ host runtime (control mesh, shared-memory arena)."""
    global _RUNTIME
    if _RUNTIME is None:
        p = runtime_path()
        if not p.exists():
            raise NativeLibraryError(f"{p} is missing: build it with `python -m mstar_b200.build`")
        _RUNTIME = ctypes.CDLL(str(p))
    return _RUNTIME


def use_cuda(*tensors: torch.Tensor) -> bool:
    """True when the op must run the CUDA kernel (any tensor on a GPU)."""
    return any(t is not None and t.is_cuda for t in tensors)


def check(rc: int, what: str) -> None:
    _counters.bump()
    if rc != 0:
        msg = kernels().mstar_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed: {msg}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


def read_status(clear: bool = True) -> tuple[int, int, int, int]:
    """Status word written by kernels whose bounded waits ran out: (code, block, aux0, aux1); code 0 = ok.
    code = kernel_id << 16 | phase."""
    buf = (ctypes.c_uint * 4)()
    kernels().mstar_read_status(buf, 1 if clear else 0)
    return tuple(int(x) for x in buf)


def status_copy_async(pinned: torch.Tensor) -> None:
    """Queue a copy of the current device's status word into ``pinned`` (int32[4], pinned host memory) on the
    current stream; the caller reads it after synchronising with an event recorded behind the copy."""
    rc = kernels().mstar_status_copy_async(ctypes.c_void_p(pinned.data_ptr()), ctypes.c_void_p(stream_ptr()))
    if rc != 0:
        raise RuntimeError("status copy failed: " + kernels().mstar_last_error().decode(errors="replace"))


def prefetch_hint(w=None, lo: int = 0, nbytes: int | None = None, l2_hints: int = 1) -> None:
    """Tell the next GEMM / decode-attention launch on the current device to pull bytes [lo, lo + nbytes) of ``w`` (a
    tensor or a packed weight: the projection that runs AFTER that launch) into the L2 while it runs, and to mark its
    own streamed operand evict-first. ``w=None`` asks for the evict-first marking only (``l2_hints=0``: clears a pending hint). Used once by the launch that takes it."""
    L = kernels()
    if w is None:
        L.mstar_prefetch_hint(ctypes.c_void_p(0), ctypes.c_ulonglong(0), int(l2_hints) if nbytes is None else 0)
        return
    t = w.data
    total = t.numel() * t.element_size()
    lo = min(max(0, int(lo)), total)
    n = total - lo if nbytes is None else max(0, min(int(nbytes), total - lo))
    L.mstar_prefetch_hint(ctypes.c_void_p(t.data_ptr() + lo), ctypes.c_ulonglong(n), int(l2_hints))


def decode_status(code: int) -> str:
    """Readable form of a status code: which kernel gave up in which phase."""
    names = {1: "gemm", 2: "attention", 3: "decode attention", 4: "expert gemm", 5: "collective", 6: "gemm+all-reduce",
             7: "ulysses exchange", 8: "cfg combine", 9: "expert dispatch/combine", 10: "test", 11: "gemm+reduce-scatter",
             12: "all-gather+gemm", 13: "sharded sampler"}
    return f"{names.get(code >> 16, 'kernel ' + str(code >> 16))} wait ran out in phase {code & 0xffff}"


def set_wait_limit_ns(ns: int) -> None:
    kernels().mstar_set_wait_limit_ns(int(ns))


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")
