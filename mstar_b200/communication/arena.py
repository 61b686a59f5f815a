"""Python face of the C++ shared-memory arena (``csrc/runtime/arena.cpp``): the producer reserves blocks and
writes tensors into them, consumers in other processes map the segments and read in place. Host segments can be
registered with CUDA (``cudaHostRegister``) so that H2D copies from them are asynchronous.

Reference counterparts: PyO3 ``ShmArena`` / ``SegmentedShmArena`` (rust/src/lib.rs:120-298) and the arena transport
(mstar/communication/arena.py:153-809: pin budget, TTL reclaim, orphan sweep).
"""
from __future__ import annotations

import ctypes
import glob
import os
import time

import numpy as np
import torch

from ..ops import _lib

_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "int64": torch.int64,
           "int32": torch.int32, "uint8": torch.uint8, "int8": torch.int8, "bool": torch.bool,
           "float64": torch.float64, "int16": torch.int16}


def dtype_name(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


def dtype_from_name(name: str) -> torch.dtype:
    return _DTYPES[name]


def _bind(lib):
    lib.mstar_arena_create.restype = ctypes.c_void_p
    lib.mstar_arena_create.argtypes = [ctypes.c_char_p, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int]
    lib.mstar_arena_reserve.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong, ctypes.POINTER(ctypes.c_int),
                                        ctypes.POINTER(ctypes.c_ulonglong)]
    lib.mstar_arena_free.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong]
    lib.mstar_arena_ptr.restype = ctypes.c_void_p
    lib.mstar_arena_ptr.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong]
    lib.mstar_arena_bytes_in_use.restype = ctypes.c_ulonglong
    lib.mstar_arena_bytes_in_use.argtypes = [ctypes.c_void_p]
    lib.mstar_arena_num_segments.argtypes = [ctypes.c_void_p]
    lib.mstar_arena_largest_free.restype = ctypes.c_ulonglong
    lib.mstar_arena_largest_free.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.mstar_arena_open_segment.restype = ctypes.c_void_p
    lib.mstar_arena_open_segment.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.mstar_arena_view_ptr.restype = ctypes.c_void_p
    lib.mstar_arena_view_ptr.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong]
    lib.mstar_arena_close_segment.argtypes = [ctypes.c_void_p]
    lib.mstar_arena_destroy.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.mstar_arena_pin.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong]
    lib.mstar_arena_pinned_bytes.restype = ctypes.c_ulonglong
    lib.mstar_arena_pinned_bytes.argtypes = [ctypes.c_void_p]
    lib.mstar_arena_pin_segment.argtypes = [ctypes.c_void_p]
    lib.mstar_arena_set_pin_hooks.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return lib


def default_pin_budget() -> int:
    """Bytes of arena memory a process may page-lock (``MSTAR_SHM_ARENA_PIN_MB``, default 1024; 0 turns pinning off)."""
    return int(os.environ.get("MSTAR_SHM_ARENA_PIN_MB", "1024")) << 20


def _tensor_at(ptr: int, nbytes: int, dtype: torch.dtype, dims) -> torch.Tensor:
    if not nbytes:          # an empty tensor (a codec chunk without frames) has a block but no bytes to view
        return torch.empty(tuple(dims), dtype=dtype)
    buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
    return torch.frombuffer(buf, dtype=torch.uint8, count=nbytes).view(dtype).view(*dims)


class ShmArena:
    """Producer-side arena. ``base_name`` must be unique per producing entity."""

    def __init__(self, base_name: str, segment_bytes: int = 256 << 20, max_segments: int = 8, canaries: bool = True):
        self.lib = _bind(_lib.runtime())
        self.base_name = base_name
        self.h = self.lib.mstar_arena_create(base_name.encode(), segment_bytes, max_segments, 1 if canaries else 0)
        if not self.h:
            raise RuntimeError(f"arena: cannot create {base_name}")
        self._blocks: dict[str, tuple[int, int, float]] = {}     # uuid -> (segment, offset, time)

    def pin(self, budget_bytes: int | None = None) -> int:
        """Page-lock the segments for CUDA (``cudaHostRegister`` inside the C++ arena) so that copies between them
        and a GPU are asynchronous DMA; at most ``budget_bytes`` in total, segments added later included. Returns the
        number of pinned segments, -1 when the process has no CUDA runtime (the arena then stays pageable)."""
        return int(self.lib.mstar_arena_pin(self.h, default_pin_budget() if budget_bytes is None else budget_bytes))

    @property
    def pinned_bytes(self) -> int:
        return int(self.lib.mstar_arena_pinned_bytes(self.h))

    def write(self, uuid: str, t: torch.Tensor) -> tuple[int, int]:
        """Copy ``t`` (any device) into a fresh block; returns (segment, offset)."""
        src = t.detach().contiguous()
        nbytes = src.numel() * src.element_size()
        seg, off = ctypes.c_int(), ctypes.c_ulonglong()
        if self.lib.mstar_arena_reserve(self.h, nbytes, ctypes.byref(seg), ctypes.byref(off)) != 0:
            raise MemoryError(f"arena {self.base_name}: out of space for {nbytes} bytes")
        ptr = self.lib.mstar_arena_ptr(self.h, seg.value, off.value)
        dst = _tensor_at(ptr, nbytes, src.dtype, src.shape)
        dst.copy_(src)          # D2H when the source is on a GPU
        self._blocks[uuid] = (seg.value, off.value, time.time())
        return seg.value, off.value

    def free(self, uuid: str) -> bool:
        blk = self._blocks.pop(uuid, None)
        if blk is None:
            return False
        rc = self.lib.mstar_arena_free(self.h, blk[0], blk[1])
        if rc == 1:
            raise RuntimeError(f"arena {self.base_name}: canary around block {uuid} was overwritten")
        return rc == 0

    def reclaim_older_than(self, ttl_s: float) -> int:
        now = time.time()
        old = [u for u, (_, _, t0) in self._blocks.items() if now - t0 > ttl_s]
        for u in old:
            self.free(u)
        return len(old)

    @property
    def bytes_in_use(self) -> int:
        return int(self.lib.mstar_arena_bytes_in_use(self.h))

    @property
    def num_segments(self) -> int:
        return int(self.lib.mstar_arena_num_segments(self.h))

    def largest_free(self, seg: int = 0) -> int:
        return int(self.lib.mstar_arena_largest_free(self.h, seg))

    def close(self, unlink: bool = True) -> None:
        if self.h:
            self.lib.mstar_arena_destroy(self.h, 1 if unlink else 0)
            self.h = None


class ShmArenaReader:
    """Consumer side: maps producers' segments on first use and hands out zero-copy views."""

    def __init__(self, pin: bool = False):
        self.lib = _bind(_lib.runtime())
        self._segs: dict[tuple[str, int], int] = {}
        self.pin = pin          # page-lock producers' segments as they are mapped (consumer uploads to a GPU)
        self.pinned_segments = 0

    def read_bytes(self, base_name: str, seg: int, off: int, nbytes: int) -> bytes:
        """The block's bytes as one ``bytes`` object (one copy, no tensor in between)."""
        if not nbytes:
            return b""
        return ctypes.string_at(self._ptr(base_name, seg, off), nbytes)

    def view(self, base_name: str, seg: int, off: int, nbytes: int, dtype: torch.dtype, dims) -> torch.Tensor:
        return _tensor_at(self._ptr(base_name, seg, off), nbytes, dtype, dims)

    def _ptr(self, base_name: str, seg: int, off: int) -> int:
        key = (base_name, seg)
        h = self._segs.get(key)
        if h is None:
            h = self.lib.mstar_arena_open_segment(base_name.encode(), seg)
            if not h:
                raise FileNotFoundError(f"arena segment {base_name}.seg{seg} not found")
            self._segs[key] = h
            if self.pin:
                self.pinned_segments += int(self.lib.mstar_arena_pin_segment(h))
        ptr = self.lib.mstar_arena_view_ptr(h, off)
        if not ptr:
            raise ValueError("arena: offset outside the segment")
        return ptr

    def close(self) -> None:
        for h in self._segs.values():
            self.lib.mstar_arena_close_segment(h)
        self._segs.clear()


def sweep_orphans(prefix: str) -> int:
    """Remove arena segments and mailboxes left behind by a crashed deployment with this prefix."""
    n = 0
    for path in glob.glob(f"/dev/shm/{prefix}*"):
        try:
            os.unlink(path)
            n += 1
        except OSError:
            pass
    return n
