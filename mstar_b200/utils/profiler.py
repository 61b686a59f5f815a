"""NVTX ranges for the worker's main-loop phases, off unless enabled (``--enable-nvtx``); never synchronises the
device unless asked, so overlap is not destroyed.
Reference counterpart: mstar/utils/profiler.py:16-55."""
from __future__ import annotations

from contextlib import contextmanager

import torch

_ENABLED = False


def enable(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(on) and torch.cuda.is_available()


def range_push(name: str, synchronize: bool = False) -> None:
    if _ENABLED:
        if synchronize:
            torch.cuda.synchronize()
        torch.cuda.nvtx.range_push(name)


def range_pop(synchronize: bool = False) -> None:
    if _ENABLED:
        if synchronize:
            torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()


def mark(name: str) -> None:
    if _ENABLED:
        torch.cuda.nvtx.mark(name)


@contextmanager
def nvtx_range(name: str, synchronize: bool = False):
    range_push(name, synchronize)
    try:
        yield
    finally:
        range_pop(synchronize)
