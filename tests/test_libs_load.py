"""Both shared libraries resolve every symbol at load time (no GPU needed: the CUDA runtime is linked, not called)."""
import ctypes
import os

import pytest

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mstar_b200", "lib")


@pytest.mark.parametrize("name", ["libmstar_kernels.so", "libmstar_runtime.so"])
def test_library_loads_with_all_symbols_bound(name):
    path = os.path.join(LIB, name)
    if not os.path.exists(path):
        from mstar_b200 import build
        build.build_all()
    ctypes.CDLL(path, mode=os.RTLD_NOW | os.RTLD_LOCAL)
