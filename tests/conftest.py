import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")
    config.addinivalue_line("markers", "expects_status: the test makes a bounded device wait run out on purpose and "
                                       "reads the status word itself")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _kernel_status_clean(request):
    """After every GPU test, the device status word must be clean (no bounded wait ran out)."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from mstar_b200.ops import _lib
        if request.node.get_closest_marker("expects_status") is None:
            code = _lib.read_status(clear=True)[0]
            assert code == 0, f"kernel status word set: {code:#x}"


def reference_module(name: str):
    """Import a module of the reference project installed under ``baseline/_ref`` (the CPU oracle of the parity
    tests); the test is skipped when the package is not there or does not import on this machine."""
    import importlib
    import os
    import sys
    ref = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "mstar")):
        pytest.skip("reference package not installed under baseline/_ref")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        return importlib.import_module(name)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"reference module {name} does not import here: {type(e).__name__}: {e}")
