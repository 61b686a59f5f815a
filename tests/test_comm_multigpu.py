"""Symmetric-heap collectives on 2+ GPUs (child processes under torchrun)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, nproc, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", str(nproc), os.path.join(ROOT, "tests", script)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_heap_collectives():
    n = min(torch.cuda.device_count(), 4)
    n = 2 if n < 4 else 4
    res = _run("mp_comm_worker.py", n)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "FAIL" not in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_cosmos3_tp2_sp2_on_four_gpus():
    """Dual-pathway transformer on a tp2 x sp2 mesh of GPUs (symmetric-heap all-reduce and Ulysses exchange, prefix
    tower cut four ways) against the same model on one GPU."""
    res = _run("mp_cosmos_worker.py", 4, {"NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "matches one GPU" in res.stdout
