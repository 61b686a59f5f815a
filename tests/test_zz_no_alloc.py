"""The allocation-free GEMM entry point, called through its exported C symbol.

Some embedders of the kernel library cannot let a library call reach the CUDA allocator: their process has given
all device memory to its own pool, or the call sits in a latency-critical loop where an allocation would take the
driver lock and may synchronise the device. ``mstar_gemm_bf16_noalloc`` keeps its split-K scratch in a device
array inside the library instead. This test drives that symbol directly with ctypes (raw pointers, no Python
wrapper in between) and requires its output to agree with the regular entry point's output for the same problem
(within the tolerance the GEMM tests use: the two sum the split-K partials in a different order), twice in a row,
because the second call reuses the scratch that the first one left behind.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

from mstar_b200.ops import _lib, gemm

pytestmark = pytest.mark.gpu


def _call_noalloc(x, w, out):
    lib = _lib.kernels()
    fn = lib.mstar_gemm_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    M, K = x.shape
    N = w.shape[0]
    rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), out.stride(0),
            torch.cuda.current_stream().cuda_stream)
    return rc, lib.mstar_last_error().decode(errors="replace")


@pytest.mark.parametrize("M,N,K", [(32, 512, 8192), (64, 3072, 3072), (300, 1024, 512)])
def test_noalloc_entry_matches_regular_entry_twice(M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    want = gemm.linear(x, w)
    ref = gemm.linear_ref(x, w)
    tol = 2e-2 * max(1.0, ref.float().abs().max().item())
    for attempt in range(2):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc, err = _call_noalloc(x, w, out)
        assert rc == 0, err
        torch.cuda.synchronize()
        assert (out.float() - want.float()).abs().max().item() <= tol, f"call {attempt} differs from the regular entry"
        assert (out.float() - ref.float()).abs().max().item() <= tol


def test_noalloc_entry_refuses_plans_beyond_its_scratch():
    # 1280 x 1792 x 8192 plans 70 tiles of 128 x 256 with two K splits: 18.4 MB of fp32 partial tiles, more than the
    # 16 MiB array inside the library. The entry point must say so on the host and launch nothing.
    M, N, K = 1280, 1792, 8192
    plan = gemm.gemm_plan(M, N, K)
    assert plan["ws_bytes"] > (16 << 20), plan
    x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    rc, err = _call_noalloc(x, w, out)
    assert rc != 0 and "scratch" in err, (rc, err)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "a refused call must not touch its output"
