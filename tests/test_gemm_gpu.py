"""tcgen05 GEMM against the fp32 PyTorch oracle (decode/swapped, split-K, prefill tiles, epilogues)."""
import pytest
import torch

from mstar_b200.ops import gemm

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _check(y, ref, K):
    err = (y.float() - ref.float()).abs().max().item()
    tol = 2e-2 * max(1.0, ref.float().abs().max().item())
    assert err <= tol, f"max err {err} > {tol}"


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (7, 384, 512), (16, 3072, 3072), (64, 5120, 3072),
                                   (64, 3072, 8192), (100, 1000, 264), (128, 1024, 1024)])
def test_gemm_decode_shapes(M, N, K):
    x, w = _rand((M, K), 1.0, 1), _rand((N, K), 0.05, 2)
    y = gemm.linear(x, w)
    _check(y, gemm.linear_ref(x, w), K)


@pytest.mark.parametrize("M,N,K", [(129, 256, 128), (512, 1024, 768), (1000, 3072, 1024), (4096, 2048, 2048)])
def test_gemm_prefill_shapes(M, N, K):
    x, w = _rand((M, K), 1.0, 3), _rand((N, K), 0.05, 4)
    y = gemm.linear(x, w)
    _check(y, gemm.linear_ref(x, w), K)


@pytest.mark.parametrize("M", [8, 64, 300])
def test_gemm_epilogues(M):
    N, K = 1024, 512
    x, w = _rand((M, K), 1.0, 5), _rand((N, K), 0.05, 6)
    b = _rand((N,), 0.5, 7)
    r = _rand((M, N), 1.0, 8)
    y = gemm.linear(x, w, bias=b, residual=r)
    _check(y, gemm.linear_ref(x, w, b, r), K)
    y = gemm.linear(x, w, epilogue=gemm.EPILOGUE_SWIGLU)
    assert y.shape == (M, N // 2)
    _check(y, gemm.linear_ref(x, w, epilogue=gemm.EPILOGUE_SWIGLU), K)
    y = gemm.linear(x, w, bias=b, epilogue=gemm.EPILOGUE_GELU, out_dtype=torch.float32)
    assert y.dtype == torch.float32
    _check(y, gemm.linear_ref(x, w, b, epilogue=gemm.EPILOGUE_GELU, out_dtype=torch.float32), K)


def test_gemm_splitk_deterministic_and_counter_reset():
    M, N, K = 32, 512, 8192
    x, w = _rand((M, K), 1.0, 9), _rand((N, K), 0.02, 10)
    plan = gemm.gemm_plan(M, N, K)
    assert plan["splits"] > 1 and plan["ws_bytes"] > 0
    y1 = gemm.linear(x, w)
    y2 = gemm.linear(x, w)
    assert torch.equal(y1, y2)
    _check(y1, gemm.linear_ref(x, w), K)
    y3 = gemm.linear(x, w, force_splits=1)
    _check(y3, gemm.linear_ref(x, w), K)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,epilogue", [(64, 3072, 3072, 0), (64, 3072, 8192, 0), (64, 16384, 3072, 1),
                                             (17, 5120, 3072, 0), (128, 1024, 512, 0)])
def test_gemm_with_folded_norms_matches_the_pytorch_statement(M, N, K, epilogue):
    """Decode-layout projection with RMSNorms folded in: output rows scaled by 1 / rms from the incoming sums of
    squares, residual added in place, sums of squares of the stored bf16 rows accumulated (one atomic per row and
    tile slice), the other accumulator cleared."""
    from mstar_b200.ops import gemm
    torch.manual_seed(M + N)
    dev = "cuda"
    x = (torch.randn(M, K, device=dev) * 2).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev).to(torch.bfloat16) if epilogue == 0 and N == 5120 else None
    n_out = N // 2 if epilogue else N
    ss_in = (x.float() ** 2).sum(-1).contiguous()
    for consumer in (True, False):
        if consumer:        # scales by 1 / rms of the activation rows; SwiGLU or plain
            fn = gemm.FoldedNorm(K, 1e-5, ss_in=ss_in)
            ref_fn = gemm.FoldedNorm(K, 1e-5, ss_in=ss_in.clone())
            got = gemm.linear(x, w, bias=bias, epilogue=epilogue, norm=fn)
            want = ref_fn.linear_ref(x, w, bias, None, epilogue, None)
            assert got.shape == (M, n_out)
            err = (got.float() - want.float()).abs().max().item()
            assert err <= 0.02 * max(1.0, want.float().abs().max().item()), err
        elif epilogue == 0:  # adds into the residual stream in place, accumulates its sums of squares, clears `other`
            r = torch.randn(M, N, device=dev).to(torch.bfloat16)
            r_ref = r.clone()
            acc, other = torch.zeros(128, device=dev), torch.full((128,), 7.0, device=dev)
            acc_ref, other_ref = acc.clone(), other.clone()
            gemm.linear(x, w, bias=bias, residual=r, out=r, norm=gemm.FoldedNorm(N, 1e-5, ss_out=acc, ss_zero=other))
            gemm.FoldedNorm(N, 1e-5, ss_out=acc_ref, ss_zero=other_ref).linear_ref(x, w, bias, r_ref, 0, r_ref)
            torch.cuda.synchronize()
            assert (r.float() - r_ref.float()).abs().max().item() <= 0.03 * max(1.0, r_ref.float().abs().max().item())
            assert float(other.abs().sum()) == 0.0
            # the accumulator holds the sums of squares of what was STORED
            stored = (r.float() ** 2).sum(-1)
            assert torch.allclose(acc[:M], stored, rtol=2e-3, atol=1e-2), (acc[:M] - stored).abs().max()
            assert float(acc[M:].abs().sum()) == 0.0
