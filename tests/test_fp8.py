"""Block-scaled fp8 projections and expert GEMMs: quantisers, the CPU oracle, and (GPU tier) the tcgen05 kernels
against that oracle."""
import pytest
import torch

from mstar_b200.ops import gemm, gemm_fp8
from mstar_b200.ops import moe as moe_ops


def test_weight_and_activation_quantisers_round_trip():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(300, 520, generator=g) * 0.05
    q = gemm_fp8.quantize_weight(w)
    assert q.data.dtype == torch.float8_e4m3fn and q.scale.shape == (3, 5)
    assert (q.dequant() - w).abs().max() <= 0.07 * w.abs().max()          # e4m3: 3 mantissa bits
    x = torch.randn(7, 520, generator=g)
    x8, st = gemm_fp8.quantize_act_ref(x)
    assert st.shape == (5, 7)
    assert (gemm_fp8._dequant_act(x8, st) - x).abs().max() <= 0.07 * x.abs().max()


def test_fp8_linear_oracle_is_close_to_bf16():
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(9, 384, generator=g) * 0.5).bfloat16()
    w = (torch.randn(256, 384, generator=g) * 0.05).bfloat16()
    y8 = gemm_fp8.linear_fp8(x, gemm_fp8.quantize_weight(w)).float()
    y = gemm.linear_ref(x, w).float()
    assert (y8 - y).abs().max() < 0.06 * y.abs().max() + 0.02


def test_fp8_moe_oracle_is_close_to_bf16():
    g = torch.Generator().manual_seed(2)
    T, H, E, I, k = 11, 256, 8, 128, 2
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    router = torch.randn(E, H, generator=g) * 0.1
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
    logits = x.float() @ router.t()
    y = moe_ops.fused_moe(x, logits, w13, w2, k).float()
    y8 = moe_ops.fused_moe(x, logits, gemm_fp8.quantize_weight(w13), gemm_fp8.quantize_weight(w2), k).float()
    assert (y8 - y).abs().max() < 0.08 * y.abs().max() + 0.02


def test_qwen3_omni_small_accepts_fp8_experts():
    from mstar_b200.models.registry import get_model_class
    m = get_model_class("qwen3_omni")(small=True, fp8_experts=True, skip_weight_loading=True)
    sub = m.get_submodule("Thinker", "cpu")
    assert sub is not None


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(64, 512, 1024), (7, 384, 256), (128, 256, 2048), (300, 512, 1024), (1000, 384, 640)])
def test_fp8_gemm_kernel_matches_oracle(M, N, K):
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    wq = gemm_fp8.quantize_weight(w)
    ref = gemm_fp8.linear_fp8_ref(x, wq).float()
    wq_d = gemm_fp8.Fp8Weight(wq.data.cuda(), wq.scale.cuda())
    got = gemm_fp8.linear_fp8(x.cuda(), wq_d).float().cpu()
    assert (got - ref).abs().max() < 0.02 * ref.abs().max() + 0.02


@pytest.mark.gpu
def test_fp8_activation_quantiser_kernel():
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(37, 640, generator=g)).bfloat16()
    q_ref, s_ref = gemm_fp8.quantize_act_ref(x)
    q, s = gemm_fp8.quantize_act(x.cuda())
    assert torch.allclose(s[:, :37].cpu(), s_ref, rtol=1e-5, atol=0)
    d = (q.float().cpu() - q_ref.float()).abs()
    assert d.max() <= 32.0 and (d > 0).float().mean() < 0.02        # a handful of values on a rounding boundary


@pytest.mark.gpu
def test_fp8_gemm_kernel_swiglu_and_residual():
    g = torch.Generator().manual_seed(9)
    M, N, K = 48, 512, 768
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    res = torch.randn(M, N, generator=g).bfloat16()
    wq = gemm_fp8.quantize_weight(w)
    wq_d = gemm_fp8.Fp8Weight(wq.data.cuda(), wq.scale.cuda())
    ref = gemm_fp8.linear_fp8_ref(x, wq, epilogue=gemm.EPILOGUE_SWIGLU).float()
    got = gemm_fp8.linear_fp8(x.cuda(), wq_d, epilogue=gemm.EPILOGUE_SWIGLU).float().cpu()
    assert (got - ref).abs().max() < 0.02 * ref.abs().max() + 0.02
    ref = gemm_fp8.linear_fp8_ref(x, wq, residual=res).float()
    got = gemm_fp8.linear_fp8(x.cuda(), wq_d, residual=res.cuda()).float().cpu()
    assert (got - ref).abs().max() < 0.02 * ref.abs().max() + 0.03


@pytest.mark.gpu
@pytest.mark.parametrize("T", [5, 70, 600])
def test_fp8_moe_kernel_matches_oracle(T):
    g = torch.Generator().manual_seed(T)
    H, E, I, k = 512, 16, 256, 4
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16()
    router = torch.randn(E, H, generator=g) * 0.1
    w13 = gemm_fp8.quantize_weight((torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16())
    w2 = gemm_fp8.quantize_weight((torch.randn(E, H, I, generator=g) * 0.05).bfloat16())
    logits = x.float() @ router.t()
    ref = moe_ops.fused_moe(x, logits, w13, w2, k).float()
    dev = lambda q: gemm_fp8.Fp8Weight(q.data.cuda(), q.scale.cuda())
    got = moe_ops.fused_moe(x.cuda(), logits.cuda(), dev(w13), dev(w2), k).float().cpu()
    assert (got - ref).abs().max() < 0.03 * ref.abs().max() + 0.03
