"""Fused MoE (routing + grouped tcgen05 GEMMs) against the dense per-expert oracle, at toy and thinker shapes."""
import pytest
import torch

from mstar_b200.ops import moe as M

pytestmark = pytest.mark.gpu


def _case(T, H, E, I, top_k, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    router = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16).cuda()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).cuda()
    return x, router, w13, w2


@pytest.mark.parametrize("T,H,E,I,k", [(5, 256, 8, 128, 2), (64, 2048, 128, 768, 8), (300, 512, 16, 256, 4),
                                       (1, 2048, 128, 768, 8)])
def test_fused_moe_matches_dense_oracle(T, H, E, I, k):
    x, router, w13, w2 = _case(T, H, E, I, k)
    logits = torch.nn.functional.linear(x.float(), router.float())
    out = M.fused_moe(x, logits, w13, w2, k)
    ref = M.moe_ref(x, router, w13, w2, k)
    err = (out.float() - ref.float()).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.float().abs().max().item()), err
    ids, w = M.route_ref(logits, k)
    ws = M._workspace(x.device, T, k, E, H, I, M.choose_block_rows(T * k, E))
    assert torch.equal(ws.topk_ids.sort(-1).values, ids.cuda().sort(-1).values)


def test_expert_range_shards_sum_to_full():
    T, H, E, I, k = 32, 512, 16, 256, 4
    x, router, w13, w2 = _case(T, H, E, I, k, seed=3)
    logits = torch.nn.functional.linear(x.float(), router.float())
    full = M.fused_moe(x, logits, w13, w2, k)
    a = M.fused_moe(x, logits, w13[:8].contiguous(), w2[:8].contiguous(), k, expert_range=(0, 8))
    b = M.fused_moe(x, logits, w13[8:].contiguous(), w2[8:].contiguous(), k, expert_range=(8, 16))
    assert (a.float() + b.float() - full.float()).abs().max().item() < 3e-2
