"""DiT family on the GPU: bf16 kernels against the same modules run in fp32 on the CPU (the ops' oracles)."""
import copy
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _to(module, device, dtype):
    m = copy.deepcopy(module)
    for p in m.parameters():
        p.data = p.data.to(device=device, dtype=dtype if p.dtype != torch.float32 or dtype == torch.float32 else p.dtype)
    return m


def test_attn_merge_kernel_matches_reference():
    from mstar_b200.ops import attention as A
    g = torch.Generator().manual_seed(0)
    T, H, D = 777, 6, 128
    oa, ob = torch.randn(T, H, D, generator=g), torch.randn(T, H, D, generator=g)
    la, lb = torch.randn(T, H, generator=g) * 3, torch.randn(T, H, generator=g) * 3
    la[5] = -math.inf
    lb[9] = -math.inf
    la[11], lb[11] = -math.inf, -math.inf
    ref, lref = A.attn_merge_ref(oa.bfloat16(), la, ob.bfloat16(), lb)
    out, lse = A.attn_merge(oa.bfloat16().cuda(), la.cuda(), ob.bfloat16().cuda(), lb.cuda(), lse=True)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 0.03
    fin = torch.isfinite(lref)
    assert (lse.cpu()[fin] - lref[fin]).abs().max().item() < 1e-3 and torch.isinf(lse.cpu()[~fin]).all()


def test_gated_residual_vectorised():
    from mstar_b200.ops import elementwise as E
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(96, 256, generator=g).bfloat16(), torch.randn(96, 256, generator=g).bfloat16()
    gate = torch.randn(3, 6, 256, generator=g).bfloat16()[:, 2]          # strided modulation slice
    ref = E.gated_residual_ref(x, y, gate)
    out = E.gated_residual(x.cuda(), y.cuda(), gate.cuda())
    assert (out.float().cpu() - ref.float()).abs().max().item() < 0.02
    out = E.gated_residual(x.cuda(), y.cuda(), None)
    assert (out.float().cpu() - (x.float() + y.float())).abs().max().item() < 0.02


def test_adaln_dit_gpu_matches_cpu():
    from mstar_b200.models.dit import AdaLNDiT, DiTConfig
    kw = dict(hidden_size=256, num_layers=2, num_heads=4, head_dim=64, ffn_dim=512, in_channels=4, out_channels=4,
              text_dim=64, text_len=16, rope_axes=(16, 24, 24))
    ref = AdaLNDiT(DiTConfig(dtype=torch.float32, **kw)).init_random(2)
    gpu = AdaLNDiT(DiTConfig(dtype=torch.bfloat16, **kw), device="cuda")
    for (n, p), (_, q) in zip(ref.named_parameters(), gpu.named_parameters()):
        q.data.copy_(p.data.to(q.dtype))
        p.data.copy_(q.data.float().cpu() if p.dtype == torch.float32 and q.dtype != torch.float32 else p.data)
    g = torch.Generator().manual_seed(0)
    lat = torch.randn(2, 4, 3, 16, 16, generator=g)
    text = torch.randn(16 + 9, 64, generator=g)
    ts = torch.tensor([900.0, 900.0])
    r = ref(lat, ts, ref.encode_context(text), [16, 9])
    o = gpu(lat.cuda(), ts.cuda(), gpu.encode_context(text.cuda()), [16, 9]).float().cpu()
    rel = (o - r).norm() / r.norm()
    assert rel.item() < 0.03, rel.item()


def test_mot_tower_prefix_plus_fresh_gpu_matches_cpu():
    from mstar_b200.engine.cache_manager import BatchedCacheManager
    from mstar_b200.engine.kv_store import KVCacheConfig
    from mstar_b200.models.cosmos3 import Cosmos3Transformer
    from mstar_b200.models.decoder import DecoderConfig
    from mstar_b200.models.dit import grid_positions

    def run(device, dtype):
        cfg = DecoderConfig(hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                            intermediate_size=512, vocab_size=512, qk_norm=True, mrope_sections=[8, 12, 12],
                            has_lm_head=False, dtype=dtype)
        m = Cosmos3Transformer(cfg, 4, device=device).init_random(0)
        kvc = KVCacheConfig(2, 2, 64, max_seq_len=256, max_num_pages=16, page_size=16, num_qo_heads=4, dtype=dtype)
        cm = BatchedCacheManager(kvc, device, max_batch=4, max_tokens=1024, n_pos_axes=3)
        gen = torch.Generator().manual_seed(5)
        ids, neg = torch.randint(0, 512, (37,), generator=gen), torch.randint(0, 512, (5,), generator=gen)
        ctx = cm.plan(["r", "r"], [37, 5], labels=["main", "uncond"], causal=True, group=2)
        m.und.forward_hidden(m.und.embed(torch.cat([ids, neg]).to(device)), ctx)
        cm.advance_seq_lens(ctx)
        S = 2 * 8 * 8
        tok = (torch.randn(S, 256, generator=gen) * 0.5).to(device=device, dtype=dtype)
        pos = grid_positions(2, 8, 8, device, (37, 37, 37))
        gctx = cm.plan(["r", "r"], [S, S], labels=["main", "uncond"], causal=False, write_cache=False, group=2)
        return m.denoise(tok, pos, 500.0, 2, gctx, m.proj_out_w, m.proj_out_b).float().cpu()
    r = run("cpu", torch.float32)
    o = run("cuda", torch.bfloat16)
    rel = (o - r).norm() / r.norm()
    assert rel.item() < 0.04, rel.item()
