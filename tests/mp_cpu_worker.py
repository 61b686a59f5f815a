"""CPU (gloo) ranks: CommGroup wrappers, Ulysses exchange fallback, TP decoder == single-rank decoder."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mstar_b200.parallel.comm import init_from_env  # noqa: E402
from mstar_b200.parallel.sequence_parallel import UlyssesExchange, gather_sequence, scatter_sequence  # noqa: E402


def main():
    g = init_from_env("gloo")
    W, R = g.size, g.rank
    x = torch.full((4,), float(R + 1))
    assert g.all_reduce(x.clone()).tolist() == [3.0] * 4
    assert g.all_gather(torch.tensor([float(R)]), 0).tolist() == [0.0, 1.0]
    rs = g.reduce_scatter(torch.arange(4.0) + R)
    assert rs.tolist() == ([1.0, 3.0] if R == 0 else [5.0, 7.0])
    a2a = g.all_to_all(torch.tensor([10.0 * R, 10.0 * R + 1]))
    assert a2a.tolist() == [0.0 + R, 10.0 + R]
    # sequence scatter / gather with an uneven split
    gen = torch.Generator().manual_seed(0)
    full = torch.randn(7, 4, 8, generator=gen)
    mine = scatter_sequence(full, g)
    assert torch.equal(gather_sequence(mine, g, 7), full)
    ex = UlyssesExchange(g, 7, 4, 4, 8, torch.float32)
    q, k, v = ex.to_heads(mine, mine * 2, mine * 3)
    assert torch.equal(q, full[:, R * 2:(R + 1) * 2]) and torch.equal(v, 3 * full[:, R * 2:(R + 1) * 2])
    back = ex.to_sequence(q)
    assert torch.equal(back, mine)
    # tensor-parallel tiny decoder: both ranks produce the single-rank logits
    from mstar_b200.engine.cache_manager import BatchedCacheManager
    from mstar_b200.engine.kv_store import KVCacheConfig
    from mstar_b200.models import tiny
    ref_model = tiny.build_tiny()
    tp_model = tiny.build_tiny(tp=g)
    ids = torch.randint(0, 32000, (11,), generator=gen)

    def logits(m, kvh):
        kvc = KVCacheConfig(2, kvh, 64, max_seq_len=64, max_num_pages=8, page_size=16, num_qo_heads=4, dtype=torch.float32)
        cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=64)
        cm.add_request("r")
        ctx = cm.plan(["r"], [11])
        return m(ctx, input_ids=ids)
    a, b = logits(ref_model, 2), logits(tp_model, 1)
    assert (a - b).abs().max().item() < 1e-3, (a - b).abs().max().item()
    # MoE decoder: column-sharded experts (TP) and expert-sharded experts over the same group both match one rank
    from mstar_b200.models.decoder import DecoderConfig, DecoderLM
    from mstar_b200.parallel.comm import CommGroup
    for ep_mode in (False, True):
        cfg = DecoderConfig(hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8, intermediate_size=64,
                            vocab_size=64, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16,
                            shared_expert_intermediate_size=32, moe_expert_parallel=ep_mode, dtype=torch.float32)
        one = DecoderLM(cfg, tp=CommGroup.trivial()).init_random(3)
        two = DecoderLM(cfg, tp=g).init_random(3)
        mids = torch.randint(0, 64, (9,), generator=gen)

        def mlogits(m, kvh):
            kvc = KVCacheConfig(2, kvh, 8, max_seq_len=64, max_num_pages=8, page_size=16, num_qo_heads=4, dtype=torch.float32)
            cm = BatchedCacheManager(kvc, "cpu", max_batch=2, max_tokens=64)
            return m(cm.plan(["r"], [9]), input_ids=mids)
        d = (mlogits(one, 2) - mlogits(two, 1)).abs().max().item()
        assert d < 1e-4, (ep_mode, d)
    # AdaLN DiT (Wan2.2-class): heads and MLP columns cut over the ranks, q / k norms over all heads through an
    # exchange of the sums of squares; same weights by seed, same velocity as one rank
    from mstar_b200.models.dit import AdaLNDiT, DiTConfig
    dc = DiTConfig(hidden_size=48, num_layers=2, num_heads=4, head_dim=12, ffn_dim=64, in_channels=4, out_channels=4,
                   text_dim=16, text_len=8, freq_dim=32, dtype=torch.float32)
    one = AdaLNDiT(dc).init_random(5)
    two = AdaLNDiT(dc, tp=g).init_random(5)
    assert two.blocks[0].qkv_w.shape == (3 * 24, 48) and one.blocks[0].qkv_w.shape == (3 * 48, 48)
    assert torch.equal(two.blocks[1].ffn2_w, one.blocks[1].ffn2_w[:, R * 32:(R + 1) * 32])
    lat = torch.randn(2, 4, 2, 4, 6, generator=gen)
    text = torch.randn(2 * 8, 16, generator=gen)
    ts = torch.tensor([[900.0, 0.0], [500.0, 500.0]])
    with torch.no_grad():
        want = one(lat, ts, one.encode_context(text), [8, 8])
        got = two(lat, ts, two.encode_context(text), [8, 8])
    assert (got - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item()), (got - want).abs().max().item()
    # the same model sequence-parallel: every rank keeps one guidance branch's rows, attention swaps rows for heads
    sq = AdaLNDiT(dc, sp=g).init_random(5)
    with torch.no_grad():
        got = sq(lat, torch.tensor([900.0, 500.0]), sq.encode_context(text), [8, 8])
        want = one(lat, torch.tensor([900.0, 500.0]), one.encode_context(text), [8, 8])
    assert (got - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item()), (got - want).abs().max().item()
    with torch.no_grad():                                  # per-frame timesteps: a rank's rows are whole groups
        got = sq(lat, ts, sq.encode_context(text), [8, 8])
        want = one(lat, ts, one.encode_context(text), [8, 8])
    assert (got - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item()), (got - want).abs().max().item()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
