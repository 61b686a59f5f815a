"""Four CPU (gloo) ranks as a tp2 x sp2 instance of the dual-pathway transformer: prefix prefill over the whole
instance + one packed two-branch denoising forward must equal the single-rank result."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mstar_b200.engine.cache_manager import BatchedCacheManager  # noqa: E402
from mstar_b200.engine.kv_store import KVCacheConfig  # noqa: E402
from mstar_b200.models.cosmos3 import Cosmos3Transformer  # noqa: E402
from mstar_b200.models.decoder import DecoderConfig  # noqa: E402
from mstar_b200.models.dit import grid_positions  # noqa: E402
from mstar_b200.parallel.comm import CommGroup, init_from_env  # noqa: E402


def run(tp, sp, shards, ids, neg, tok, pos):
    cfg = DecoderConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=16, intermediate_size=128,
                        vocab_size=512, qk_norm=True, mrope_sections=[2, 3, 3], has_lm_head=False, dtype=torch.float32)
    m = Cosmos3Transformer(cfg, 4, tp=tp, sp=sp).init_random(0)
    kvc = KVCacheConfig(2, 4 // shards, 16, max_seq_len=64, max_num_pages=16, page_size=8, num_qo_heads=4 // shards,
                        dtype=torch.float32)
    cm = BatchedCacheManager(kvc, "cpu", max_batch=4, max_tokens=256, n_pos_axes=3)
    ctx = cm.plan(["r", "r"], [ids.numel(), neg.numel()], labels=["main", "uncond"], causal=True)
    m.und.forward_hidden(m.und.embed(torch.cat([ids, neg])), ctx)
    cm.advance_seq_lens(ctx)
    S = tok.shape[0]
    gctx = cm.plan(["r", "r"], [S, S], labels=["main", "uncond"], causal=False, write_cache=False)
    return m.denoise(tok, pos, 640.0, 2, gctx, m.proj_out_w, m.proj_out_b)


def main():
    world = init_from_env("gloo")
    R = world.rank
    assert world.size == 4
    groups = {}
    for tup in ([0, 1], [2, 3], [0, 2], [1, 3], [0, 2, 1, 3]):
        g = dist.new_group(tup)
        if R in tup:
            groups[tuple(tup)] = CommGroup(g, tup, R)
    tp = groups[(0, 1)] if R < 2 else groups[(2, 3)]
    sp = groups[(0, 2)] if R % 2 == 0 else groups[(1, 3)]
    tp.instance = sp.instance = groups[(0, 2, 1, 3)]
    gen = torch.Generator().manual_seed(5)
    ids, neg = torch.randint(0, 512, (9,), generator=gen), torch.randint(0, 512, (4,), generator=gen)
    tok = torch.randn(2 * 3 * 3 + 1, 64, generator=gen)[:18]
    pos = grid_positions(2, 3, 3, "cpu", (9, 9, 9))
    out = run(tp, sp, 4, ids, neg, tok, pos)
    ref = run(CommGroup.trivial(), CommGroup.trivial(), 1, ids, neg, tok, pos)
    err = (out - ref).abs().max().item()
    assert err < 1e-3 * max(1.0, ref.abs().max().item()), err
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
