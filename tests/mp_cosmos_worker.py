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


def run(tp, sp, shards, ids, neg, tok, pos, device="cpu", dtype=torch.float32):
    k = 4 if device != "cpu" else 1          # GPU: 64-wide heads so that the tensor-core kernels run
    cfg = DecoderConfig(hidden_size=64 * k, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=16 * k,
                        intermediate_size=128 * k, vocab_size=512, qk_norm=True, mrope_sections=[2 * k, 3 * k, 3 * k],
                        has_lm_head=False, dtype=dtype)
    m = Cosmos3Transformer(cfg, 4, tp=tp, sp=sp, device=device).init_random(0)
    ids, neg, tok, pos = ids.to(device), neg.to(device), tok.to(device=device, dtype=dtype), pos.to(device)
    kvc = KVCacheConfig(2, 4 // shards, 16 * k, max_seq_len=64, max_num_pages=16, page_size=8 if device == "cpu" else 16,
                        num_qo_heads=4 // shards, dtype=dtype)
    cm = BatchedCacheManager(kvc, device, max_batch=4, max_tokens=256, n_pos_axes=3)
    ctx = cm.plan(["r", "r"], [ids.numel(), neg.numel()], labels=["main", "uncond"], causal=True)
    m.und.forward_hidden(m.und.embed(torch.cat([ids, neg])), ctx)
    cm.advance_seq_lens(ctx)
    S = tok.shape[0]
    gctx = cm.plan(["r", "r"], [S, S], labels=["main", "uncond"], causal=False, write_cache=False)
    return m.denoise(tok, pos, 640.0, 2, gctx, m.proj_out_w, m.proj_out_b)


def main():
    gpu = torch.cuda.is_available() and torch.cuda.device_count() >= 4 and os.environ.get("MSTAR_TEST_BACKEND") != "gloo"
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    world = init_from_env("nccl" if gpu else "gloo")
    R = world.rank
    assert world.size == 4
    device, dtype = (f"cuda:{torch.cuda.current_device()}", torch.bfloat16) if gpu else ("cpu", torch.float32)
    groups = {}
    for tup in ([0, 1], [2, 3], [0, 2], [1, 3], [0, 2, 1, 3]):
        g = dist.new_group(tup)
        if R in tup:
            groups[tuple(tup)] = CommGroup(g, tup, R)
            if gpu:      # peer-memory collectives over the symmetric heap (plain loads / stores; NVLS off in the test env)
                from mstar_b200.parallel.symm import attach_symmetric_heap
                attach_symmetric_heap(groups[tuple(tup)], torch.device(device))
    tp = groups[(0, 1)] if R < 2 else groups[(2, 3)]
    sp = groups[(0, 2)] if R % 2 == 0 else groups[(1, 3)]
    tp.instance = sp.instance = groups[(0, 2, 1, 3)]
    gen = torch.Generator().manual_seed(5)
    ids, neg = torch.randint(0, 512, (9,), generator=gen), torch.randint(0, 512, (4,), generator=gen)
    H = 256 if gpu else 64
    tok = torch.randn(2 * 3 * 3 + 1, H, generator=gen)[:18] * 0.5
    pos = grid_positions(2, 3, 3, "cpu", (9, 9, 9))
    out = run(tp, sp, 4, ids, neg, tok, pos, device, dtype).float().cpu()
    ref = run(CommGroup.trivial(), CommGroup.trivial(), 1, ids, neg, tok, pos, device, dtype).float().cpu()
    if gpu:
        rel = ((out - ref).norm() / ref.norm()).item()
        assert rel < 0.05, rel
        print(f"rank {R}: tp2 x sp2 on GPUs matches one GPU, relative error {rel:.4f}", flush=True)
    else:
        err = (out - ref).abs().max().item()
        assert err < 1e-3 * max(1.0, ref.abs().max().item()), err
        # the AdaLN transformer (Wan2.2-class) on the same tp2 x sp2 mesh against one rank
        from mstar_b200.models.dit import AdaLNDiT, DiTConfig
        dc = DiTConfig(hidden_size=48, num_layers=2, num_heads=4, head_dim=12, ffn_dim=64, in_channels=4, out_channels=4,
                       text_dim=16, text_len=8, freq_dim=32, dtype=torch.float32)
        lat, text = torch.randn(2, 4, 2, 4, 6, generator=gen), torch.randn(16, 16, generator=gen)
        ts = torch.tensor([[900.0, 0.0], [500.0, 500.0]])
        one, mesh = AdaLNDiT(dc).init_random(5), AdaLNDiT(dc, tp=tp, sp=sp).init_random(5)
        with torch.no_grad():
            want = one(lat, ts, one.encode_context(text), [8, 8])
            got = mesh(lat, ts, mesh.encode_context(text), [8, 8])
        err = (got - want).abs().max().item()
        assert err < 1e-4 * max(1.0, want.abs().max().item()), err
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
