"""Engine building blocks on CPU: page allocator under threads, label snapshots, host offload / reload, KV engine
cleanup and allocation-failure envelope, sampler determinism, media containers, tensor store ownership."""
import io
import struct
import threading

import pytest
import torch

from mstar_b200.engine.cache_manager import BatchedCacheManager
from mstar_b200.engine.kv_store import AllocationFailedError, KVCacheConfig, PageAllocator, PagedAllocationManager


def test_page_allocator_threads_conserve_pages():
    alloc = PageAllocator(512)
    errors, held = [], [[] for _ in range(8)]

    def work(i):
        g = torch.Generator().manual_seed(i)
        try:
            for _ in range(400):
                if held[i] and torch.rand(1, generator=g).item() < 0.5:
                    alloc.free(held[i].pop())
                else:
                    try:
                        held[i].append(alloc.allocate(int(torch.randint(1, 9, (1,), generator=g))))
                    except AllocationFailedError:
                        pass
        except Exception as e:  # noqa: BLE001
            errors.append(e)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errors
    out = [p for h in held for blk in h for p in blk]
    assert len(out) == len(set(out))                       # no page handed out twice
    assert alloc.num_free + len(out) == 512                # none lost
    for h in held:
        for blk in h:
            alloc.free(blk)
    assert alloc.num_free == 512


def _kvc(**kw):
    base = dict(num_layers=2, num_kv_heads=2, head_dim=8, max_seq_len=128, max_num_pages=8, page_size=8, num_qo_heads=2,
                dtype=torch.float32)
    base.update(kw)
    return KVCacheConfig(**base)


def test_label_snapshot_copies_pages_and_offload_roundtrip():
    m = PagedAllocationManager(_kvc(cpu_offload_pages=8), "cpu")
    m.add_request("r")
    m.alloc_batch([("r", "main", 12)])
    st = m.get_state("r", "main")
    st.seq_len = 12
    for layer in m.kv_layers:
        layer[st.pages] = torch.randn_like(layer[st.pages])
    m.copy_label("r", "main", "cfg")
    c = m.get_state("r", "cfg")
    assert c.seq_len == 12 and set(c.pages).isdisjoint(st.pages)
    assert all(torch.equal(l[c.pages], l[st.pages]) for l in m.kv_layers)
    before = [l[st.pages].clone() for l in m.kv_layers]
    free0 = m.num_free_pages
    freed = m.offload_request("r")
    assert freed == 4 and m.is_offloaded("r") and m.num_free_pages == free0 + 4
    m.reload_request("r")
    st = m.get_state("r", "main")
    assert not m.is_offloaded("r") and all(torch.equal(l[st.pages], b) for l, b in zip(m.kv_layers, before))
    m.remove_request("r")
    assert m.num_free_pages == m.total_pages


def test_plan_raises_allocation_failed_and_leaves_the_pool_consistent():
    cm = BatchedCacheManager(_kvc(max_num_pages=2), "cpu", max_batch=2, max_tokens=32)
    cm.add_request("a")
    cm.plan(["a"], [16])
    cm.add_request("b")
    with pytest.raises(AllocationFailedError):
        cm.plan(["b"], [4])
    assert cm.alloc.pages_of("b") == 0
    cm.remove_request("a")
    assert cm.alloc.num_free_pages == 2
    cm.plan(["b"], [4])          # now it fits


def test_sampler_reference_is_seeded_and_respects_top_k_and_penalty():
    from mstar_b200.ops.sampling import sample_ref
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(3, 50, generator=g)
    a = sample_ref(logits, [0.8] * 3, [5] * 3, [0.9] * 3, [1.0] * 3, [7, 8, 9], [0, 0, 0], None, None)
    b = sample_ref(logits, [0.8] * 3, [5] * 3, [0.9] * 3, [1.0] * 3, [7, 8, 9], [0, 0, 0], None, None)
    c = sample_ref(logits, [0.8] * 3, [5] * 3, [0.9] * 3, [1.0] * 3, [7, 8, 9], [1, 1, 1], None, None)
    assert torch.equal(a, b) and a.shape == c.shape
    top5 = logits.topk(5, dim=-1).indices
    assert all(int(a[i]) in top5[i].tolist() for i in range(3))
    greedy = sample_ref(logits, [0.0] * 3, [0] * 3, [1.0] * 3, [1.0] * 3, [0] * 3, [0] * 3, None, None)
    assert torch.equal(greedy, logits.argmax(-1))
    seen = torch.zeros(3, 50, dtype=torch.uint8)
    seen[torch.arange(3), logits.argmax(-1)] = 1
    pen = sample_ref(logits, [0.0] * 3, [0] * 3, [1.0] * 3, [100.0] * 3, [0] * 3, [0] * 3, seen, None)
    assert not torch.equal(pen, logits.argmax(-1))


def test_media_containers():
    from mstar_b200.api_server import media_io as M
    pcm = M.float_to_pcm16(torch.linspace(-1, 1, 480))
    wav = M.pcm16_to_wav(pcm, 24000)
    assert wav[:4] == b"RIFF" and wav[8:12] == b"WAVE" and struct.unpack("<I", wav[24:28])[0] == 24000
    t, sr = M.read_wav(wav)
    assert sr == 24000 and t.numel() == 480 and abs(float(t[-1]) - 1.0) < 1e-3
    png = M.tensor_to_png(torch.rand(3, 9, 7))
    from PIL import Image
    assert Image.open(io.BytesIO(png)).size == (7, 9)
    frames = torch.rand(4, 3, 16, 24)
    avi = M.frames_to_avi(frames, fps=12, audio_pcm=pcm, sample_rate=24000)
    assert avi[:4] == b"RIFF" and avi[8:12] == b"AVI " and avi.count(b"00dc") >= 4 and b"01wb" in avi and b"idx1" in avi
    assert struct.unpack("<I", avi[4:8])[0] == len(avi) - 8


def test_tensor_store_ownership_is_constant_time_and_adopt_keeps_results_alive():
    from mstar_b200.communication.tensors import TensorStore
    s = TensorStore("w")
    ids = [s.put(f"req{i % 5}", torch.zeros(1)) for i in range(50)]
    assert s.owner_of(ids[7]) == "req2"
    s.adopt(ids[7], "req2#emit")
    assert s.remove_request("req2") == 9 and s.get(ids[7]) is not None      # the adopted tensor survives teardown
    assert s.dereference(ids[7], 2) and s.get(ids[7]) is None and s.owner_of(ids[7]) is None
    assert s.dereference(ids[0]) and len(s) == 50 - 10 - 1
