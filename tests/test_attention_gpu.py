"""tcgen05 attention kernel against the fp32 oracle: paged prefill/decode, split-KV, dense varlen, masks, GQA."""
import itertools

import pytest
import torch

from mstar_b200.ops import attention as A

pytestmark = pytest.mark.gpu


def _paged_case(q_lens, kv_lens, Hq, Hkv, D, page_size, seed=0):
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    T = sum(q_lens)
    q = (torch.randn(T, Hq, D, generator=g)).to(torch.bfloat16).cuda()
    pages_per = [(n + page_size - 1) // page_size for n in kv_lens]
    total = sum(pages_per) + 3
    cache = (torch.randn(total, 2, Hkv, page_size, D, generator=g)).to(torch.bfloat16).cuda()
    perm = torch.randperm(total, generator=g).tolist()
    idx, indptr = [], [0]
    for n in pages_per:
        idx += [perm.pop() for _ in range(n)]
        indptr.append(len(idx))
    dev = "cuda"
    plan = A.AttnPlan(
        q_indptr=torch.tensor([0] + list(itertools.accumulate(q_lens)), dtype=torch.int32, device=dev),
        kv_lens=torch.tensor(kv_lens, dtype=torch.int32, device=dev), batch=B, num_q_tokens=T,
        num_q_tiles=A.count_q_tiles(q_lens, Hq // Hkv),
        page_indptr=torch.tensor(indptr, dtype=torch.int32, device=dev),
        page_indices=torch.tensor(idx, dtype=torch.int32, device=dev))
    return q, cache, plan


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    assert err < tol, f"max err {err}"


@pytest.mark.parametrize("Hq,Hkv,D,ps", [(4, 2, 64, 16), (24, 8, 128, 128), (28, 4, 128, 64), (32, 4, 128, 128)])
def test_paged_decode(Hq, Hkv, D, ps):
    kv_lens = [1, 17, 128, 129, 700, 1300]
    q, cache, plan = _paged_case([1] * len(kv_lens), kv_lens, Hq, Hkv, D, ps)
    ref = A.attention_ref(q, plan, kv_cache=cache)
    _close(A.attention(q, plan, kv_cache=cache), ref)       # general kernel (q_len unknown)
    plan.max_q_len = 1                                       # swapped decode kernel when D == 128
    _close(A.attention(q, plan, kv_cache=cache), ref)


def test_decode_kernel_multi_token_window_and_splits():
    """Swapped decode kernel: 2 new tokens per request (causal inside the pair), sliding window, split-KV."""
    q, cache, plan = _paged_case([2, 1, 2], [500, 1, 1030], 24, 8, 128, 128, seed=21)
    plan.max_q_len = 2
    ref = A.attention_ref(q, plan, kv_cache=cache)
    _close(A.attention(q, plan, kv_cache=cache), ref)
    plan.splits = 4
    out = A.attention(q, plan, kv_cache=cache)
    _close(out, ref)
    assert torch.equal(out, A.attention(q, plan, kv_cache=cache))
    plan.window, plan.splits = 300, 1
    _close(A.attention(q, plan, kv_cache=cache), A.attention_ref(q, plan, kv_cache=cache))


@pytest.mark.parametrize("splits", [2, 5])
def test_paged_decode_split_kv(splits):
    kv_lens = [3000, 130, 1]
    q, cache, plan = _paged_case([1] * 3, kv_lens, 24, 8, 128, 128, seed=3)
    plan.splits = splits
    plan.max_q_len = 0
    out = A.attention(q, plan, kv_cache=cache)
    ref = A.attention_ref(q, plan, kv_cache=cache)
    _close(out, ref)
    out2 = A.attention(q, plan, kv_cache=cache)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("Hq,Hkv,D,ps", [(4, 2, 64, 16), (24, 8, 128, 128)])
def test_paged_prefill_causal(Hq, Hkv, D, ps):
    q_lens = [5, 64, 200, 31]
    kv_lens = [5, 64, 333, 431]     # last two extend an existing prefix
    q, cache, plan = _paged_case(q_lens, kv_lens, Hq, Hkv, D, ps, seed=5)
    out, lse = A.attention(q, plan, kv_cache=cache, lse=True)
    ref, lse_ref = A.attention_ref(q, plan, kv_cache=cache, lse=True)
    _close(out, ref)
    _close(lse, lse_ref, 5e-2)


def test_sliding_window():
    q, cache, plan = _paged_case([300, 1], [300, 900], 8, 2, 128, 128, seed=7)
    plan.window = 256
    _close(A.attention(q, plan, kv_cache=cache), A.attention_ref(q, plan, kv_cache=cache))


@pytest.mark.parametrize("causal", [False, True])
def test_dense_varlen(causal):
    g = torch.Generator().manual_seed(11)
    Hq, Hkv, D = 16, 16, 128
    q_lens, kv_lens = [700, 130], [700, 130]
    q = torch.randn(sum(q_lens), Hq, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(sum(kv_lens), Hkv, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(sum(kv_lens), Hkv, D, generator=g).to(torch.bfloat16).cuda()
    plan = A.dense_plan(q_lens, kv_lens, Hq // Hkv, "cuda", causal=causal)
    _close(A.attention(q, plan, k=k, v=v), A.attention_ref(q, plan, k=k, v=v))


@pytest.mark.parametrize("D", [72, 40, 96])
def test_dense_odd_head_sizes_run_on_the_padded_kernel(D):
    """Encoder head sizes between the kernel's 64 and 128 (SigLIP 72, ViT 80 / 96) and below 64."""
    g = torch.Generator().manual_seed(17)
    Hq = Hkv = 6
    q_lens = [300, 77]
    q = torch.randn(sum(q_lens), Hq, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(sum(q_lens), Hkv, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(sum(q_lens), Hkv, D, generator=g).to(torch.bfloat16).cuda()
    plan = A.dense_plan(q_lens, q_lens, 1, "cuda", causal=False)
    from mstar_b200.ops import _counters
    n0 = _counters.get()
    got = A.attention(q, plan, k=k, v=v)
    assert _counters.get() > n0, "the tensor-core kernel must have been launched"
    assert got.shape == q.shape
    _close(got, A.attention_ref(q, plan, k=k, v=v))


def test_dense_cross_attention_from_fused_buffer():
    """K/V as strided views (cross attention: q_len != kv_len, non-causal)."""
    g = torch.Generator().manual_seed(13)
    Hq, Hkv, D = 8, 8, 64
    q = torch.randn(257, Hq, D, generator=g).to(torch.bfloat16).cuda()
    kv = torch.randn(77, 2, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    k, v = kv[:, 0], kv[:, 1]
    plan = A.dense_plan([257], [77], 1, "cuda", causal=False)
    _close(A.attention(q, plan, k=k, v=v), A.attention_ref(q, plan, k=k, v=v))
