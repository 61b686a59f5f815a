"""Elementwise / norm / rope / sampling kernels against their fp32 oracles."""
import pytest
import torch

from mstar_b200.ops import elementwise as E
from mstar_b200.ops import norm as N
from mstar_b200.ops import rope as R
from mstar_b200.ops import sampling as S

pytestmark = pytest.mark.gpu


def _r(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol, f"max err {err}"


@pytest.mark.parametrize("rows,hidden", [(1, 256), (64, 3072), (37, 2048), (5, 8192), (3, 3584)])
def test_rmsnorm_residual(rows, hidden):
    x, w, r = _r((rows, hidden), 1), _r((hidden,), 2, 0.3) + 1, _r((rows, hidden), 3)
    y, _ = N.norm(x, w, 1e-6)
    _close(y, N.norm_ref(x, w, 1e-6)[0], 3e-2)
    r2 = r.clone()
    y, nr = N.norm(x, w, 1e-5, residual=r2)
    yr, nrr = N.norm_ref(x, w, 1e-5, residual=r)
    _close(y, yr, 3e-2)
    assert torch.equal(nr, nrr)


def test_layernorm_modulated():
    rows, hidden, nmod = 48, 2048, 2
    x, sc, sh = _r((rows, hidden), 4), _r((nmod, hidden), 5, 0.2), _r((nmod, hidden), 6, 0.2)
    y, _ = N.norm(x, None, 1e-6, scale=sc, shift=sh, layernorm=True)
    _close(y, N.norm_ref(x, None, 1e-6, scale=sc, shift=sh, layernorm=True)[0], 4e-2)
    w = _r((hidden,), 7, 0.1)
    y, _ = N.norm(x, w, 1e-6, gemma=True)
    _close(y, N.norm_ref(x, w, 1e-6, gemma=True)[0], 4e-2)


@pytest.mark.parametrize("Hq,Hkv,D,qknorm,inter", [(4, 2, 64, False, False), (24, 8, 128, False, False),
                                                     (32, 4, 128, True, False), (8, 8, 128, True, True)])
def test_rope_kv_write(Hq, Hkv, D, qknorm, inter):
    T, ps = 19, 16
    qkv = _r((T, (Hq + 2 * Hkv) * D), 8)
    pos = torch.arange(100, 100 + T, dtype=torch.int32).cuda()
    inv = R.make_inv_freq(D, 1e6, "cuda")
    qw = _r((D,), 9, 0.2) + 1 if qknorm else None
    kw = _r((D,), 10, 0.2) + 1 if qknorm else None
    cache = torch.zeros(8, 2, Hkv, ps, D, dtype=torch.bfloat16).cuda()
    cache_ref = cache.clone()
    token_req = torch.tensor([0] * 10 + [1] * 9, dtype=torch.int32).cuda()
    cache_pos = torch.tensor(list(range(20, 30)) + list(range(0, 9)), dtype=torch.int32).cuda()
    page_indptr = torch.tensor([0, 2, 3], dtype=torch.int32).cuda()
    page_indices = torch.tensor([5, 2, 7], dtype=torch.int32).cuda()
    q, k, v = R.rope_kv(qkv, pos, inv, Hq, Hkv, D, q_norm_w=qw, k_norm_w=kw, interleaved=inter, cache=cache,
                        token_req=token_req, cache_pos=cache_pos, page_indptr=page_indptr,
                        page_indices=page_indices, dense_kv=True)
    qr, kr, vr = R.rope_kv_ref(qkv, pos, inv, Hq, Hkv, D, q_norm_w=qw, k_norm_w=kw, interleaved=inter)
    _close(q, qr, 4e-2)
    _close(k, kr, 4e-2)
    assert torch.equal(v, vr)
    R.write_kv_ref(cache_ref, k, v, token_req, cache_pos, page_indptr, page_indices)
    assert torch.equal(cache, cache_ref)


def test_mrope_axes_and_llama3():
    T, Hq, Hkv, D = 7, 4, 2, 128
    qkv = _r((T, (Hq + 2 * Hkv) * D), 11)
    pos = torch.randint(0, 5000, (3, T), dtype=torch.int32).cuda()
    inv = R.make_inv_freq(D, 5e5, "cuda", llama3={"factor": 32.0})
    ax = R.mrope_axis_table([24, 20, 20]).cuda()
    q, _, _ = R.rope_kv(qkv, pos, inv, Hq, Hkv, D, axis_of_freq=ax)
    qr, _, _ = R.rope_kv_ref(qkv, pos, inv, Hq, Hkv, D, axis_of_freq=ax)
    _close(q, qr, 4e-2)


def test_small_elementwise():
    x = _r((33, 2 * 688), 12)
    _close(E.act_mul(x), E.act_mul_ref(x), 2e-2)
    table = _r((1000, 256), 13)
    ids = torch.tensor([[0, 999, 500], [1200, 3, 7]], dtype=torch.int64).cuda()
    assert torch.equal(E.embed(ids, table), E.embed_ref(ids, table))
    assert torch.equal(E.embed(ids, table, vocab_start=400), E.embed_ref(ids, table, vocab_start=400))
    a, b, g = _r((24, 512), 14), _r((24, 512), 15), _r((2, 512), 16)
    _close(E.gated_residual(a, b, g), E.gated_residual_ref(a, b, g), 2e-2)
    vc, vu, xx = _r((40, 64), 17, 1, torch.float32), _r((40, 64), 18, 1, torch.float32), _r((40, 64), 19, 1, torch.float32)
    xn, v = E.cfg_combine(vc, vu, xx, -0.02, 4.0, renorm=True)
    xr, vr = E.cfg_combine_ref(vc, vu, xx, -0.02, 4.0, renorm=True)
    _close(xn, xr, 1e-4)
    _close(v, vr, 1e-3)
    kv = torch.tensor([5, 9], dtype=torch.int32).cuda()
    pos = torch.tensor([4, 8], dtype=torch.int32).cuda()
    ids2 = torch.zeros(2, dtype=torch.int64).cuda()
    E.advance_decode(kv, pos, None, ids2, torch.tensor([11, 12]).cuda())
    assert kv.tolist() == [6, 10] and pos.tolist() == [5, 9] and ids2.tolist() == [11, 12]


def test_sampling_greedy_and_nucleus():
    B, V = 16, 32000
    logits = _r((B, V), 20, 3.0, torch.float32)
    st = S.SamplerState(B, V, "cuda", track_seen=True)
    for b in range(B):
        st.assign(f"r{b}", S.SamplingConfig(V, temperature=0.0 if b < 4 else 0.8, top_k=0 if b % 2 else 50,
                                            top_p=0.9 if b < 12 else 1.0, repetition_penalty=1.0 if b % 3 else 1.3))
    rs = torch.arange(B, dtype=torch.int32).cuda()
    u = torch.rand(B, generator=torch.Generator().manual_seed(1)).cuda()
    seen0 = st.seen.clone()
    tok = st.sample(logits, rs, u=u)
    assert torch.equal(tok[:4], logits[:4].argmax(-1))
    assert st.offset.tolist() == [1] * B
    exact = 0
    for b in range(4, B):
        p, keep = S.kept_set_ref(logits[b], st.temperature[b].item(), st.top_k[b].item(), st.top_p[b].item(),
                                 seen0[b], st.rep_penalty[b].item())
        t = tok[b].item()
        # the kernel's kept set is the exact nucleus plus ties within the 24-bit threshold quantum
        assert p[t] >= p[keep].min() * (1 - 1e-3), f"row {b}: token outside the nucleus"
        assert st.seen[b, t] == 1
        ref = S.sample_ref(logits[b:b + 1], [st.temperature[b].item()], [st.top_k[b].item()], [st.top_p[b].item()],
                           [st.rep_penalty[b].item()], [0], [0], seen0[b:b + 1].clone(), [u[b].item()])
        exact += int(ref[0].item() == t)
    assert exact >= 10, f"only {exact}/12 rows match the oracle draw"


def test_sampling_distribution_and_bf16():
    V, B = 1000, 4096
    row = torch.zeros(V)
    row[:4] = torch.tensor([2.0, 1.0, 0.0, -1.0])
    row[4:] = -20.0
    logits = row.to(torch.bfloat16).cuda().repeat(B, 1)
    st = S.SamplerState(B, V, "cuda")
    for b in range(B):
        st.assign(f"q{b}", S.SamplingConfig(V, temperature=1.0), seed=b + 1)
    tok = st.sample(logits, torch.arange(B, dtype=torch.int32).cuda())
    freq = torch.bincount(tok.cpu(), minlength=V)[:4].float() / B
    expect = torch.softmax(row[:4], 0)
    assert (freq - expect).abs().max() < 0.03
    # same seeds and offsets -> same draws; CPU path of the same state agrees with the GPU path
    st.offset.zero_()
    tok2 = st.sample(logits, torch.arange(B, dtype=torch.int32).cuda())
    assert torch.equal(tok, tok2)


def test_snake_activation_matches_reference():
    from mstar_b200.ops import elementwise as E
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 20, 257, generator=g)
    a = torch.rand(1, 20, 1, generator=g) + 0.5
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        ref = E.snake_ref(x.to(dt), a)
        out = E.snake(x.to(dt).cuda(), a.cuda())
        assert (out.float().cpu() - ref.float()).abs().max().item() < tol
