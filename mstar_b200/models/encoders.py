"""Bidirectional transformer encoders shared by the model families: text (T5-style with relative position bias),
vision (ViT over image / video patches, learned or rotary positions, optional patch merger), audio (log-mel ->
strided conv stem -> transformer).

Projections, norms, MLP activations and attention run on this library's kernels when the tensors are bf16 on the
GPU and the head size is one the attention kernel has (64 or 128); other shapes (SigLIP's 72-wide heads, the
additive position bias of T5) use torch's scaled_dot_product_attention. Encoders run once per request, off the
decode loop.

Reference counterparts: BAGEL SigLIP NaViT encoder (mstar/model/bagel/components/vit_encoder.py, 405 lines),
Qwen3-Omni audio / vision encoders (HF modules wrapped in mstar/model/qwen3_omni/submodules.py), Whisper encoder
(mstar/model/whisper/submodules.py), UMT5 text encoder of Wan2.2 (mstar/model/wan22/submodules.py text_encoder),
V-JEPA2 encoder layers (mstar/model/vjepa2/components/layers.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import attention as attn_ops
from ..ops import gemm
from ..ops import norm as norm_ops


@dataclass
class EncoderConfig:
    hidden_size: int = 1024
    num_layers: int = 24
    num_heads: int = 16
    head_dim: int = 64
    ffn_dim: int = 4096
    norm: str = "layernorm"            # layernorm | rmsnorm
    act: str = "gelu"                  # gelu (tanh form, fused) | gelu_erf (exact) | gated_gelu | silu_gated
    qkv_bias: bool = True
    eps: float = 1e-6
    dtype: torch.dtype = torch.bfloat16


def _p(shape, dtype, device):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


class EncoderLayer(nn.Module):
    def __init__(self, c: EncoderConfig, device):
        super().__init__()
        self.c = c
        H, A, dt = c.hidden_size, c.num_heads * c.head_dim, c.dtype
        ln = c.norm == "layernorm"
        self.n1_w, self.n1_b = _p((H,), dt, device), (_p((H,), dt, device) if ln else None)
        self.qkv_w, self.qkv_b = _p((3 * A, H), dt, device), (_p((3 * A,), dt, device) if c.qkv_bias else None)
        self.o_w, self.o_b = _p((H, A), dt, device), (_p((H,), dt, device) if c.qkv_bias else None)
        self.n2_w, self.n2_b = _p((H,), dt, device), (_p((H,), dt, device) if ln else None)
        gated = c.act in ("gated_gelu", "silu_gated")
        self.fc1_w = _p(((2 if gated else 1) * c.ffn_dim, H), dt, device)      # gated: rows interleave (gate, up)
        self.fc1_b = _p((c.ffn_dim,), dt, device) if (ln and not gated) else None
        self.fc2_w, self.fc2_b = _p((H, c.ffn_dim), dt, device), (_p((H,), dt, device) if ln and not gated else None)

    def _norm(self, x, w, b):
        return norm_ops.norm(x, w, self.c.eps, bias=b, layernorm=self.c.norm == "layernorm")[0]

    def forward(self, x, plan, bias=None, seq_lens=None, rope=None):
        """x: [T, H] packed sequences; plan: dense bidirectional plan; bias: optional [heads, S, S] additive
        attention bias (forces the SDPA path; all sequences then have the same length S)."""
        c = self.c
        nh, D = c.num_heads, c.head_dim
        h = self._norm(x, self.n1_w, self.n1_b)
        qkv = gemm.linear(h, self.qkv_w, bias=self.qkv_b)
        A = nh * D
        q, k, v = (qkv[:, i * A:(i + 1) * A].reshape(-1, nh, D) for i in range(3))
        if rope is not None:
            q, k = rope(q), rope(k)
        if bias is None and x.is_cuda and x.dtype == torch.bfloat16 and D in (64, 128):
            a = attn_ops.attention(q.contiguous(), plan, k=k.contiguous(), v=v.contiguous())
        else:
            a = _sdpa_packed(q, k, v, seq_lens, bias, 1.0 if bias is not None and c.norm == "rmsnorm" else None)
        x = gemm.linear(a.reshape(-1, A), self.o_w, bias=self.o_b, residual=x)
        h = self._norm(x, self.n2_w, self.n2_b)
        if c.act == "gelu":
            h = gemm.linear(h, self.fc1_w, bias=self.fc1_b, epilogue=gemm.EPILOGUE_GELU)
        elif c.act == "gelu_erf":
            h = F.gelu(gemm.linear(h, self.fc1_w, bias=self.fc1_b).float()).to(x.dtype)
        elif c.act == "silu_gated":
            h = gemm.linear(h, self.fc1_w, epilogue=gemm.EPILOGUE_SWIGLU)
        else:   # gated gelu (T5 v1.1): gelu(gate) * up, rows interleaved
            g = gemm.linear(h, self.fc1_w)
            h = (F.gelu(g[:, 0::2].float(), approximate="tanh") * g[:, 1::2].float()).to(x.dtype)
        return gemm.linear(h, self.fc2_w, bias=self.fc2_b, residual=x)


def _sdpa_packed(q, k, v, seq_lens, bias, scale):
    outs, o = [], 0
    for n in seq_lens:
        qi, ki, vi = (t[o:o + n].transpose(0, 1)[None] for t in (q, k, v))
        m = None if bias is None else bias[None, :, :n, :n].to(qi.dtype)
        outs.append(F.scaled_dot_product_attention(qi, ki, vi, attn_mask=m, scale=scale)[0].transpose(0, 1))
        o += n
    return torch.cat(outs).contiguous()


class TransformerEncoder(nn.Module):
    def __init__(self, c: EncoderConfig, device="cpu", final_norm: bool = True):
        super().__init__()
        self.c, self.device = c, torch.device(device)
        self.layers = nn.ModuleList([EncoderLayer(c, device) for _ in range(c.num_layers)])
        self.fn_w = _p((c.hidden_size,), c.dtype, device) if final_norm else None
        self.fn_b = _p((c.hidden_size,), c.dtype, device) if final_norm and c.norm == "layernorm" else None
        self._plans: dict = {}

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for n, p in self.named_parameters():
            if p.dim() == 1:
                p.data.fill_(1.0) if n.endswith("_w") else p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(p.shape[-1])).to(p.dtype))
        return self

    def final_norm(self, x: torch.Tensor) -> torch.Tensor:
        if self.fn_w is None:
            return x
        return norm_ops.norm(x, self.fn_w, self.c.eps, bias=self.fn_b, layernorm=self.c.norm == "layernorm")[0]

    def forward(self, x: torch.Tensor, seq_lens: list[int], bias=None, rope=None, collect: list[int] | None = None,
                final: bool = True):
        # plans are cached per shape: a captured piece must not create tensors from host data
        key = (tuple(seq_lens), str(x.device))
        plan = self._plans.get(key)
        if plan is None:
            if len(self._plans) > 256:
                self._plans.clear()
            plan = self._plans[key] = attn_ops.dense_plan(seq_lens, seq_lens, 1, x.device, causal=False)
        taps = []
        for i, L in enumerate(self.layers):
            x = L(x, plan, bias, seq_lens, rope)
            if collect and i in collect:
                taps.append(x)
        if final:
            x = self.final_norm(x)
        return (x, taps) if collect else x


# ------------------------------------------------------------------ text
class T5Encoder(nn.Module):
    """Encoder-only T5 v1.1 / UMT5: RMSNorm, unscaled attention with a learned bucketed relative position bias
    (per layer for UMT5), gated-GELU MLP."""

    def __init__(self, vocab_size=256384, hidden=4096, layers=24, heads=64, head_dim=64, ffn=10240, buckets=32,
                 max_distance=128, per_layer_bias=True, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        c = EncoderConfig(hidden, layers, heads, head_dim, ffn, norm="rmsnorm", act="gated_gelu", qkv_bias=False,
                          dtype=dtype)
        self.c, self.buckets, self.max_distance = c, buckets, max_distance
        self.embed = _p((vocab_size, hidden), dtype, device)
        self.rel_bias = _p((layers if per_layer_bias else 1, buckets, heads), dtype, device)
        self.enc = TransformerEncoder(c, device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.embed.data.copy_((torch.randn(self.embed.shape, generator=g) * 0.5).to(self.embed.dtype))
        self.rel_bias.data.copy_((torch.randn(self.rel_bias.shape, generator=g) * 0.1).to(self.rel_bias.dtype))
        self.enc.init_random(seed + 1)
        return self

    def _bucket(self, S, device):
        ctx = torch.arange(S, device=device)
        rel = ctx[None, :] - ctx[:, None]
        nb = self.buckets // 2
        out = (rel > 0).long() * nb
        n = rel.abs()
        exact = nb // 2
        large = exact + (torch.log(n.float().clamp_min(1) / exact) / math.log(self.max_distance / exact)
                         * (nb - exact)).long()
        return out + torch.where(n < exact, n, large.clamp_max(nb - 1))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids: [S] -> [S, hidden]."""
        S = ids.numel()
        x = self.embed[ids.reshape(-1)]
        bucket = self._bucket(S, x.device)
        plan = attn_ops.dense_plan([S], [S], 1, x.device, causal=False)
        for i, L in enumerate(self.enc.layers):
            tbl = self.rel_bias[i if self.rel_bias.shape[0] > 1 else 0]
            x = L(x, plan, tbl[bucket].permute(2, 0, 1).float(), [S])
        return norm_ops.norm(x, self.enc.fn_w, self.c.eps)[0]


# ------------------------------------------------------------------ vision
class VisionEncoder(nn.Module):
    """ViT over packed patch sequences of any resolution. ``pos`` = "learned" interpolates a learned 2D table
    to each image's grid (NaViT style); "rope2d" rotates q/k halves by the patch's (row, col)."""

    def __init__(self, c: EncoderConfig, patch: int = 14, in_channels: int = 3, temporal_patch: int = 1,
                 pos: str = "learned", pos_grid: int = 70, out_dim: int | None = None, merge: int = 1, device="cpu",
                 projector: str = "mlp"):
        """``projector``: "mlp" (linear, GELU, linear — BAGEL's connector, the Qwen mergers) or "linear" (one layer,
        PaliGemma's multi-modal projector); used when ``out_dim`` is given."""
        super().__init__()
        self.c, self.patch, self.tp, self.pos, self.merge = c, patch, temporal_patch, pos, merge
        pdim = in_channels * temporal_patch * patch * patch
        self.patch_w, self.patch_b = _p((c.hidden_size, pdim), c.dtype, device), _p((c.hidden_size,), c.dtype, device)
        self.pos_table = _p((pos_grid * pos_grid, c.hidden_size), c.dtype, device) if pos == "learned" else None
        self.pos_grid = pos_grid
        self.enc = TransformerEncoder(c, device)
        md = c.hidden_size * merge * merge
        self.out_dim, self.projector = out_dim, projector
        if out_dim:
            if projector == "mlp":
                self.proj1_w, self.proj1_b = _p((md, md), c.dtype, device), _p((md,), c.dtype, device)
            self.proj2_w, self.proj2_b = _p((out_dim, md), c.dtype, device), _p((out_dim,), c.dtype, device)

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for n, p in self.named_parameters():
            if n.startswith("enc."):
                continue
            p.data.copy_((torch.randn(p.shape, generator=g) * (0.02 if p.dim() == 1 else 1 / math.sqrt(p.shape[-1]))).to(p.dtype))
        self.enc.init_random(seed + 1)
        return self

    def patches(self, img: torch.Tensor):
        """[C, H, W] or [C, T, H, W] -> ([n, C*tp*p*p], (t, h, w))."""
        if img.dim() == 3:
            img = img[:, None].expand(-1, self.tp, -1, -1)
        C, T, H, W = img.shape
        p, tp = self.patch, self.tp
        t, h, w = T // tp, H // p, W // p
        x = img[:, :t * tp, :h * p, :w * p].reshape(C, t, tp, h, p, w, p).permute(1, 3, 5, 0, 2, 4, 6)
        return x.reshape(t * h * w, C * tp * p * p), (t, h, w)

    def _pos_embed(self, grid, device):
        t, h, w = grid
        G = self.pos_grid
        tbl = self.pos_table.float().reshape(1, G, G, -1).permute(0, 3, 1, 2)
        e = F.interpolate(tbl, size=(h, w), mode="bilinear", align_corners=False)[0].permute(1, 2, 0).reshape(h * w, -1)
        return e.repeat(t, 1).to(self.c.dtype)

    def _rope(self, grids, device):
        D = self.c.head_dim
        quarter = D // 4
        inv = 1.0 / (10000.0 ** (torch.arange(quarter, dtype=torch.float32, device=device) / quarter))
        rows, cols = [], []
        for t, h, w in grids:
            r = torch.arange(h, device=device).repeat_interleave(w).repeat(t)
            cc = torch.arange(w, device=device).repeat(h * t)
            rows.append(r)
            cols.append(cc)
        ang = torch.cat([torch.cat(rows)[:, None] * inv, torch.cat(cols)[:, None] * inv], dim=-1)   # [T, D/2]
        cs, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]

        def apply(x):
            xf = x.float()
            a, b = xf[..., :D // 2], xf[..., D // 2:]
            return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1).to(x.dtype)
        return apply

    def forward(self, images: list[torch.Tensor], collect: list[int] | None = None):
        """Returns (features [sum tokens_out, out_dim or hidden], tokens per image, grids)."""
        toks, grids = [], []
        for im in images:
            p, g = self.patches(im.to(self.c.dtype))
            toks.append(p)
            grids.append(g)
        x = gemm.linear(torch.cat(toks), self.patch_w, bias=self.patch_b)
        if self.pos == "learned":
            x = x + torch.cat([self._pos_embed(g, x.device) for g in grids])
        rope = self._rope(grids, x.device) if self.pos == "rope2d" else None
        lens = [g[0] * g[1] * g[2] for g in grids]
        out = self.enc(x, lens, rope=rope, collect=collect)
        x, taps = out if collect else (out, [])
        m = self.merge * self.merge
        if m > 1:
            x = self._merge(x, grids)
            taps = [self._merge(t, grids) for t in taps]
            lens = [n // m for n in lens]
        if self.out_dim:
            if self.projector == "mlp":
                x = gemm.linear(x, self.proj1_w, bias=self.proj1_b, epilogue=gemm.EPILOGUE_GELU)
            x = gemm.linear(x, self.proj2_w, bias=self.proj2_b)
        return (x, lens, grids, taps) if collect else (x, lens, grids)

    def _merge(self, x, grids):
        m, outs, o = self.merge, [], 0
        for t, h, w in grids:
            n = t * h * w
            g = x[o:o + n].reshape(t, h // m, m, w // m, m, -1).permute(0, 1, 3, 2, 4, 5)
            outs.append(g.reshape(t * (h // m) * (w // m), -1))
            o += n
        return torch.cat(outs)


# ------------------------------------------------------------------ audio
def log_mel_spectrogram(wav: torch.Tensor, sample_rate: int = 16000, n_fft: int = 400, hop: int = 160,
                        n_mels: int = 128) -> torch.Tensor:
    """Whisper-style log-mel features [n_mels, frames] of a mono waveform in [-1, 1]."""
    wav = wav.float().reshape(-1)
    win = torch.hann_window(n_fft, device=wav.device)
    spec = torch.stft(wav, n_fft, hop, window=win, return_complex=True)[..., :-1].abs() ** 2
    fb = _mel_filterbank(sample_rate, n_fft, n_mels, wav.device)
    mel = (fb @ spec).clamp_min(1e-10).log10()
    mel = torch.maximum(mel, mel.max() - 8.0)
    return (mel + 4.0) / 4.0


_MEL_BANKS: dict = {}


def _mel_filterbank(sr, n_fft, n_mels, device):
    key = (sr, n_fft, n_mels, str(device))
    if key not in _MEL_BANKS:
        _MEL_BANKS[key] = _build_mel_filterbank(sr, n_fft, n_mels).to(device)
    return _MEL_BANKS[key]


def _build_mel_filterbank(sr, n_fft, n_mels):
    """Triangular filters on the Slaney mel scale (linear below 1 kHz, logarithmic above), each scaled by 2 / width:
    the bank Whisper's feature extractor uses."""
    step, knee, logstep = 200.0 / 3.0, 1000.0, math.log(6.4) / 27.0

    def hz2mel(f):
        return f / step if f < knee else knee / step + math.log(f / knee) / logstep

    mels = torch.linspace(hz2mel(0.0), hz2mel(sr / 2), n_mels + 2, dtype=torch.float64)
    hz = torch.where(mels < knee / step, mels * step, knee * torch.exp(logstep * (mels - knee / step)))
    bins = torch.linspace(0, sr / 2, n_fft // 2 + 1, dtype=torch.float64)
    fb = torch.zeros(n_mels, n_fft // 2 + 1, dtype=torch.float64)
    for i in range(n_mels):
        lo, ce, hi = hz[i], hz[i + 1], hz[i + 2]
        fb[i] = torch.clamp(torch.minimum((bins - lo) / (ce - lo), (hi - bins) / (hi - ce)), min=0) * (2.0 / (hi - lo))
    return fb.float()


class AudioEncoder(nn.Module):
    """Whisper-class encoder: two conv1d (second with stride 2) + sinusoidal positions + pre-LN transformer;
    optional projection to the language model's width. ``pool`` > 1 averages that many consecutive frames of each
    sequence between the last layer and the final norm (a trailing remainder is dropped)."""

    def __init__(self, c: EncoderConfig, n_mels: int = 128, max_frames: int = 1500, out_dim: int | None = None,
                 device="cpu", pool: int = 1):
        super().__init__()
        self.c, self.pool = c, pool
        self.conv1 = nn.Conv1d(n_mels, c.hidden_size, 3, padding=1).to(device=device, dtype=c.dtype)
        self.conv2 = nn.Conv1d(c.hidden_size, c.hidden_size, 3, stride=2, padding=1).to(device=device, dtype=c.dtype)
        half = c.hidden_size // 2
        inc = math.log(10000.0) / (half - 1)
        t = torch.arange(max_frames)[:, None] * torch.exp(-inc * torch.arange(half))[None]
        self.register_buffer("pos", torch.cat([t.sin(), t.cos()], dim=1).to(c.dtype).to(device), persistent=False)
        self.enc = TransformerEncoder(c, device)
        self.out_w = _p((out_dim, c.hidden_size), c.dtype, device) if out_dim else None

    def init_random(self, seed=0):
        self.enc.init_random(seed)
        if self.out_w is not None:
            g = torch.Generator().manual_seed(seed + 7)
            self.out_w.data.copy_((torch.randn(self.out_w.shape, generator=g) / math.sqrt(self.out_w.shape[-1])).to(self.out_w.dtype))
        return self

    def forward(self, mels: list[torch.Tensor]):
        """mels: list of [n_mels, frames] -> (features [sum frames/2, dim], lengths)."""
        xs, lens = [], []
        for m in mels:
            h = F.gelu(self.conv1(m[None].to(self.c.dtype)))
            h = F.gelu(self.conv2(h))[0].transpose(0, 1)
            n = min(h.shape[0], self.pos.shape[0])
            xs.append(h[:n] + self.pos[:n])
            lens.append(n)
        if self.pool > 1:
            x = self.enc(torch.cat(xs).contiguous(), lens, final=False)
            k, parts = self.pool, []
            for h in x.split(lens):
                parts.append(h[:h.shape[0] // k * k].reshape(h.shape[0] // k, k, -1).float().mean(1).to(h.dtype))
            lens = [n // k for n in lens]
            x = self.enc.final_norm(torch.cat(parts).contiguous())
        else:
            x = self.enc(torch.cat(xs).contiguous(), lens)
        if self.out_w is not None:
            x = gemm.linear(x, self.out_w)
        return x, lens
