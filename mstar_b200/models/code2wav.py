"""Qwen3-Omni's codec decoder in the published architecture: 16 code layers per frame -> 24 kHz waveform.

The codes of a frame are embedded (one table over all layers, offset by layer) and averaged; a small causal
transformer with a sliding attention window (rotary positions, RMSNorm, SwiGLU MLP, learned per-channel scales on both
residual branches) mixes the frames; two stages of (causal transposed convolution x2, ConvNeXt block) and a
BigVGAN-style decoder (causal transposed convolutions x8, x5, x4, x3, each followed by three dilated residual units
with the SnakeBeta activation) produce 1920 samples per frame, clamped to [-1, 1]. Every convolution is causal (left
padding only), so a chunk decoded with a few frames of left context continues the previous chunk.

The transformer's projections, norms, rotary embedding and windowed attention run on this library's kernels; the
convolutions run on cuDNN, like those of the other codecs. Reference: mstar/model/qwen3_omni/components/code2wav.py
(535 lines; checkpoint prefix ``code2wav.``). Parity with the Hugging Face module on shared weights is tested on CPU.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops


def _p(shape, dtype=torch.float32, device="cpu"):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


class CausalConv1d(nn.Module):
    """Conv1d padded on the left by (receptive field - stride), and on the right only up to a whole last window."""

    def __init__(self, cin, cout, kernel, dilation=1, stride=1, groups=1):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, kernel, stride=stride, dilation=dilation, groups=groups)
        self.stride, self.field = stride, (kernel - 1) * dilation + 1
        self.pad = self.field - stride

    def forward(self, x):
        n = x.shape[-1]
        frames = math.ceil((n - self.field + self.pad) / self.stride + 1)
        extra = (frames - 1) * self.stride + (self.field - self.pad) - n
        return self.conv(F.pad(x, (self.pad, extra)))


class CausalConvTranspose1d(nn.Module):
    """ConvTranspose1d whose (kernel - stride) overhang is trimmed from both ends."""

    def __init__(self, cin, cout, kernel, stride):
        super().__init__()
        self.conv = nn.ConvTranspose1d(cin, cout, kernel, stride=stride)
        self.trim = kernel - stride

    def forward(self, x):
        y = self.conv(x)
        return y[..., self.trim:y.shape[-1] - self.trim]


class SnakeBeta(nn.Module):
    """x + sin²(x e^alpha) / e^beta, per channel."""

    def __init__(self, channels):
        super().__init__()
        self.alpha, self.beta = nn.Parameter(torch.zeros(channels)), nn.Parameter(torch.zeros(channels))

    def forward(self, x):
        a, b = self.alpha.exp()[None, :, None], self.beta.exp()[None, :, None]
        return x + torch.sin(x * a).pow(2) / (b + 1e-9)


class ConvNeXtBlock(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.dwconv = CausalConv1d(dim, dim, 7, groups=dim)
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.pwconv1, self.pwconv2 = nn.Linear(dim, 4 * dim), nn.Linear(4 * dim, dim)
        self.gamma = nn.Parameter(1e-6 * torch.ones(dim))

    def forward(self, x):
        h = self.norm(self.dwconv(x).transpose(1, 2))
        h = self.pwconv2(F.gelu(self.pwconv1(h))) * self.gamma
        return x + h.transpose(1, 2)


class ResidualUnit(nn.Module):
    def __init__(self, dim, dilation):
        super().__init__()
        self.act1, self.conv1 = SnakeBeta(dim), CausalConv1d(dim, dim, 7, dilation=dilation)
        self.act2, self.conv2 = SnakeBeta(dim), CausalConv1d(dim, dim, 1)

    def forward(self, x):
        return x + self.conv2(self.act2(self.conv1(self.act1(x))))


class UpBlock(nn.Module):
    def __init__(self, cin, cout, rate):
        super().__init__()
        self.act, self.up = SnakeBeta(cin), CausalConvTranspose1d(cin, cout, 2 * rate, rate)
        self.res = nn.ModuleList([ResidualUnit(cout, d) for d in (1, 3, 9)])

    def forward(self, x):
        x = self.up(self.act(x))
        for r in self.res:
            x = r(x)
        return x


class _FrameLayer(nn.Module):
    def __init__(self, H, heads, head_dim, ffn, dtype, device):
        super().__init__()
        A = heads * head_dim
        self.n1, self.n2 = _p((H,), dtype, device), _p((H,), dtype, device)
        self.qkv, self.o = _p((3 * A, H), dtype, device), _p((H, A), dtype, device)
        self.gate_up, self.down = _p((2 * ffn, H), dtype, device), _p((H, ffn), dtype, device)   # gate rows, then up rows
        self.s1, self.s2 = _p((H,), dtype, device), _p((H,), dtype, device)


class FrameTransformer(nn.Module):
    """Causal sliding-window transformer over codec frames (packed sequences [T, H])."""

    def __init__(self, H=1024, layers=8, heads=16, head_dim=64, ffn=3072, window=72, eps=1e-5, theta=10000.0,
                 dtype=torch.float32, device="cpu"):
        super().__init__()
        self.H, self.heads, self.D, self.window, self.eps, self.dtype = H, heads, head_dim, window, eps, dtype
        self.layers = nn.ModuleList([_FrameLayer(H, heads, head_dim, ffn, dtype, device) for _ in range(layers)])
        self.norm = _p((H,), dtype, device)
        self.register_buffer("inv_freq", rope_ops.make_inv_freq(head_dim, theta, device), persistent=False)
        self._plans: dict = {}

    def forward(self, x: torch.Tensor, seq_lens: list[int]) -> torch.Tensor:
        key = (tuple(seq_lens), str(x.device))          # per shape: nothing is built from host data on a repeat
        if key not in self._plans:
            if len(self._plans) > 64:
                self._plans.clear()
            self._plans[key] = (attn_ops.dense_plan(seq_lens, seq_lens, 1, x.device, causal=True, window=self.window),
                                torch.cat([torch.arange(n, dtype=torch.int32, device=x.device) for n in seq_lens]))
        plan, pos = self._plans[key]
        nh, D = self.heads, self.D
        for L in self.layers:
            h = norm_ops.norm(x, L.n1, self.eps)[0]
            q, k, v = rope_ops.rope_kv(gemm.linear(h, L.qkv), pos, self.inv_freq, nh, nh, D, dense_kv=True)
            a = attn_ops.attention(q, plan, k=k, v=v)
            x = x + gemm.linear(a.reshape(-1, nh * D), L.o) * L.s1
            h = norm_ops.norm(x, L.n2, self.eps)[0]
            x = x + gemm.linear(ew.act_mul(gemm.linear(h, L.gate_up), "silu"), L.down) * L.s2
        return norm_ops.norm(x, self.norm, self.eps)[0]


class OmniCode2Wav(nn.Module):
    def __init__(self, n_codebooks=16, codebook_size=2048, hidden=1024, layers=8, heads=16, head_dim=64, ffn=3072,
                 window=72, upsampling_ratios=(2, 2), upsample_rates=(8, 5, 4, 3), decoder_dim=1536,
                 dtype=torch.float32, device="cpu"):
        super().__init__()
        self.K, self.codebook_size = n_codebooks, codebook_size
        self.code_embedding = _p((codebook_size * n_codebooks, hidden), dtype, device)
        self.pre = FrameTransformer(hidden, layers, heads, head_dim, ffn, window, dtype=dtype, device=device)
        self.upsample = nn.ModuleList([nn.ModuleList([CausalConvTranspose1d(hidden, hidden, f, f), ConvNeXtBlock(hidden)])
                                       for f in upsampling_ratios])
        self.inp = CausalConv1d(hidden, decoder_dim, 7)
        self.blocks = nn.ModuleList([UpBlock(decoder_dim // 2 ** i, decoder_dim // 2 ** (i + 1), r)
                                     for i, r in enumerate(upsample_rates)])
        c = decoder_dim // 2 ** len(upsample_rates)
        self.out_act, self.out = SnakeBeta(c), CausalConv1d(c, 1, 7)
        self.hop = math.prod(upsampling_ratios) * math.prod(upsample_rates)
        self.to(device=device, dtype=dtype)
        self.pre.inv_freq = rope_ops.make_inv_freq(head_dim, 10000.0, device)       # stays fp32 whatever the dtype

    def init_random(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        for n, p in self.named_parameters():
            if n.endswith((".n1", ".n2", "pre.norm")) or n.endswith("norm.weight"):
                p.data.fill_(1.0)
            elif n.endswith((".s1", ".s2")):
                p.data.fill_(0.5)
            elif n.endswith(("alpha", "beta")) or p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(max(1, p[0].numel()))).to(p.dtype))
        return self

    @torch.no_grad()
    def forward(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n_codebooks, T] -> waveform [B, T * hop] in [-1, 1]."""
        B, K, T = codes.shape
        if K != self.K:
            raise ValueError(f"expected {self.K} code layers, got {K}")
        off = torch.arange(K, device=codes.device)[None, :, None] * self.codebook_size
        h = self.code_embedding[(codes.clamp(0, self.codebook_size - 1) + off).reshape(-1)].reshape(B, K, T, -1).float().mean(1)
        h = self.pre(h.reshape(B * T, -1).to(self.pre.dtype).contiguous(), [T] * B).reshape(B, T, -1)
        x = h.transpose(1, 2).to(self.inp.conv.weight.dtype)
        for up, block in self.upsample:
            x = block(up(x))
        x = self.inp(x)
        for b in self.blocks:
            x = b(x)
        return self.out(self.out_act(x))[:, 0].float().clamp(-1, 1)
