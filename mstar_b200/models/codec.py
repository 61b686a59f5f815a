"""Neural audio codec decoders (SNAC-style multi-scale residual VQ, and a generic code-to-waveform stack).

Convolutions run on cuDNN (the plan keeps codec / VAE convolutions on the library until profiling puts them on the
critical path); the Snake activation and the code lookup are plain tensor ops.

Reference counterparts: SNAC decoder (mstar/model/orpheus/components/snac.py, 424 lines: Snake1d :43, LocalMHA :106,
ResidualUnit :140, NoiseBlock :175, DecoderBlock :189, Decoder :239, VectorQuantize :275), Code2Wav
(mstar/model/qwen3_omni/components/code2wav.py).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn


class Snake1d(nn.Module):
    def __init__(self, channels: int):
        super().__init__()
        self.alpha = nn.Parameter(torch.ones(1, channels, 1))

    def forward(self, x):
        from ..ops.elementwise import snake
        return snake(x, self.alpha)


class ResidualUnit(nn.Module):
    """Snake, dilated kernel-7 convolution (depthwise when ``groups`` = ``dim``), Snake, 1x1 convolution, skip."""

    def __init__(self, dim: int, dilation: int, kernel: int = 7, groups: int = 1):
        super().__init__()
        pad = (kernel - 1) * dilation // 2
        self.block = nn.Sequential(Snake1d(dim), nn.Conv1d(dim, dim, kernel, dilation=dilation, padding=pad, groups=groups),
                                   Snake1d(dim), nn.Conv1d(dim, dim, 1))

    def forward(self, x):
        return x + self.block(x)


class DecoderBlock(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int, noise: bool = False, groups: int = 1):
        super().__init__()
        self.up = nn.Sequential(Snake1d(cin), nn.ConvTranspose1d(cin, cout, 2 * stride, stride=stride,
                                                                 padding=math.ceil(stride / 2), output_padding=stride % 2))
        self.noise = nn.Conv1d(cout, cout, 1, bias=False) if noise else None
        self.res = nn.Sequential(ResidualUnit(cout, 1, groups=groups), ResidualUnit(cout, 3, groups=groups),
                                 ResidualUnit(cout, 9, groups=groups))

    HALO = 3 * (1 + 3 + 9)          # inputs that the three residual units (kernel 7, dilations 1, 3, 9) reach per side

    def forward(self, x, noise_gen: torch.Generator | None = None):
        x = self.up(x)
        if self.noise is not None:
            n = torch.randn((x.shape[0], 1, x.shape[2]), device=x.device, dtype=x.dtype, generator=noise_gen)
            x = x + n * self.noise(x)
        return self.res(x)

    def input_range(self, a: int, b: int, length_in: int) -> tuple[int, int, int, int]:
        """For output positions [a, b): the range [ra, rb) that the residual units must see (their halo, clipped to
        the signal) and the input range [ia, ib) whose transposed-convolution outputs cover it."""
        conv = self.up[1]
        r, p, k = conv.stride[0], conv.padding[0], conv.kernel_size[0]
        ra, rb = max(0, a - self.HALO), min(length_in * r, b + self.HALO)
        ia = max(0, -((-(ra + p - k + 1)) // r))                # ceil((ra + p - k + 1) / r)
        ib = min(length_in, (rb - 1 + p) // r + 1)
        return ra, rb, ia, ib

    def forward_range(self, x, x_off: int, length_in: int, a: int, b: int, noise_gen=None):
        """``x`` holds input positions [x_off, x_off + x.shape[-1]) of a signal of ``length_in`` positions; returns the
        block's output on [ra, rb) ⊇ [a, b) — exact on [a, b), the halo towards a cut edge is not — and ra."""
        ra, rb, ia, ib = self.input_range(a, b, length_in)
        r = self.up[1].stride[0]
        y = self.up(x[..., ia - x_off:ib - x_off])                 # output positions [ia * r, ib * r)
        y = y[..., ra - ia * r:rb - ia * r]
        if self.noise is not None:
            n = torch.randn((y.shape[0], 1, y.shape[2]), device=y.device, dtype=y.dtype, generator=noise_gen)
            y = y + n * self.noise(y)
        return self.res(y), ra


class SnacDecoder(nn.Module):
    """Codes of 3 resolutions (1 / 2 / 4 per 7-token frame) -> 24 kHz waveform; 2048 samples per frame. The defaults
    are the published 24 kHz model: depthwise kernel-7 convolutions (in the input stage and in every residual unit)
    with 1x1 convolutions between them, noise injection after every upsampling, no attention layer."""

    def __init__(self, codebook_size: int = 4096, codebook_dim: int = 8, latent_dim: int = 768, channels: int = 1024,
                 rates=(8, 8, 4, 2), vq_strides=(4, 2, 1), noise: bool = True, depthwise: bool = True):
        super().__init__()
        self.vq_strides = list(vq_strides)
        self.codebook_size = codebook_size
        self.codebooks = nn.ModuleList([nn.Embedding(codebook_size, codebook_dim) for _ in vq_strides])
        self.out_proj = nn.ModuleList([nn.Conv1d(codebook_dim, latent_dim, 1) for _ in vq_strides])
        if depthwise:
            self.inp = nn.Sequential(nn.Conv1d(latent_dim, latent_dim, 7, padding=3, groups=latent_dim),
                                     nn.Conv1d(latent_dim, channels, 1))
        else:
            self.inp = nn.Conv1d(latent_dim, channels, 7, padding=3)
        blocks, c = [], channels
        for r in rates:
            blocks.append(DecoderBlock(c, c // 2, r, noise, groups=c // 2 if depthwise else 1))
            c //= 2
        self.blocks = nn.ModuleList(blocks)
        self.out = nn.Sequential(Snake1d(c), nn.Conv1d(c, 1, 7, padding=3), nn.Tanh())
        self.hop = math.prod(rates)

    def latent(self, codes: list[torch.Tensor]) -> torch.Tensor:
        """codes[l]: [B, T_l] ints with T_l = T_fine / vq_stride[l]."""
        z = 0
        for emb, proj, s, c in zip(self.codebooks, self.out_proj, self.vq_strides, codes):
            e = proj(emb(c.clamp(0, self.codebook_size - 1)).transpose(1, 2))
            z = z + e.repeat_interleave(s, dim=-1)
        return z

    def forward(self, codes: list[torch.Tensor], noise_gen=None, keep: tuple[int, int] | None = None) -> torch.Tensor:
        """Waveform [B, T_fine * hop], or with ``keep`` = (lo, hi) only its samples [lo, hi): every stage then computes
        just the positions that those samples depend on (their receptive field), which for the middle frame of a
        4-frame streaming window is about a quarter of the two finest stages. The kept samples are the same numbers
        as the slice of the full decode (noise aside)."""
        x = self.inp(self.latent(codes))
        if keep is None:
            for b in self.blocks:
                x = b(x, noise_gen)
            return self.out(x)[:, 0]
        lens = [x.shape[-1]]
        for b in self.blocks:
            lens.append(lens[-1] * b.up[1].stride[0])
        lo, hi = max(0, keep[0]), min(lens[-1], keep[1])
        need = [(max(0, lo - 3), min(lens[-1], hi + 3))]           # the output convolution has kernel 7
        for i in reversed(range(len(self.blocks))):
            _, _, ia, ib = self.blocks[i].input_range(*need[0], lens[i])
            need.insert(0, (ia, ib))
        off = 0
        for i, b in enumerate(self.blocks):
            x, off = b.forward_range(x, off, lens[i], *need[i + 1], noise_gen)
        y = self.out(x)[:, 0]
        return y[..., lo - off:hi - off]


def orpheus_tokens_to_codes(tokens: torch.Tensor, base_id: int, codebook_size: int = 4096) -> list[torch.Tensor]:
    """[B, 7 * F] LLM audio tokens -> SNAC code layers ([B,F], [B,2F], [B,4F]). Token at slot s of a frame carries
    code = id - base - 10 - s * codebook_size; slots (0) / (1,4) / (2,3,5,6) feed the coarse / middle / fine layer."""
    B, n = tokens.shape
    Fr = n // 7
    t = tokens[:, :Fr * 7].reshape(B, Fr, 7).long()
    slot = torch.arange(7, device=tokens.device)
    c = (t - base_id - 10 - slot * codebook_size) % codebook_size
    # (slices, not index lists: the function also runs inside CUDA-graph capture, where host index data cannot be copied)
    return [c[:, :, 0], c[:, :, 1:5:3].reshape(B, -1), torch.cat([c[:, :, 2:4], c[:, :, 5:7]], dim=2).reshape(B, -1)]


class Code2Wav(nn.Module):
    """Generic multi-codebook code -> waveform stack (sum of code embeddings, causal conv upsampler)."""

    def __init__(self, n_codebooks: int = 16, codebook_size: int = 2048, dim: int = 512, rates=(8, 5, 4, 3),
                 channels: int = 512):
        super().__init__()
        self.emb = nn.ModuleList([nn.Embedding(codebook_size, dim) for _ in range(n_codebooks)])
        self.inp = nn.Conv1d(dim, channels, 7, padding=3)
        blocks, c = [], channels
        for r in rates:
            blocks.append(DecoderBlock(c, max(32, c // 2), r, False))
            c = max(32, c // 2)
        self.blocks = nn.ModuleList(blocks)
        self.out = nn.Sequential(Snake1d(c), nn.Conv1d(c, 1, 7, padding=3), nn.Tanh())
        self.hop = math.prod(rates)

    def forward(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, n_codebooks, T] -> [B, T * hop]."""
        z = sum(e(codes[:, i].clamp(0, e.num_embeddings - 1)) for i, e in enumerate(self.emb)).transpose(1, 2)
        x = self.inp(z)
        for b in self.blocks:
            x = b(x)
        return self.out(x)[:, 0]
