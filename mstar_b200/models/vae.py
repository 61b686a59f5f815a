"""Convolutional latent autoencoders for images (2D) and videos (causal 3D): residual stacks, one mid-block
attention, strided down / nearest-neighbour up sampling. Convolutions run on cuDNN in channels-last layout; the
mid-block attention uses this library's dense attention kernel on the GPU.

Reference counterparts: BAGEL autoencoder (mstar/model/bagel/components/autoencoder.py, 322 lines: AttnBlock :34-60,
ResnetBlock :63-95, Encoder :120-190, Decoder :193-270, 16 latent channels, 8x spatial), Wan VAE through diffusers
(mstar/model/wan22/submodules.py vae nodes; 48 channels, 16x spatial, 4x temporal; tiling switch
mstar/model/wan22/config.py:79-81), Cosmos3 vae nodes (mstar/model/cosmos3/submodules.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import attention as attn_ops


@dataclass
class VAEConfig:
    dims: int = 2                       # 2: images [B,C,H,W]; 3: videos [B,C,T,H,W] with causal time
    in_channels: int = 3
    latent_channels: int = 16
    base_channels: int = 128
    channel_mult: tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    temporal_down: tuple[bool, ...] = field(default_factory=tuple)   # per down stage (dims == 3)
    scaling_factor: float = 1.0
    shift_factor: float = 0.0

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.channel_mult) - 1)

    @property
    def temporal_factor(self) -> int:
        return 2 ** sum(1 for t in self.temporal_down if t)


class _Conv(nn.Module):
    """2D conv, or 3D conv that pads time on the past side only (frame t never sees frame t+1). A strided 2D conv
    pads on the right and bottom only, as the published image autoencoder weights were trained
    (mstar/model/bagel/components/autoencoder.py:83-93)."""

    def __init__(self, dims, cin, cout, k=3, stride=1, t_stride=1):
        super().__init__()
        self.dims, self.k = dims, k
        self.one_sided = dims == 2 and stride > 1
        if dims == 2:
            self.conv = nn.Conv2d(cin, cout, k, stride=stride, padding=0 if self.one_sided else k // 2)
        else:
            self.conv = nn.Conv3d(cin, cout, k, stride=(t_stride, stride, stride), padding=(0, k // 2, k // 2))

    def forward(self, x):
        if self.dims == 3 and self.k > 1:
            x = F.pad(x, (0, 0, 0, 0, self.k - 1, 0), mode="replicate")
        elif self.one_sided:
            x = F.pad(x, (0, self.k // 2, 0, self.k // 2))
        return self.conv(x)


class _ChannelRMS(nn.Module):
    """Per-position RMS norm over channels: keeps a video autoencoder causal in time (group statistics would mix
    frames)."""

    def __init__(self, ch):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(1, ch, 1, 1, 1))
        self.scale = ch ** 0.5

    def forward(self, x):
        return F.normalize(x, dim=1) * self.scale * self.gamma


def _norm(dims, ch):
    return nn.GroupNorm(min(32, ch), ch, eps=1e-6) if dims == 2 else _ChannelRMS(ch)


class _Res(nn.Module):
    def __init__(self, dims, cin, cout):
        super().__init__()
        self.n1, self.c1 = _norm(dims, cin), _Conv(dims, cin, cout)
        self.n2, self.c2 = _norm(dims, cout), _Conv(dims, cout, cout)
        self.skip = _Conv(dims, cin, cout, k=1) if cin != cout else None

    def forward(self, x):
        h = self.c1(F.silu(self.n1(x)))
        h = self.c2(F.silu(self.n2(h)))
        return (x if self.skip is None else self.skip(x)) + h


class _MidAttn(nn.Module):
    """Single-head attention over the spatial positions of every frame."""

    def __init__(self, dims, ch):
        super().__init__()
        self.norm = _norm(dims, ch)
        self.qkv, self.proj = nn.Linear(ch, 3 * ch), nn.Linear(ch, ch)
        self.dims = dims

    def forward(self, x):
        h = self.norm(x)
        if self.dims == 3:
            B, C, T, H, W = h.shape
            seq = h.permute(0, 2, 3, 4, 1).reshape(B * T, H * W, C)
        else:
            B, C, H, W = h.shape
            seq = h.permute(0, 2, 3, 1).reshape(B, H * W, C)
        n, S, C = seq.shape
        qkv = self.qkv(seq)
        q, k, v = qkv.chunk(3, dim=-1)
        if seq.is_cuda and seq.dtype == torch.bfloat16 and C in (64, 128):
            plan = attn_ops.dense_plan([S] * n, [S] * n, 1, seq.device, causal=False)
            o = attn_ops.attention(q.reshape(n * S, 1, C).contiguous(), plan, k=k.reshape(n * S, 1, C).contiguous(),
                                   v=v.reshape(n * S, 1, C).contiguous()).reshape(n, S, C)
        else:
            o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        o = self.proj(o)
        if self.dims == 3:
            o = o.reshape(B, T, H, W, C).permute(0, 4, 1, 2, 3)
        else:
            o = o.reshape(B, H, W, C).permute(0, 3, 1, 2)
        return x + o


class _Up(nn.Module):
    def __init__(self, dims, ch, temporal):
        super().__init__()
        self.dims, self.temporal = dims, temporal
        self.conv = _Conv(dims, ch, ch)

    def forward(self, x):
        if self.dims == 2:
            x = F.interpolate(x, scale_factor=2.0, mode="nearest")
        else:
            x = F.interpolate(x, scale_factor=(2.0 if self.temporal else 1.0, 2.0, 2.0), mode="nearest")
            if self.temporal:
                x = x[:, :, 1:]          # causal: the first latent frame stands for one output frame
        return self.conv(x)


class Encoder(nn.Module):
    def __init__(self, c: VAEConfig):
        super().__init__()
        d = c.dims
        chs = [c.base_channels * m for m in c.channel_mult]
        self.inp = _Conv(d, c.in_channels, chs[0])
        blocks, cin = [], chs[0]
        for i, ch in enumerate(chs):
            for _ in range(c.num_res_blocks):
                blocks.append(_Res(d, cin, ch))
                cin = ch
            if i < len(chs) - 1:
                td = 2 if (d == 3 and i < len(c.temporal_down) and c.temporal_down[i]) else 1
                blocks.append(_Conv(d, cin, cin, stride=2, t_stride=td))
        self.down = nn.Sequential(*blocks)
        self.mid = nn.Sequential(_Res(d, cin, cin), _MidAttn(d, cin), _Res(d, cin, cin))
        self.norm, self.out = _norm(d, cin), _Conv(d, cin, 2 * c.latent_channels)

    def forward(self, x):
        h = self.mid(self.down(self.inp(x)))
        return self.out(F.silu(self.norm(h)))


class Decoder(nn.Module):
    def __init__(self, c: VAEConfig):
        super().__init__()
        d = c.dims
        chs = [c.base_channels * m for m in c.channel_mult]
        cin = chs[-1]
        self.inp = _Conv(d, c.latent_channels, cin)
        self.mid = nn.Sequential(_Res(d, cin, cin), _MidAttn(d, cin), _Res(d, cin, cin))
        blocks = []
        for i in reversed(range(len(chs))):
            for _ in range(c.num_res_blocks + 1):
                blocks.append(_Res(d, cin, chs[i]))
                cin = chs[i]
            if i > 0:
                temporal = d == 3 and (i - 1) < len(c.temporal_down) and c.temporal_down[i - 1]
                blocks.append(_Up(d, cin, temporal))
        self.up = nn.Sequential(*blocks)
        self.norm, self.out = _norm(d, cin), _Conv(d, cin, c.in_channels)

    def forward(self, z):
        h = self.up(self.mid(self.inp(z)))
        return self.out(F.silu(self.norm(h)))


class ConvVAE(nn.Module):
    def __init__(self, cfg: VAEConfig, seed: int | None = 0):
        """``seed``: the random initialisation (before a checkpoint is loaded) is drawn from its own generator state,
        so that every process and every replica of a deployment builds the same weights."""
        super().__init__()
        self.cfg = cfg
        if seed is None:
            self.encoder, self.decoder = Encoder(cfg), Decoder(cfg)
        else:
            with torch.random.fork_rng(devices=[]):
                torch.manual_seed(seed)
                self.encoder, self.decoder = Encoder(cfg), Decoder(cfg)

    @torch.no_grad()
    def encode(self, x: torch.Tensor, sample: bool = False, generator=None) -> torch.Tensor:
        """Pixels in [-1, 1] -> normalised latents (mean of the posterior unless ``sample``)."""
        mean, logvar = self.encoder(x).chunk(2, dim=1)
        z = mean
        if sample:
            z = mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(mean.shape, generator=generator,
                                                                             device=mean.device, dtype=mean.dtype)
        return (z - self.cfg.shift_factor) * self.cfg.scaling_factor

    @torch.no_grad()
    def decode(self, z: torch.Tensor, tile: int = 0) -> torch.Tensor:
        """Latents -> pixels in [-1, 1]. ``tile`` > 0 decodes spatial tiles of that many latent pixels with an
        overlap of a quarter tile and blends them linearly (bounds activation memory on long videos)."""
        z = z / self.cfg.scaling_factor + self.cfg.shift_factor
        if tile <= 0 or (z.shape[-1] <= tile and z.shape[-2] <= tile):
            return self.decoder(z).clamp(-1, 1)
        f = self.cfg.spatial_factor
        ov = max(1, tile // 4)
        step = tile - ov
        H, W = z.shape[-2:]
        out = torch.zeros((*z.shape[:1], self.cfg.in_channels, *([(z.shape[2] - 1) * self.cfg.temporal_factor + 1]
                           if self.cfg.dims == 3 else []), H * f, W * f), dtype=z.dtype, device=z.device)
        wsum = torch.zeros_like(out[:1, :1])
        for y0 in range(0, max(1, H - ov), step):
            for x0 in range(0, max(1, W - ov), step):
                y1, x1 = min(H, y0 + tile), min(W, x0 + tile)
                px = self.decoder(z[..., y0:y1, x0:x1])
                wy = _ramp(y1 - y0, ov, y0 > 0, y1 < H, f, z.device, z.dtype)
                wx = _ramp(x1 - x0, ov, x0 > 0, x1 < W, f, z.device, z.dtype)
                w = wy[:, None] * wx[None, :]
                out[..., y0 * f:y1 * f, x0 * f:x1 * f] += px * w
                wsum[..., y0 * f:y1 * f, x0 * f:x1 * f] += w
        return (out / wsum.clamp_min(1e-6)).clamp(-1, 1)


def _ramp(n, ov, lo, hi, f, device, dtype):
    w = torch.ones(n * f, device=device, dtype=dtype)
    r = torch.linspace(0, 1, ov * f + 2, device=device, dtype=dtype)[1:-1]
    if lo:
        w[:ov * f] = r
    if hi:
        w[-ov * f:] = r.flip(0)
    return w


def bagel_vae_config() -> VAEConfig:
    return VAEConfig(dims=2, latent_channels=16, base_channels=128, channel_mult=(1, 2, 4, 4), num_res_blocks=2,
                     scaling_factor=0.3611, shift_factor=0.1159)


def wan22_vae_config() -> VAEConfig:
    return VAEConfig(dims=3, latent_channels=48, base_channels=160, channel_mult=(1, 2, 4, 4, 4), num_res_blocks=2,
                     temporal_down=(False, True, True, False))


def cosmos3_vae_config() -> VAEConfig:
    return VAEConfig(dims=3, latent_channels=16, base_channels=96, channel_mult=(1, 2, 4, 4), num_res_blocks=2,
                     temporal_down=(False, True, True))


def tiny_vae_config(dims: int = 2, latent_channels: int = 4) -> VAEConfig:
    return VAEConfig(dims=dims, latent_channels=latent_channels, base_channels=8, channel_mult=(1, 2),
                     num_res_blocks=1, temporal_down=(True,) if dims == 3 else ())
