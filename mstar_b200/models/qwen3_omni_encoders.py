"""The audio and vision towers of Qwen3-Omni in the published architecture, on this library's encoder layers.

``OmniAudioEncoder``: log-mel frames are cut into chunks of ``2 * n_window`` frames; every chunk goes through three
stride-2 3x3 convolutions (8x fewer frames and mel bins), a linear layer over (channels x bins) and sinusoidal
positions that restart in every chunk; the valid rows of all chunks then run through a pre-LN transformer whose
attention is confined to windows of ``n_window_infer`` input frames, a final LayerNorm and a two-layer projection.

``OmniVisionEncoder``: patches of ``temporal_patch x patch x patch`` pixels, a learned position table interpolated
bilinearly (corner-aligned) to the image's grid, a 2D rotary embedding, attention inside each frame, a patch merger
(LayerNorm, then ``merge x merge`` neighbours concatenated, two linear layers) and "deepstack" mergers that tap
intermediate layers (LayerNorm after the concatenation); the decoder adds the tapped features to its first layers'
outputs at the image rows.

The reference wraps the Hugging Face modules (mstar/model/qwen3_omni/qwen3_omni_model.py:1507-1580, prefixes
``thinker.audio_tower`` / ``thinker.visual``; submodules.py:49-200); here they are restated on ``TransformerEncoder`` so
that projections, norms and attention run on this library's kernels. Parity with the Hugging Face modules on shared
weights is tested on CPU.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import gemm
from ..ops import norm as norm_ops
from .encoders import EncoderConfig, TransformerEncoder, _p


def audio_output_length(frames: int, chunk: int = 100) -> int:
    """Rows the audio tower gives for ``frames`` mel frames: 13 per full chunk of 100, and the three stride-2
    convolutions' count for the tail."""
    tail = frames % chunk
    t = (tail - 1) // 2 + 1
    return ((t - 1) // 2 + 1 - 1) // 2 + 1 + (frames // chunk) * 13 if tail else (frames // chunk) * 13


def _conv_len(n: int) -> int:
    for _ in range(3):
        n = (n - 1) // 2 + 1
    return n


def _randomize(module: nn.Module, seed: int) -> None:
    g = torch.Generator().manual_seed(seed)
    for n, p in module.named_parameters():
        if n.startswith("enc."):
            continue
        if p.dim() == 1:
            p.data.copy_((torch.ones(p.shape) if n.endswith(("n_w", "norm_w")) else torch.zeros(p.shape)).to(p.dtype))
        else:
            fan_in = p[0].numel()
            p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(fan_in)).to(p.dtype))


class OmniAudioEncoder(nn.Module):
    def __init__(self, c: EncoderConfig, n_mels: int = 128, conv_channels: int = 480, out_dim: int = 2048,
                 n_window: int = 50, n_window_infer: int = 400, max_positions: int = 1500, device="cpu"):
        super().__init__()
        if c.act != "gelu_erf" or c.norm != "layernorm":
            raise ValueError("the audio tower uses LayerNorm and the exact GELU")
        self.c, self.n_mels, self.chunk, self.n_window_infer = c, n_mels, 2 * n_window, n_window_infer
        dt = c.dtype
        self.conv2d1 = nn.Conv2d(1, conv_channels, 3, 2, padding=1).to(device=device, dtype=dt)
        self.conv2d2 = nn.Conv2d(conv_channels, conv_channels, 3, 2, padding=1).to(device=device, dtype=dt)
        self.conv2d3 = nn.Conv2d(conv_channels, conv_channels, 3, 2, padding=1).to(device=device, dtype=dt)
        self.conv_out_w = _p((c.hidden_size, conv_channels * _conv_len(n_mels)), dt, device)
        half = c.hidden_size // 2
        t = torch.arange(max_positions)[:, None] * torch.exp(-math.log(10000.0) / (half - 1) * torch.arange(half).float())[None]
        self.register_buffer("pos", torch.cat([t.sin(), t.cos()], dim=1).to(dt).to(device), persistent=False)
        self.enc = TransformerEncoder(c, device)                       # its final norm is the tower's ``ln_post``
        self.proj1_w, self.proj1_b = _p((c.hidden_size, c.hidden_size), dt, device), _p((c.hidden_size,), dt, device)
        self.proj2_w, self.proj2_b = _p((out_dim, c.hidden_size), dt, device), _p((out_dim,), dt, device)

    def init_random(self, seed=0):
        self.enc.init_random(seed)
        _randomize(self, seed + 7)
        return self

    def forward(self, mels: list[torch.Tensor]):
        """mels: list of [n_mels, frames] -> (features [sum rows, out_dim], rows per input)."""
        dt, W = self.c.dtype, self.chunk
        chunks, chunk_lens, per_audio = [], [], []
        for m in mels:
            parts = list(m.to(dt).split(W, dim=1))
            chunks += parts
            chunk_lens += [p.shape[1] for p in parts]
            per_audio.append(sum(_conv_len(p.shape[1]) for p in parts))
        longest = max(chunk_lens)
        x = torch.stack([F.pad(p, (0, longest - p.shape[1])) for p in chunks])[:, None]         # [n, 1, mels, frames]
        for conv in (self.conv2d1, self.conv2d2, self.conv2d3):
            x = F.gelu(conv(x))
        n, ch, f, t = x.shape
        x = gemm.linear(x.permute(0, 3, 1, 2).reshape(n * t, ch * f).contiguous(), self.conv_out_w).reshape(n, t, -1)
        x = x + self.pos[:t]
        x = torch.cat([x[i, :_conv_len(L)] for i, L in enumerate(chunk_lens)]).contiguous()
        window = t * (self.n_window_infer // W)
        seq_lens = []
        for rows in per_audio:
            seq_lens += [window] * (rows // window) + ([rows % window] if rows % window else [])
        x = self.enc(x, seq_lens)
        x = gemm.linear(x, self.proj1_w, bias=self.proj1_b)
        x = F.gelu(x.float()).to(dt)
        return gemm.linear(x, self.proj2_w, bias=self.proj2_b), per_audio


class _Merger(nn.Module):
    """LayerNorm + (merge² neighbours concatenated) + linear, exact GELU, linear. ``post_shuffle``: the norm runs over
    the concatenated row instead of over every patch."""

    def __init__(self, hidden: int, unit: int, out_dim: int, post_shuffle: bool, dtype, device):
        super().__init__()
        self.unit, self.post_shuffle, self.wide = unit, post_shuffle, hidden * unit
        n = self.wide if post_shuffle else hidden
        self.norm_w, self.norm_b = _p((n,), dtype, device), _p((n,), dtype, device)
        self.fc1_w, self.fc1_b = _p((self.wide, self.wide), dtype, device), _p((self.wide,), dtype, device)
        self.fc2_w, self.fc2_b = _p((out_dim, self.wide), dtype, device), _p((out_dim,), dtype, device)

    def forward(self, x):
        """x: [n * unit, hidden] with the rows of a merge block adjacent."""
        if self.post_shuffle:
            x = x.reshape(-1, self.wide)
        x = norm_ops.norm(x.contiguous(), self.norm_w, 1e-6, bias=self.norm_b, layernorm=True)[0].reshape(-1, self.wide)
        x = gemm.linear(x, self.fc1_w, bias=self.fc1_b)
        return gemm.linear(F.gelu(x.float()).to(x.dtype), self.fc2_w, bias=self.fc2_b)


class OmniVisionEncoder(nn.Module):
    def __init__(self, c: EncoderConfig, patch: int = 16, temporal_patch: int = 2, merge: int = 2, pos_grid: int = 48,
                 out_dim: int = 2048, deepstack: tuple[int, ...] = (8, 16, 24), in_channels: int = 3, device="cpu"):
        super().__init__()
        if c.norm != "layernorm" or c.act != "gelu":
            raise ValueError("the vision tower uses LayerNorm and the tanh GELU")
        self.c, self.patch, self.tp, self.merge, self.pos_grid = c, patch, temporal_patch, merge, pos_grid
        self.deepstack, self.out_dim = tuple(deepstack), out_dim
        dt = c.dtype
        pdim = in_channels * temporal_patch * patch * patch
        self.patch_w, self.patch_b = _p((c.hidden_size, pdim), dt, device), _p((c.hidden_size,), dt, device)
        self.pos_table = _p((pos_grid * pos_grid, c.hidden_size), dt, device)
        self.enc = TransformerEncoder(c, device, final_norm=False)
        self.merger = _Merger(c.hidden_size, merge * merge, out_dim, False, dt, device)
        self.deep_mergers = nn.ModuleList([_Merger(c.hidden_size, merge * merge, out_dim, True, dt, device)
                                           for _ in self.deepstack])

    def init_random(self, seed=0):
        self.enc.init_random(seed)
        _randomize(self, seed + 11)
        return self

    # ---- input layout ----
    def patches(self, img: torch.Tensor):
        """[C, H, W] image or [C, T, H, W] clip -> ([t*h*w, C*tp*p*p] with the patches of a merge block adjacent,
        (t, h, w)). A still image is repeated over the temporal patch."""
        if img.dim() == 3:
            img = img[:, None].expand(-1, self.tp, -1, -1)
        C, T, H, W = img.shape
        p, tp, m = self.patch, self.tp, self.merge
        t, h, w = T // tp, H // p // m * m, W // p // m * m
        x = img[:, :t * tp, :h * p, :w * p].reshape(C, t, tp, h // m, m, p, w // m, m, p)
        x = x.permute(1, 3, 6, 4, 7, 0, 2, 5, 8)                   # t, h/m, w/m, m, m, C, tp, p, p
        return x.reshape(t * h * w, C * tp * p * p), (t, h, w)

    def _block_order(self, grid, device):
        """(row, col) of every patch in the tower's row order (merge blocks adjacent, frames repeated)."""
        t, h, w = grid
        m = self.merge
        rows = torch.arange(h, device=device).reshape(h // m, 1, m, 1).expand(h // m, w // m, m, m).reshape(-1)
        cols = torch.arange(w, device=device).reshape(1, w // m, 1, m).expand(h // m, w // m, m, m).reshape(-1)
        return rows.repeat(t), cols.repeat(t)

    def _pos_embed(self, grid, rows, cols):
        """The learned table read at corner-aligned fractional coordinates (four-neighbour weights)."""
        _, h, w = grid
        G, tbl = self.pos_grid, self.pos_table.float()
        ys = torch.linspace(0, G - 1, h, device=tbl.device)[rows]
        xs = torch.linspace(0, G - 1, w, device=tbl.device)[cols]
        y0, x0 = ys.int(), xs.int()
        y1, x1 = (y0 + 1).clamp(max=G - 1), (x0 + 1).clamp(max=G - 1)
        dy, dx = (ys - y0)[:, None], (xs - x0)[:, None]
        y0, x0, y1, x1 = y0.long(), x0.long(), y1.long(), x1.long()
        e = (tbl[y0 * G + x0] * (1 - dy) * (1 - dx) + tbl[y0 * G + x1] * (1 - dy) * dx
             + tbl[y1 * G + x0] * dy * (1 - dx) + tbl[y1 * G + x1] * dy * dx)
        return e.to(self.c.dtype)

    def _rope(self, rows, cols):
        D = self.c.head_dim
        q = D // 4
        inv = 1.0 / (10000.0 ** (torch.arange(q, dtype=torch.float32, device=rows.device) / q))
        ang = torch.cat([rows[:, None].float() * inv, cols[:, None].float() * inv], dim=-1)          # [T, D/2]
        cs, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]

        def apply(x):
            xf = x.float()
            a, b = xf[..., :D // 2], xf[..., D // 2:]
            return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1).to(x.dtype)
        return apply

    def forward(self, images: list[torch.Tensor]):
        """Returns (features [sum t*h*w / merge², out_dim], deepstack features (same shape each), rows per image,
        grids (t, h, w) in patches)."""
        toks, grids, rows, cols, seq_lens = [], [], [], [], []
        for im in images:
            p, g = self.patches(im.to(self.c.dtype))
            r, cc = self._block_order(g, p.device)
            toks.append(p), grids.append(g), rows.append(r), cols.append(cc)
            seq_lens += [g[1] * g[2]] * g[0]                       # attention stays inside a frame
        x = gemm.linear(torch.cat(toks).contiguous(), self.patch_w, bias=self.patch_b)
        x = x + torch.cat([self._pos_embed(g, r, cc) for g, r, cc in zip(grids, rows, cols)])
        rope = self._rope(torch.cat(rows), torch.cat(cols))
        taps = []
        if self.deepstack:
            x, taps = self.enc(x, seq_lens, rope=rope, collect=list(self.deepstack))
        else:
            x = self.enc(x, seq_lens, rope=rope)
        deep = [mg(t) for mg, t in zip(self.deep_mergers, taps)]
        unit = self.merge * self.merge
        return self.merger(x), deep, [g[0] * g[1] * g[2] // unit for g in grids], grids
