"""Decoder of the Cosmos3 sound tokenizer: jointly denoised sound latents [B, 64, T] -> stereo waveform
[B, 2, T * hop] at 48 kHz (hop = product of the up-sampling strides, 1920 for the published geometry).

An Oobleck-style stack: input conv (k7) -> five up-sampling blocks (snake, transposed conv of stride s and kernel 2s,
three dilated residual units with dilations 1 / 3 / 9) -> snake -> output conv (k7, no bias). The checkpoint stores
every convolution weight-normalised (``weight_g`` / ``weight_v``); the norm is folded into a plain weight once at
load time, so inference runs plain convolutions, and the snake activation ``x + sin^2(a x) / b`` uses ``a = exp(alpha)``
and ``1 / (exp(beta) + 1e-9)`` computed once as well.

``load_sound_decoder`` reads ``sound_tokenizer/config.json`` and ``diffusion_pytorch_model.safetensors`` under a model
directory, takes the ``decoder.*`` tensors (a full auto-encoder checkpoint also carries an encoder, which is not
built) and fails if any decoder tensor is missing, unknown or of the wrong shape.

Reference counterpart: mstar/model/cosmos3/components/sound_tokenizer.py (:24-119 modules, :131-231 config, loading,
latent de-normalisation and ``decode``).
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.nn.functional as F
from torch import nn


def sound_decoder_config(small: bool = False) -> dict:
    if small:
        return dict(sampling_rate=480, dec_out_channels=2, vocoder_input_dim=8, dec_strides=[2, 2], dec_dim=8,
                    dec_c_mults=[1, 2], normalization_type="none")
    return dict(sampling_rate=48000, dec_out_channels=2, vocoder_input_dim=64, dec_strides=[2, 4, 5, 6, 8], dec_dim=320,
                dec_c_mults=[1, 2, 4, 8, 16], normalization_type="none")


def _first(cfg: dict, *keys, default=None):
    for k in keys:
        if cfg.get(k) is not None:
            return cfg[k]
    return default


class Snake(nn.Module):
    """x + sin^2(a x) / b per channel; ``a`` and ``1 / b`` are stored ready to use."""

    def __init__(self, channels: int):
        super().__init__()
        self.a = nn.Parameter(torch.ones(1, channels, 1), requires_grad=False)
        self.inv_b = nn.Parameter(torch.ones(1, channels, 1), requires_grad=False)

    def set_log_params(self, alpha: torch.Tensor, beta: torch.Tensor) -> None:
        self.a.data.copy_(torch.exp(alpha.float()).reshape(self.a.shape).to(self.a.dtype))
        self.inv_b.data.copy_((torch.exp(beta.float()) + 1e-9).reciprocal().reshape(self.inv_b.shape).to(self.inv_b.dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.addcmul(x, self.inv_b, torch.sin(self.a * x).square())


class ResidualUnit(nn.Module):
    def __init__(self, dim: int, dilation: int):
        super().__init__()
        self.snake1, self.snake2 = Snake(dim), Snake(dim)
        self.conv1 = nn.Conv1d(dim, dim, 7, dilation=dilation, padding=3 * dilation)
        self.conv2 = nn.Conv1d(dim, dim, 1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.conv2(self.snake2(self.conv1(self.snake1(x))))


class UpBlock(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int):
        super().__init__()
        self.snake1 = Snake(cin)
        self.conv_t1 = nn.ConvTranspose1d(cin, cout, 2 * stride, stride=stride, padding=math.ceil(stride / 2),
                                          output_padding=stride % 2)
        self.res_unit1, self.res_unit2, self.res_unit3 = ResidualUnit(cout, 1), ResidualUnit(cout, 3), ResidualUnit(cout, 9)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.res_unit3(self.res_unit2(self.res_unit1(self.conv_t1(self.snake1(x)))))


class SoundDecoder(nn.Module):
    def __init__(self, config: dict | None = None):
        super().__init__()
        cfg = dict(config or sound_decoder_config())
        self.sample_rate = int(_first(cfg, "sampling_rate", "sample_rate", default=48000))
        self.audio_channels = int(_first(cfg, "dec_out_channels", "audio_channels", default=2 if cfg.get("stereo", True) else 1))
        self.latent_ch = int(_first(cfg, "vocoder_input_dim", "io_channels", "latent_ch", default=64))
        strides = [int(s) for s in _first(cfg, "dec_strides", default=[2, 4, 5, 6, 8])]
        self.hop_size = int(_first(cfg, "hop_size", default=math.prod(strides)))
        if math.prod(strides) != self.hop_size:
            raise ValueError(f"sound decoder: strides {strides} do not multiply to the hop size {self.hop_size}")
        self.latent_fps = self.sample_rate / self.hop_size
        norm = str(_first(cfg, "normalization_type", default="none"))
        if norm == "none" and cfg.get("normalize_latents"):
            norm = "tanh"
        if norm not in ("none", "tanh"):
            raise ValueError(f"sound decoder: unknown latent normalisation {norm!r}")
        self.normalization = norm
        self.tanh_in = float(_first(cfg, "tanh_input_scale", default=1.5))
        self.tanh_out = float(_first(cfg, "tanh_output_scale", default=3.5))
        self.tanh_clamp = float(_first(cfg, "tanh_clamp", default=0.995))
        dim = int(_first(cfg, "dec_dim", default=320))
        mults = [1] + [int(m) for m in _first(cfg, "dec_c_mults", default=[1, 2, 4, 8, 16])]
        ups = list(reversed(strides))                       # the widest layer up-samples with the largest stride
        self.conv1 = nn.Conv1d(self.latent_ch, dim * mults[-1], 7, padding=3)
        self.block = nn.ModuleList(UpBlock(dim * mults[len(ups) - i], dim * mults[len(ups) - i - 1], s)
                                   for i, s in enumerate(ups))
        self.snake1 = Snake(dim)
        self.conv2 = nn.Conv1d(dim, self.audio_channels, 7, padding=3, bias=False)
        self.requires_grad_(False)

    def num_samples(self, latent_frames: int) -> int:
        return int(latent_frames) * self.hop_size

    def num_latent_frames(self, samples: int) -> int:
        return max(1, math.ceil(max(1, int(samples)) / self.hop_size))

    def denormalize(self, z: torch.Tensor) -> torch.Tensor:
        if self.normalization == "none":
            return z
        y = torch.clamp(z.float() / self.tanh_out, -self.tanh_clamp, self.tanh_clamp)
        return (torch.atanh(y) * self.tanh_in).to(z.dtype)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """[B, C, T] or [C, T] -> waveform in [-1, 1], [B, channels, T * hop] (batch dimension dropped for [C, T])."""
        single = latents.dim() == 2
        x = latents[None] if single else latents
        x = self.conv1(self.denormalize(x).to(self.conv1.weight.dtype))
        for b in self.block:
            x = b(x)
        wav = self.conv2(self.snake1(x)).clamp(-1.0, 1.0)
        return wav[0] if single else wav

    forward = decode

    # ---- checkpoint layout ----
    def checkpoint_entries(self) -> dict[str, tuple]:
        """Checkpoint key -> (kind, module): every tensor a decoder checkpoint must hold."""
        out: dict[str, tuple] = {}

        def conv(prefix, m, bias=True):
            out[prefix + ".weight_g"] = ("g", m)
            out[prefix + ".weight_v"] = ("v", m)
            if bias:
                out[prefix + ".bias"] = ("bias", m)

        def snake(prefix, m):
            out[prefix + ".alpha"] = ("alpha", m)
            out[prefix + ".beta"] = ("beta", m)
        conv("decoder.conv1", self.conv1)
        for i, b in enumerate(self.block):
            p = f"decoder.block.{i}"
            snake(p + ".snake1", b.snake1)
            conv(p + ".conv_t1", b.conv_t1)
            for j, ru in enumerate((b.res_unit1, b.res_unit2, b.res_unit3), 1):
                q = f"{p}.res_unit{j}"
                snake(q + ".snake1", ru.snake1)
                conv(q + ".conv1", ru.conv1)
                snake(q + ".snake2", ru.snake2)
                conv(q + ".conv2", ru.conv2)
        snake("decoder.snake1", self.snake1)
        conv("decoder.conv2", self.conv2, bias=False)
        return out

    def load_checkpoint_tensors(self, tensors: dict[str, torch.Tensor]) -> None:
        """Strict: every decoder key present with the right shape, no unknown ``decoder.*`` key; other prefixes (an
        encoder shipped in the same file) are ignored."""
        entries = self.checkpoint_entries()
        have = {k: v for k, v in tensors.items() if k.startswith("decoder.")}
        missing = sorted(set(entries) - set(have))
        unknown = sorted(set(have) - set(entries))
        if missing or unknown:
            raise KeyError(f"sound decoder checkpoint: missing {missing[:8]} unknown {unknown[:8]}")
        g_of, v_of, snakes = {}, {}, {}
        for k, (kind, m) in entries.items():
            t = have[k]
            if kind == "g":
                g_of[id(m)] = (k, t, m)
            elif kind == "v":
                v_of[id(m)] = (k, t, m)
            elif kind == "bias":
                if tuple(t.shape) != tuple(m.bias.shape):
                    raise ValueError(f"{k}: shape {tuple(t.shape)} != {tuple(m.bias.shape)}")
                m.bias.data.copy_(t.to(m.bias.dtype))
            else:
                snakes.setdefault(id(m), [m, None, None])[1 if kind == "alpha" else 2] = (k, t)
        for mid, (kv, v, m) in v_of.items():
            kg, g, _ = g_of[mid]
            if tuple(v.shape) != tuple(m.weight.shape):
                raise ValueError(f"{kv}: shape {tuple(v.shape)} != {tuple(m.weight.shape)}")
            if g.numel() != v.shape[0]:
                raise ValueError(f"{kg}: {g.numel()} gains for {v.shape[0]} slices")
            vf = v.float()
            norm = vf.flatten(1).norm(dim=1).reshape(-1, *([1] * (vf.dim() - 1)))
            m.weight.data.copy_((vf * (g.float().reshape(norm.shape) / norm)).to(m.weight.dtype))
        for m, a, b in snakes.values():
            for (k, t) in (a, b):
                if t.numel() != m.a.numel():
                    raise ValueError(f"{k}: {t.numel()} values for {m.a.numel()} channels")
            m.set_log_params(a[1], b[1])


def load_sound_decoder(model_dir: str, device="cpu", dtype=torch.bfloat16) -> SoundDecoder:
    """``model_dir/sound_tokenizer/{config.json, diffusion_pytorch_model.safetensors}`` -> decoder on ``device``."""
    from safetensors.torch import load_file
    d = os.path.join(model_dir, "sound_tokenizer")
    with open(os.path.join(d, "config.json")) as f:
        dec = SoundDecoder(json.load(f))
    dec.load_checkpoint_tensors(load_file(os.path.join(d, "diffusion_pytorch_model.safetensors")))
    return dec.eval().to(device=device, dtype=dtype)


def pcm_layout(wav: torch.Tensor) -> torch.Tensor:
    """[channels, N] -> [N, channels]: the sample order of interleaved PCM."""
    return wav.transpose(0, 1).contiguous() if wav.dim() == 2 else wav


__all__ = ["SoundDecoder", "load_sound_decoder", "sound_decoder_config", "pcm_layout", "F"]
