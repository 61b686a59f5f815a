"""Diffusion-transformer family. Two block styles share the kernels:

``AdaLNDiT`` (Wan2.2-class): LayerNorm without affine + (shift, scale, gate) modulation from the timestep
embedding, bidirectional self-attention with full-width q/k RMSNorm and 3-axis rotary embedding, cross-attention to
a fixed text context (its K/V are projected once per request), GELU MLP. Classifier-free guidance runs as a batch
of two sequences.

``MoTGenTower`` (Cosmos3 / BAGEL-class "mixture of transformers"): a second set of decoder weights (the
generation expert) that runs over the noisy latent tokens and attends to [cached prefix ‖ fresh tokens]; the
prefix K/V were written to the paged pool by the understanding tower's prefill, the fresh K/V never enter the
pool. The two key sets are attended separately (paged kernel, dense kernel) and merged by their log-sum-exps.
Tensor parallel (column / row sharded projections) and Ulysses sequence parallel (rows sharded, heads exchanged
around attention over the symmetric heap) compose as a [sp][tp] mesh.

Fused on the GPU: norm + modulation in one kernel, q/k norm + rotary + K/V layout in one kernel, bias / GELU /
SwiGLU / residual in the GEMM epilogue, gate * y + x in one kernel.

Reference counterparts: Wan2.2 DiT (mstar/model/wan22/components/dit.py:225-364: block :225-274, rope :100-140,
head :276-300), Cosmos3 transformer (mstar/model/cosmos3/components/transformer.py: forward_gen :372-382,
timestep scatter-add :483-499, patchify :501-562, _sp_run_gen_layers :831-859, denoise_step_batched_cfg
:943-1037), BAGEL MoT split (mstar/model/bagel/components/language_model.py:58-84).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops import elementwise as ew_ops
from ..ops import gemm
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from ..parallel.comm import CommGroup
from ..parallel.sequence_parallel import UlyssesExchange
from .decoder import DecoderConfig, _param, tp_reduce


# ------------------------------------------------------------------ shared helpers
def sinusoidal_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    """fp32 [n, dim]: cos half then sin half (the diffusers / Wan convention)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = t.float().reshape(-1, 1) * freqs[None]
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1)


def rope_axes_tables(head_dim: int, axes_dims: tuple[int, ...] | None, theta: float, device):
    """inv_freq [D/2] fp32 and axis_of_freq [D/2] int8 for a rotary embedding whose frequency bands belong to
    different position axes (t, h, w). Every axis gets its own geometric ladder over its own width."""
    if not axes_dims:
        return rope_ops.make_inv_freq(head_dim, theta, device), None
    assert sum(axes_dims) == head_dim and all(d % 2 == 0 for d in axes_dims)
    inv, ax = [], []
    for a, d in enumerate(axes_dims):
        inv.append(1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
        ax += [a] * (d // 2)
    return torch.cat(inv).to(device), torch.tensor(ax, dtype=torch.int8, device=device)


def grid_positions(F: int, H: int, W: int, device, offset: tuple[int, int, int] = (0, 0, 0)) -> torch.Tensor:
    """int32 [3, F*H*W] (t, h, w) coordinates of a row-major latent token grid."""
    t = torch.arange(F, dtype=torch.int32, device=device) + offset[0]
    h = torch.arange(H, dtype=torch.int32, device=device) + offset[1]
    w = torch.arange(W, dtype=torch.int32, device=device) + offset[2]
    g = torch.stack(torch.meshgrid(t, h, w, indexing="ij"), dim=0)
    return g.reshape(3, -1).contiguous()


def patchify(x: torch.Tensor, patch: tuple[int, int, int]) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """[C, F, H, W] -> ([F' H' W', C pt ph pw], (F', H', W'))."""
    C, F, H, W = x.shape
    pt, ph, pw = patch
    Fp, Hp, Wp = F // pt, H // ph, W // pw
    x = x.reshape(C, Fp, pt, Hp, ph, Wp, pw).permute(1, 3, 5, 0, 2, 4, 6)
    return x.reshape(Fp * Hp * Wp, C * pt * ph * pw).contiguous(), (Fp, Hp, Wp)


def unpatchify(tok: torch.Tensor, grid: tuple[int, int, int], patch: tuple[int, int, int], C: int) -> torch.Tensor:
    """[F' H' W', pt ph pw C] -> [C, F, H, W] (channel is the fastest index of a token, as the heads emit it)."""
    Fp, Hp, Wp = grid
    pt, ph, pw = patch
    x = tok.reshape(Fp, Hp, Wp, pt, ph, pw, C).permute(6, 0, 3, 1, 4, 2, 5)
    return x.reshape(C, Fp * pt, Hp * ph, Wp * pw).contiguous()


REGION_AR_MIN_ROWS = 2048


def row_parallel(x, w, tp: CommGroup, bias=None, residual=None):
    """sum over the TP group of x_shard @ w_shard.T, + bias, + residual (both fused when there is one rank)."""
    if tp.size == 1:
        return gemm.linear(x, w, bias=bias, residual=residual)
    if (tp.symm is not None and x.is_cuda and x.dim() == 2 and x.shape[0] >= REGION_AR_MIN_ROWS and w.shape[0] % 8 == 0
            and x.dtype == torch.bfloat16 and residual is None and os.environ.get("MSTAR_REGION_AR", "1") != "0"):
        # large M: the GEMM writes its partial straight into the group's symmetric scratch and the all-reduce runs in
        # place there (nothing staged, nothing copied out; 0.85 x the time of GEMM + NCCL all-reduce at 21120 x 2048
        # on two GPUs). The result lives in the scratch until the next such call; callers consume it at once.
        M, N = x.shape[0], w.shape[0]
        reg, off = tp.symm.scratch(2 * M * N * 2 + (1 << 20))
        if os.environ.get("MSTAR_GEMM_TILE_AR", "0") == "1" and x.shape[1] % 8 == 0 and not isinstance(w, gemm.PackedWeight):
            # the all-reduce inside the GEMM kernel, row group by row group (correct, but slower on two GPUs: a
            # communication CTA moves about 10 GB/s over NVLink, so the few SMs the GEMM can spare do not fill a link)
            return tp.symm.linear_all_reduce_tiles(x.contiguous(), w, reg, off, bias=bias if tp.rank == 0 else None)
        y = reg.view(off, (M, N), torch.bfloat16)
        gemm.linear(x, w, bias=bias if tp.rank == 0 else None, out=y)
        tp.symm.all_reduce_inplace(reg, off, M * N)
        return y
    y = gemm.linear(x, w, bias=bias if tp.rank == 0 else None)
    if tp.symm is not None and y.is_cuda:
        return tp.symm.all_reduce(y.contiguous(), residual=residual)
    y = tp.all_reduce(y)
    return y if residual is None else (y.float() + residual.float()).to(y.dtype)


@dataclass
class DiTConfig:
    hidden_size: int = 3072
    num_layers: int = 30
    num_heads: int = 24
    head_dim: int = 128
    ffn_dim: int = 14336
    in_channels: int = 48
    out_channels: int = 48
    patch_size: tuple[int, int, int] = (1, 2, 2)
    text_dim: int = 4096
    text_len: int = 512
    freq_dim: int = 256
    rope_theta: float = 10000.0
    eps: float = 1e-6
    dtype: torch.dtype = torch.bfloat16
    rope_axes: tuple[int, ...] = field(default_factory=tuple)     # () -> derived from head_dim (Wan split)

    def axes(self) -> tuple[int, int, int]:
        if self.rope_axes:
            return tuple(self.rope_axes)
        d = self.head_dim
        return (d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6))


def wan22_5b_config() -> DiTConfig:
    return DiTConfig()


# ------------------------------------------------------------------ AdaLN DiT (Wan2.2-class)
class AdaLNBlock(nn.Module):
    """``tp``: tensor-parallel group. Attention heads (self and cross) and the MLP's inner dimension are cut over it;
    the output projections are row-parallel sums. The q / k norms of this architecture normalise over ALL heads, so
    the ranks exchange the per-token sums of squares (two floats per token) before scaling their own heads."""

    def __init__(self, cfg: DiTConfig, device, tp: CommGroup | None = None):
        super().__init__()
        self.tp = tp or CommGroup.trivial()
        t = self.tp.size
        if cfg.num_heads % t or cfg.ffn_dim % t:
            raise ValueError(f"{cfg.num_heads} heads / MLP width {cfg.ffn_dim} cannot be cut {t} ways")
        H, Fd, dt = cfg.hidden_size, cfg.ffn_dim // t, cfg.dtype
        A = cfg.num_heads * cfg.head_dim // t               # this rank's attention width
        self.cfg, self.A = cfg, A
        self.modulation = _param((6, H), torch.float32, device)
        self.qkv_w, self.qkv_b = _param((3 * A, H), dt, device), _param((3 * A,), dt, device)
        self.norm_q, self.norm_k = _param((A,), dt, device), _param((A,), dt, device)
        self.o_w, self.o_b = _param((H, A), dt, device), _param((H,), dt, device)
        self.norm3_w, self.norm3_b = _param((H,), dt, device), _param((H,), dt, device)
        self.cq_w, self.cq_b = _param((A, H), dt, device), _param((A,), dt, device)
        self.ckv_w, self.ckv_b = _param((2 * A, H), dt, device), _param((2 * A,), dt, device)
        self.cnorm_q, self.cnorm_k = _param((A,), dt, device), _param((A,), dt, device)
        self.co_w, self.co_b = _param((H, A), dt, device), _param((H,), dt, device)
        self.ffn1_w, self.ffn1_b = _param((Fd, H), dt, device), _param((Fd,), dt, device)
        self.ffn2_w, self.ffn2_b = _param((H, Fd), dt, device), _param((H,), dt, device)

    def _norm_all_heads(self, parts: list[torch.Tensor], weights: list[torch.Tensor]) -> list[torch.Tensor]:
        """RMS norm over the full attention width of tensors of which this rank holds its heads' columns."""
        ss = torch.stack([p.float().pow(2).sum(-1) for p in parts], dim=-1)
        ss = self.tp.all_reduce(ss)
        full = self.A * self.tp.size
        return [(p.float() * torch.rsqrt(ss[:, i:i + 1] / full + self.cfg.eps) * w.float()).to(p.dtype)
                for i, (p, w) in enumerate(zip(parts, weights))]

    def project_context(self, ctx: torch.Tensor):
        """K/V of the text context for this block: [L_total, heads, D] each (done once per request)."""
        c = self.cfg
        kv = gemm.linear(ctx, self.ckv_w, bias=self.ckv_b)
        A = self.A
        if self.tp.size > 1:
            k = self._norm_all_heads([kv[:, :A]], [self.cnorm_k])[0]
        else:
            k, _ = norm_ops.norm(kv[:, :A], self.cnorm_k, c.eps)
        return (k.reshape(-1, A // c.head_dim, c.head_dim).contiguous(),
                kv[:, A:].reshape(-1, A // c.head_dim, c.head_dim).contiguous())

    def forward_tp(self, x, mod, positions, rope, self_plan, cross_plan, ctx_kv, exchange=None):
        """The block over this rank's heads and MLP columns and, with ``exchange`` (a ``UlyssesExchange``), over this
        rank's rows of the packed sequence: everything is row-local except the self-attention, around which heads
        and rows are swapped (every rank then attends over the full sequence for a part of its heads). Same
        result as ``forward``."""
        c, A, tp = self.cfg, self.A, self.tp
        nh, D = A // c.head_dim, c.head_dim
        inv_freq, axis = rope
        h, _ = norm_ops.norm(x, None, c.eps, layernorm=True, scale=mod[:, 1], shift=mod[:, 0])
        qkv = gemm.linear(h, self.qkv_w, bias=self.qkv_b)
        if tp.size > 1:
            qn, kn = self._norm_all_heads([qkv[:, :A], qkv[:, A:2 * A]], [self.norm_q, self.norm_k])
            qkv = torch.cat([qn, kn, qkv[:, 2 * A:]], dim=-1).contiguous()
        else:
            norm_ops.norm(qkv[:, :A], self.norm_q, c.eps, out=qkv[:, :A])
            norm_ops.norm(qkv[:, A:2 * A], self.norm_k, c.eps, out=qkv[:, A:2 * A])
        q, k, v = rope_ops.rope_kv(qkv, positions, inv_freq, nh, nh, D, axis_of_freq=axis, interleaved=True, dense_kv=True)
        if exchange is not None:
            q, k, v = exchange.to_heads(q, k, v)
        a = attn_ops.attention(q.contiguous(), self_plan, k=k.contiguous(), v=v.contiguous())
        if exchange is not None:
            a = exchange.to_sequence(a)
        y = row_parallel(a.reshape(-1, A), self.o_w, tp, bias=self.o_b)
        x = ew_ops.gated_residual(x, y, mod[:, 2])
        h, _ = norm_ops.norm(x, self.norm3_w, c.eps, layernorm=True, bias=self.norm3_b)
        q = gemm.linear(h, self.cq_w, bias=self.cq_b)
        q = self._norm_all_heads([q], [self.cnorm_q])[0] if tp.size > 1 else norm_ops.norm(q, self.cnorm_q, c.eps)[0]
        a = attn_ops.attention(q.reshape(-1, nh, D), cross_plan, k=ctx_kv[0], v=ctx_kv[1])
        x = row_parallel(a.reshape(-1, A), self.co_w, tp, bias=self.co_b, residual=x)
        h, _ = norm_ops.norm(x, None, c.eps, layernorm=True, scale=mod[:, 4], shift=mod[:, 3])
        h = gemm.linear(h, self.ffn1_w, bias=self.ffn1_b, epilogue=gemm.EPILOGUE_GELU)
        y = row_parallel(h, self.ffn2_w, tp, bias=self.ffn2_b)
        return ew_ops.gated_residual(x, y, mod[:, 5])

    def forward(self, x, mod, positions, rope, self_plan, cross_plan, ctx_kv):
        """x: [T, H]; mod: [n_mod, 6, H] bf16 = modulation + timestep projection; T rows split evenly over n_mod."""
        if self.tp.size > 1:
            return self.forward_tp(x, mod, positions, rope, self_plan, cross_plan, ctx_kv)
        c = self.cfg
        H, nh, D = c.hidden_size, c.num_heads, c.head_dim
        inv_freq, axis = rope
        # self-attention
        h, _ = norm_ops.norm(x, None, c.eps, layernorm=True, scale=mod[:, 1], shift=mod[:, 0])
        qkv = gemm.linear(h, self.qkv_w, bias=self.qkv_b)
        norm_ops.norm(qkv[:, :H], self.norm_q, c.eps, out=qkv[:, :H])
        norm_ops.norm(qkv[:, H:2 * H], self.norm_k, c.eps, out=qkv[:, H:2 * H])
        q, k, v = rope_ops.rope_kv(qkv, positions, inv_freq, nh, nh, D, axis_of_freq=axis, interleaved=True,
                                   dense_kv=True)
        a = attn_ops.attention(q, self_plan, k=k, v=v)
        y = gemm.linear(a.reshape(-1, H), self.o_w, bias=self.o_b)
        x = ew_ops.gated_residual(x, y, mod[:, 2])
        # cross-attention to the text context
        h, _ = norm_ops.norm(x, self.norm3_w, c.eps, layernorm=True, bias=self.norm3_b)
        q = gemm.linear(h, self.cq_w, bias=self.cq_b)
        q, _ = norm_ops.norm(q, self.cnorm_q, c.eps)
        a = attn_ops.attention(q.reshape(-1, nh, D), cross_plan, k=ctx_kv[0], v=ctx_kv[1])
        x = gemm.linear(a.reshape(-1, H), self.co_w, bias=self.co_b, residual=x)
        # MLP
        h, _ = norm_ops.norm(x, None, c.eps, layernorm=True, scale=mod[:, 4], shift=mod[:, 3])
        h = gemm.linear(h, self.ffn1_w, bias=self.ffn1_b, epilogue=gemm.EPILOGUE_GELU)
        y = gemm.linear(h, self.ffn2_w, bias=self.ffn2_b)
        return ew_ops.gated_residual(x, y, mod[:, 5])


# parameters of a block that are cut over the tensor-parallel group: name -> (dimension, number of stacked sections)
_ADALN_CUTS = {"qkv_w": (0, 3), "qkv_b": (0, 3), "norm_q": (0, 1), "norm_k": (0, 1), "o_w": (1, 1), "cq_w": (0, 1),
               "cq_b": (0, 1), "ckv_w": (0, 2), "ckv_b": (0, 2), "cnorm_q": (0, 1), "cnorm_k": (0, 1), "co_w": (1, 1),
               "ffn1_w": (0, 1), "ffn1_b": (0, 1), "ffn2_w": (1, 1)}


def adaln_shard(name: str, full: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """This rank's part of a full ``AdaLNDiT`` parameter (``blocks.N.<param>``): stacked projections (q | k | v,
    k | v) are cut section by section so that every rank keeps whole heads of each."""
    leaf = name.rsplit(".", 1)[-1]
    if size == 1 or not name.startswith("blocks.") or leaf not in _ADALN_CUTS:
        return full
    dim, sections = _ADALN_CUTS[leaf]
    parts = []
    for sec in full.chunk(sections, dim=dim):
        n = sec.shape[dim] // size
        parts.append(sec.narrow(dim, rank * n, n))
    return torch.cat(parts, dim=dim)


class AdaLNDiT(nn.Module):
    def __init__(self, cfg: DiTConfig, device="cpu", tp: CommGroup | None = None, sp: CommGroup | None = None):
        super().__init__()
        self.cfg, self.device = cfg, torch.device(device)
        self.tp = tp or CommGroup.trivial()
        self.sp = sp or CommGroup.trivial()
        self._exchange: dict = {}
        H, dt = cfg.hidden_size, cfg.dtype
        pdim = cfg.in_channels * math.prod(cfg.patch_size)
        self.patch_w, self.patch_b = _param((H, pdim), dt, device), _param((H,), dt, device)
        self.text1_w, self.text1_b = _param((H, cfg.text_dim), dt, device), _param((H,), dt, device)
        self.text2_w, self.text2_b = _param((H, H), dt, device), _param((H,), dt, device)
        self.time1_w, self.time1_b = _param((H, cfg.freq_dim), dt, device), _param((H,), dt, device)
        self.time2_w, self.time2_b = _param((H, H), dt, device), _param((H,), dt, device)
        self.tproj_w, self.tproj_b = _param((6 * H, H), dt, device), _param((6 * H,), dt, device)
        self.blocks = nn.ModuleList([AdaLNBlock(cfg, device, self.tp) for _ in range(cfg.num_layers)])
        self.head_mod = _param((2, H), torch.float32, device)
        odim = cfg.out_channels * math.prod(cfg.patch_size)
        self.head_w, self.head_b = _param((odim, H), dt, device), _param((odim,), dt, device)
        self.rope = rope_axes_tables(cfg.head_dim, cfg.axes(), cfg.rope_theta, self.device)

    def init_random(self, seed: int = 0) -> "AdaLNDiT":
        """Every rank draws the FULL tensors from the same generator, in the same order, and keeps its part: a sharded
        model holds the weights of the single-rank model with the same seed."""
        g = torch.Generator().manual_seed(seed)
        t, r = self.tp.size, self.tp.rank
        for n, p in self.named_parameters():
            shape = list(p.shape)
            leaf = n.rsplit(".", 1)[-1]
            if t > 1 and n.startswith("blocks.") and leaf in _ADALN_CUTS:
                shape[_ADALN_CUTS[leaf][0]] *= t
            if "norm" in n and n.endswith(("_q", "_k", "3_w")):
                full = torch.ones(shape)
            elif p.dim() == 1:
                full = torch.randn(shape, generator=g) * 0.02
            elif "modulation" in n or "head_mod" in n:
                full = torch.randn(shape, generator=g) * 0.1
            else:
                full = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            p.data.copy_(adaln_shard(n, full, r, t).to(p.dtype))
        return self

    # -- once per request --
    def encode_context(self, text_emb: torch.Tensor):
        """text_emb: [L_total, text_dim] (all guidance branches packed) -> per-block (K, V)."""
        c = gemm.linear(text_emb.to(self.cfg.dtype), self.text1_w, bias=self.text1_b, epilogue=gemm.EPILOGUE_GELU)
        c = gemm.linear(c, self.text2_w, bias=self.text2_b)
        return [blk.project_context(c) for blk in self.blocks]

    # -- one denoising forward --
    def forward(self, latents: torch.Tensor, timesteps: torch.Tensor, ctx_kv: list, ctx_lens: list[int]):
        """latents: [B, C, F, H, W] (B guidance branches / requests of one shape); timesteps: [B] or [B, F'] (one
        per latent frame: image-to-video keeps the first frame at t = 0). Returns the model output, same shape,
        fp32."""
        cfg = self.cfg
        B = latents.shape[0]
        toks, grid = [], None
        for b in range(B):
            t, grid = patchify(latents[b], cfg.patch_size)
            toks.append(t)
        S = toks[0].shape[0]
        x = gemm.linear(torch.cat(toks).to(cfg.dtype), self.patch_w, bias=self.patch_b)
        ts = timesteps.reshape(B, -1)
        n_per = ts.shape[1]
        assert S % n_per == 0
        e = sinusoidal_embedding(ts.reshape(-1), cfg.freq_dim).to(cfg.dtype)
        e = gemm.linear(e, self.time1_w, bias=self.time1_b)
        e = gemm.linear(torch.nn.functional.silu(e.float()).to(cfg.dtype), self.time2_w, bias=self.time2_b)
        e6 = gemm.linear(torch.nn.functional.silu(e.float()).to(cfg.dtype), self.tproj_w, bias=self.tproj_b,
                         out_dtype=torch.float32).reshape(B * n_per, 6, cfg.hidden_size)
        pos = grid_positions(*grid, self.device).repeat(1, B)
        G = 1
        if self.sp.size > 1:
            return self._forward_sp(x, e, e6, pos, B, S, n_per, grid, ctx_kv, ctx_lens)
        self_plan = attn_ops.dense_plan([S] * B, [S] * B, G, self.device, causal=False)
        cross_plan = attn_ops.dense_plan([S] * B, ctx_lens, G, self.device, causal=False)
        for i, blk in enumerate(self.blocks):
            mod = (blk.modulation.float()[None] + e6).to(cfg.dtype)
            x = blk(x, mod, pos, self.rope, self_plan, cross_plan, ctx_kv[i])
        hm = (self.head_mod.float()[None] + e.float().reshape(B * n_per, 1, -1)).to(cfg.dtype)
        h, _ = norm_ops.norm(x, None, cfg.eps, layernorm=True, scale=hm[:, 1], shift=hm[:, 0])
        out = gemm.linear(h, self.head_w, bias=self.head_b, out_dtype=torch.float32)
        return torch.stack([unpatchify(out[b * S:(b + 1) * S], grid, cfg.patch_size, cfg.out_channels)
                            for b in range(B)])


    def _forward_sp(self, x, e, e6, pos, B, S, n_per, grid, ctx_kv, ctx_lens):
        """Sequence-parallel blocks: this rank keeps a contiguous range of the packed rows (B branches x S tokens).
        Norms, modulation, projections, cross-attention and MLP work on those rows; the self-attention swaps rows
        for heads (Ulysses). A rank's rows must be whole modulation groups or lie inside one (a group = the tokens
        of one branch that share a timestep)."""
        from ..parallel.sequence_parallel import UlyssesExchange, gather_sequence, sp_seq_split
        cfg, sp = self.cfg, self.sp
        T = B * S
        nh_local = cfg.num_heads // self.tp.size
        if nh_local % sp.size:
            raise ValueError(f"{nh_local} heads per tensor-parallel rank cannot be cut over {sp.size} sequence ranks")
        off = sp_seq_split(T, sp.size)
        r0, r1 = off[sp.rank], off[sp.rank + 1]
        gsz = S // n_per                                   # rows per modulation group
        if (r0 % gsz == 0 and r1 % gsz == 0):
            groups = slice(r0 // gsz, r1 // gsz)
        elif r0 // gsz == (r1 - 1) // gsz:
            groups = slice(r0 // gsz, r0 // gsz + 1)
        else:
            raise ValueError(f"rows {r0}..{r1} of {T} split modulation groups of {gsz} rows unevenly: use a sequence-"
                             f"parallel degree that divides the branches or the frames")
        key = (T, nh_local)
        ex = self._exchange.get(key)
        if ex is None:
            ex = self._exchange[key] = UlyssesExchange(sp, T, nh_local, nh_local, cfg.head_dim, cfg.dtype)
        x = x[r0:r1].contiguous()
        pos = pos[:, r0:r1].contiguous()
        self_plan = attn_ops.dense_plan([S] * B, [S] * B, 1, self.device, causal=False)
        q_loc = [max(0, min(r1, (b + 1) * S) - max(r0, b * S)) for b in range(B)]
        keep = [b for b in range(B) if q_loc[b] > 0]
        cross_plan = attn_ops.dense_plan([q_loc[b] for b in keep], [ctx_lens[b] for b in keep], 1, self.device, causal=False)
        c_off = [0]
        for n in ctx_lens:
            c_off.append(c_off[-1] + n)
        rows = torch.cat([torch.arange(c_off[b], c_off[b + 1], device=self.device) for b in keep])
        for i, blk in enumerate(self.blocks):
            mod = (blk.modulation.float()[None] + e6[groups]).to(cfg.dtype)
            kv = ctx_kv[i] if len(keep) == B else (ctx_kv[i][0].index_select(0, rows), ctx_kv[i][1].index_select(0, rows))
            x = blk.forward_tp(x, mod, pos, self.rope, self_plan, cross_plan, kv, exchange=ex)
        hm = (self.head_mod.float()[None] + e.float().reshape(B * n_per, 1, -1)[groups]).to(cfg.dtype)
        h, _ = norm_ops.norm(x, None, cfg.eps, layernorm=True, scale=hm[:, 1], shift=hm[:, 0])
        out = gemm.linear(h, self.head_w, bias=self.head_b, out_dtype=torch.float32)
        out = gather_sequence(out, sp, T)                  # only the head's [rows, patch] result travels
        return torch.stack([unpatchify(out[b * S:(b + 1) * S], grid, cfg.patch_size, cfg.out_channels)
                            for b in range(B)])


# ------------------------------------------------------------------ generation expert of a mixture of transformers
class MoTGenLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int, tp: CommGroup, device):
        super().__init__()
        self.cfg, self.layer_idx, self.tp = cfg, layer_idx, tp
        H, D = cfg.hidden_size, cfg.head_dim
        self.Hq, self.Hkv = cfg.num_heads // tp.size, max(1, cfg.num_kv_heads // tp.size)
        self.F = cfg.intermediate_size // tp.size
        dt = cfg.dtype
        self.input_norm = _param((H,), dt, device)
        self.qkv_proj = _param(((self.Hq + 2 * self.Hkv) * D, H), dt, device)
        self.qkv_bias = _param(((self.Hq + 2 * self.Hkv) * D,), dt, device) if cfg.qkv_bias else None
        self.q_norm = _param((D,), dt, device) if cfg.qk_norm else None
        self.k_norm = _param((D,), dt, device) if cfg.qk_norm else None
        self.o_proj = _param((H, self.Hq * D), dt, device)
        self.post_norm = _param((H,), dt, device)
        self.gate_up_proj = _param((2 * self.F, H), dt, device)
        self.down_proj = _param((H, self.F), dt, device)


class MoTGenTower(nn.Module):
    """Generation-expert weights with the shape of the understanding decoder ``cfg``. ``forward`` runs the noisy
    tokens of a batch of (request, guidance branch) entries; every entry has the same number of tokens."""

    def __init__(self, cfg: DecoderConfig, tp: CommGroup | None = None, sp: CommGroup | None = None, device="cpu",
                 rope_axes: tuple[int, ...] | None = None):
        super().__init__()
        self.cfg = cfg
        self.tp = tp or CommGroup.trivial()
        self.sp = sp or CommGroup.trivial()
        self.device = torch.device(device)
        self.layers = nn.ModuleList([MoTGenLayer(cfg, i, self.tp, device) for i in range(cfg.num_layers)])
        self.final_norm = _param((cfg.hidden_size,), cfg.dtype, device)
        if rope_axes is None and cfg.mrope_sections:
            self.inv_freq = rope_ops.make_inv_freq(cfg.head_dim, cfg.rope_theta, self.device)
            self.axis_of_freq = rope_ops.mrope_axis_table(cfg.mrope_sections, cfg.mrope_interleaved).to(self.device)
        else:
            self.inv_freq, self.axis_of_freq = rope_axes_tables(cfg.head_dim, rope_axes, cfg.rope_theta, self.device)
        self._exchange: dict[tuple, UlyssesExchange] = {}

    @torch.no_grad()
    def init_random(self, seed: int = 1) -> "MoTGenTower":
        """Every rank draws the full tensors from the same generator and keeps its tensor-parallel slice."""
        from .decoder import shard_qkv
        g = torch.Generator().manual_seed(seed)
        c, tp = self.cfg, self.tp
        H, D, Hq, Hkv, Fi = c.hidden_size, c.head_dim, c.num_heads, c.num_kv_heads, c.intermediate_size

        def draw(shape, fan):
            return torch.randn(shape, generator=g) / math.sqrt(fan)
        for L in self.layers:
            q, k, v = draw((Hq * D, H), H), draw((Hkv * D, H), H), draw((Hkv * D, H), H)
            L.qkv_proj.copy_(shard_qkv(q, k, v, Hq, Hkv, D, tp.rank, tp.size).to(c.dtype))
            if L.qkv_bias is not None:
                L.qkv_bias.zero_()
            o = draw((H, Hq * D), Hq * D)
            L.o_proj.copy_(o[:, tp.rank * L.Hq * D:(tp.rank + 1) * L.Hq * D].to(c.dtype))
            gt, up, dn = draw((Fi, H), H), draw((Fi, H), H), draw((H, Fi), Fi)
            sl = slice(tp.rank * L.F, (tp.rank + 1) * L.F)
            L.gate_up_proj.copy_(gemm.interleave_gate_up(gt[sl], up[sl]).to(c.dtype))
            L.down_proj.copy_(dn[:, sl].to(c.dtype))
            for n in (L.input_norm, L.post_norm, L.q_norm, L.k_norm):
                if n is not None:
                    n.fill_(1.0)
        self.final_norm.fill_(1.0)
        return self

    def exchange(self, S_total: int) -> UlyssesExchange:
        key = (S_total,)
        ex = self._exchange.get(key)
        if ex is None:
            l0 = self.layers[0]
            ex = UlyssesExchange(self.sp, S_total, l0.Hq, l0.Hkv, self.cfg.head_dim, self.cfg.dtype)
            self._exchange[key] = ex
        return ex

    def layer_qkv(self, li: int, x, residual, positions, ctx=None):
        """Pre-attention half of layer ``li`` on a row subset: returns (q, k, v, residual). With ``ctx`` the K/V
        rows are also written into the paged pool at the subset's cache slots."""
        L, cfg = self.layers[li], self.cfg
        h, residual = (norm_ops.norm(x, L.input_norm, cfg.rms_eps, residual=residual) if residual is not None
                       else (norm_ops.norm(x, L.input_norm, cfg.rms_eps)[0], x.clone()))
        qkv = gemm.linear(h, L.qkv_proj, bias=L.qkv_bias)
        kw = {}
        if ctx is not None:
            kw = dict(cache=ctx["kv"], token_req=ctx["token_req"], cache_pos=ctx["cache_pos"],
                      page_indptr=ctx["page_indptr"], page_indices=ctx["page_indices"])
        q, k, v = rope_ops.rope_kv(qkv, positions, self.inv_freq, L.Hq, L.Hkv, cfg.head_dim,
                                   axis_of_freq=self.axis_of_freq, q_norm_w=L.q_norm, k_norm_w=L.k_norm,
                                   norm_eps=cfg.rms_eps, dense_kv=ctx is None, **kw)
        return q, k, v, residual

    def layer_out(self, li: int, attn, residual):
        """Post-attention half of layer ``li``: o_proj, post norm, MLP. Returns (x, residual)."""
        L, cfg = self.layers[li], self.cfg
        x = row_parallel(attn.reshape(attn.shape[0], -1), L.o_proj, self.tp)
        h, residual = norm_ops.norm(x, L.post_norm, cfg.rms_eps, residual=residual)
        g = gemm.linear(h, L.gate_up_proj, epilogue=gemm.EPILOGUE_SWIGLU)
        return row_parallel(g, L.down_proj, self.tp), residual

    def forward(self, x: torch.Tensor, positions: torch.Tensor, self_plan, *, prefix_ctx=None,
                S_total: int | None = None) -> torch.Tensor:
        """x: [T_local, H] rows of this sequence-parallel rank (all rows when sp = 1); positions: int32
        [axes, T_local]; self_plan: dense bidirectional plan over the FULL packed sequence (S_total rows);
        prefix_ctx: BatchContext planned with ``write_cache=False, causal=False`` over the cached prefixes (its
        q rows are the full packed sequence too), or None when no entry has a prefix."""
        cfg = self.cfg
        D = cfg.head_dim
        sp = self.sp.size > 1
        S_total = S_total if S_total is not None else x.shape[0]
        ex = self.exchange(S_total) if sp else None
        residual = None
        for li, L in enumerate(self.layers):
            h, residual = (norm_ops.norm(x, L.input_norm, cfg.rms_eps) if residual is None
                           else norm_ops.norm(x, L.input_norm, cfg.rms_eps, residual=residual))
            if residual is None:
                residual = x.clone()      # the residual stream is updated in place; keep the caller's tensor
            qkv = gemm.linear(h, L.qkv_proj, bias=L.qkv_bias)
            if sp and ex.can_fuse_rope(qkv, 2 * self.inv_freq.numel()):
                # QK-norm + RoPE whose stores are the Ulysses exchange: no [T, H, D] intermediate, no exchange kernels
                q, k, v = ex.rope_to_heads(qkv, positions, self.inv_freq, self.axis_of_freq, L.q_norm, L.k_norm,
                                           cfg.rms_eps)
            else:
                q, k, v = rope_ops.rope_kv(qkv, positions, self.inv_freq, L.Hq, L.Hkv, D,
                                           axis_of_freq=self.axis_of_freq, q_norm_w=L.q_norm, k_norm_w=L.k_norm,
                                           norm_eps=cfg.rms_eps, dense_kv=True)
                if sp:
                    q, k, v = ex.to_heads(q, k, v)
            if prefix_ctx is not None:
                o_f, l_f = attn_ops.attention(q, self_plan, k=k, v=v, lse=True)
                o_p, l_p = attn_ops.attention(q, prefix_ctx.plan, kv_cache=prefix_ctx.kv(li), lse=True)
                a = attn_ops.attn_merge(o_p, l_p, o_f, l_f)
            else:
                a = attn_ops.attention(q, self_plan, k=k, v=v)
            if sp:
                a = ex.to_sequence(a)
            x = row_parallel(a.reshape(a.shape[0], -1), L.o_proj, self.tp)
            h, residual = norm_ops.norm(x, L.post_norm, cfg.rms_eps, residual=residual)
            g = gemm.linear(h, L.gate_up_proj, epilogue=gemm.EPILOGUE_SWIGLU)
            x = row_parallel(g, L.down_proj, self.tp)
        h, _ = norm_ops.norm(x, self.final_norm, cfg.rms_eps, residual=residual)
        return h
