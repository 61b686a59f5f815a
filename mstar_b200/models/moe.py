"""Sparse MoE block (Qwen3-MoE style router: softmax over all experts, top-k, optional renormalisation, optional
shared expert) on the grouped tcgen05 GEMM. Parallel modes: TP-MoE (every rank holds a slice of every expert's
intermediate dim, partial sums reduced like a row-parallel layer — the reference's only mode,
mstar/model/components/moe.py:378-591) and EP (every rank holds E / P whole experts; tokens are dispatched to the
owner and combined back over the symmetric heap).
"""
from __future__ import annotations

import torch
from torch import nn

from ..ops import gemm, moe as moe_ops
from ..parallel.comm import CommGroup


def _param(shape, dtype, device):
    return nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg, tp: CommGroup, device, ep: CommGroup | None = None):
        super().__init__()
        # ``replicated``: the expert-parallel group is the tensor-parallel group itself; every rank holds the same
        # tokens (attention output was all-reduced), runs only its own experts on them and the results are summed
        # by one all-reduce. No dispatch traffic; the expert weights are cut by expert instead of by column.
        self.replicated = False
        if ep is None and getattr(cfg, "moe_expert_parallel", False) and tp.size > 1:
            ep, self.replicated = tp, True
        self.cfg, self.tp, self.ep = cfg, tp, ep
        H, E, I = cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size
        self.E, self.top_k = E, cfg.num_experts_per_tok
        self.router = _param((E, H), cfg.dtype, device)
        if ep is not None and ep.size > 1:
            assert E % ep.size == 0
            self.E_local, self.I_local = E // ep.size, I
            self.expert_range = (ep.rank * self.E_local, (ep.rank + 1) * self.E_local)
        else:
            assert I % tp.size == 0
            self.E_local, self.I_local = E, I // tp.size
            self.expert_range = (0, E)
        self.w13 = _param((self.E_local, 2 * self.I_local, H), cfg.dtype, device)
        self.w2 = _param((self.E_local, H, self.I_local), cfg.dtype, device)
        self.shared = None
        if cfg.shared_expert_intermediate_size:
            from .decoder import GatedMLP
            self.shared = GatedMLP(H, cfg.shared_expert_intermediate_size, tp, cfg.dtype, device)
            self.shared_gate = _param((1, H), cfg.dtype, device)

    @torch.no_grad()
    def init_random(self, g: torch.Generator, std: float) -> None:
        cfg = self.cfg
        H, E, I = cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size

        def draw(shape):
            return torch.randn(shape, generator=g, dtype=torch.float32) * std
        self.router.copy_(draw((E, H)).to(cfg.dtype))
        e0, e1 = self.expert_range
        r, n = (self.tp.rank, self.tp.size) if self.ep is None or self.ep.size == 1 else (0, 1)
        Il = I // n
        for e in range(E):
            gate, up, down = draw((I, H)), draw((I, H)), draw((H, I))
            if e0 <= e < e1:
                gs, us = gate[r * Il:(r + 1) * Il], up[r * Il:(r + 1) * Il]
                self.w13[e - e0].copy_(gemm.interleave_gate_up(gs, us).to(cfg.dtype))
                self.w2[e - e0].copy_(down[:, r * Il:(r + 1) * Il].to(cfg.dtype))
        if self.shared is not None:
            from .decoder import load_gated_mlp
            F_ = cfg.shared_expert_intermediate_size
            load_gated_mlp(self.shared, draw((F_, H)), draw((F_, H)), draw((H, F_)), self.tp.rank, self.tp.size, cfg.dtype)
            self.shared_gate.copy_(draw((1, H)).to(cfg.dtype))

    @torch.no_grad()
    def quantize_fp8(self) -> "SparseMoeBlock":
        """Re-store the expert weights as block-scaled e4m3 (128 x 128 scales); the expert GEMMs then quantise
        their activations per 1 x 128 block and run the fp8 grouped kernel. Router and shared expert stay bf16.
        Needs expert widths that are multiples of 128 (the scale block); other shapes are left as they are."""
        from ..ops import gemm_fp8
        if isinstance(self.w13, gemm_fp8.Fp8Weight) or (2 * self.I_local) % 128 or self.cfg.hidden_size % 128:
            return self
        w13, w2 = gemm_fp8.quantize_weight(self.w13.data), gemm_fp8.quantize_weight(self.w2.data)
        del self.w13, self.w2
        self.w13, self.w2 = w13, w2
        return self

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = gemm.linear(h, self.router, out_dtype=torch.float32)
        add = None
        if self.shared is not None:
            s = self.shared(h, reduce=False)
            gate = torch.sigmoid(gemm.linear(h, self.shared_gate, out_dtype=torch.float32))
            add = (s.float() * gate).to(h.dtype)
        if self.replicated:
            from .decoder import tp_reduce
            y = moe_ops.fused_moe(h, logits, self.w13, self.w2, self.top_k, self.cfg.norm_topk_prob,
                                  self.expert_range, add=add)
            return tp_reduce(y.contiguous(), self.tp)
        fp8 = not isinstance(self.w13, torch.Tensor)
        if self.ep is not None and self.ep.size > 1 and getattr(self.ep, "symm", None) is not None and h.is_cuda \
                and not fp8:
            from ..parallel.expert_parallel import ep_moe
            return ep_moe(self, h, logits, add)
        y = moe_ops.fused_moe(h, logits, self.w13, self.w2, self.top_k, self.cfg.norm_topk_prob,
                              self.expert_range, add=add)
        if self.ep is not None and self.ep.size > 1:
            return self.ep.all_reduce(y)           # NCCL baseline for expert parallelism: local experts, then sum
        if self.tp.size > 1:
            from .decoder import tp_reduce
            return tp_reduce(y.contiguous(), self.tp)
        return y
