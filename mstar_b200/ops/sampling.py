"""Sampling: temperature / top-k / top-p / repetition penalty / per-request seeds, graph-capturable.

GPU: ``sample_kernel`` in csrc/sampling.cu (one launch per step, no host sync). CPU path and oracle:
``sample_ref``. Per-request parameters live in slot-indexed device buffers (``SamplerState``) so that a captured
decode graph only needs the row->slot map rewritten between replays.

Reference counterparts: ``SamplingConfig`` / ``MultiSamplingConfig`` (mstar/utils/sampling.py:208-265), the Triton
prep kernel + FlashInfer sampling (mstar/utils/sampling.py:32-161,518-686), ``CudaGraphableSampler`` with
slot-indexed master buffers (mstar/utils/sampling.py:689-1283), seeds from md5(request_id)
(mstar/conductor/conductor.py:53-65). Under tensor parallelism every rank draws the same token from the same
(seed, offset), which removes the reference's broadcast from rank 0 (mstar/utils/sampling.py:269-287).
"""
from __future__ import annotations

import ctypes
import hashlib
from dataclasses import dataclass, field

import torch

from . import _lib


@dataclass
class SamplingConfig:
    vocab_size: int = 0
    temperature: float = 0.6
    top_k: int = 0
    top_p: float = 1.0
    ignore_eos: bool = False
    repetition_penalty: float = 1.0
    _seed: int | None = None

    def seed(self) -> int:
        return 0 if self._seed is None else int(self._seed)


@dataclass
class MultiSamplingConfig:
    """A main sampler plus named auxiliary samplers (e.g. a talker's code-predictor heads)."""
    main: SamplingConfig = field(default_factory=SamplingConfig)
    aux: dict[str, SamplingConfig] = field(default_factory=dict)


def request_id_to_seed(request_id: str) -> int:
    """Deterministic 63-bit seed from the request id, so that a pinned request id pins the random stream."""
    return int.from_bytes(hashlib.md5(request_id.encode()).digest()[:8], "little") & ((1 << 63) - 1)


_M32 = 0xFFFFFFFF


def philox_uniform(seed: int, offset: int) -> float:
    """The kernel's draw: Philox4x32-10 with counter (offset, 0) and key seed; first word -> (0,1)."""
    c = [offset & _M32, (offset >> 32) & _M32, 0, 0]
    k = [seed & _M32, (seed >> 32) & _M32]
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _M32, p1 & _M32, ((p0 >> 32) ^ c[3] ^ k[1]) & _M32, p0 & _M32]
        k = [(k[0] + 0x9E3779B9) & _M32, (k[1] + 0xBB67AE85) & _M32]
    return ((c[0] >> 8) + 0.5) / 16777216.0


def kept_set_ref(logits_row, temperature, top_k, top_p, seen_row=None, rep_penalty=1.0):
    """(probabilities over the vocabulary, boolean kept mask) with the exact smallest nucleus."""
    x = logits_row.float().clone()
    if seen_row is not None and rep_penalty != 1.0:
        s = seen_row.bool()
        x = torch.where(s, torch.where(x > 0, x / rep_penalty, x * rep_penalty), x)
    x = x / temperature
    p = torch.softmax(x, dim=-1)
    V = p.numel()
    keep = torch.ones(V, dtype=torch.bool, device=p.device)
    if (top_k and 0 < top_k < V) or top_p < 1.0:
        sp, si = torch.sort(p, descending=True, stable=True)
        cs = torch.cumsum(sp, 0)
        n_p = int((cs < top_p).sum().item()) + 1 if top_p < 1.0 else V
        n = min(n_p, top_k if (top_k and top_k > 0) else V, V)
        thr = sp[n - 1]
        keep = p >= thr
    return p, keep


def sample_ref(logits, temperature, top_k, top_p, rep_penalty, seeds, offsets, seen=None, u=None):
    """Row-wise oracle. All per-row parameters are python lists. Returns LongTensor [B] and updates ``seen``."""
    B = logits.shape[0]
    out = torch.zeros(B, dtype=torch.int64, device=logits.device)
    for b in range(B):
        srow = seen[b] if seen is not None else None
        if temperature[b] <= 0:
            x = logits[b].float().clone()
            if srow is not None and rep_penalty[b] != 1.0:
                s = srow.bool()
                x = torch.where(s, torch.where(x > 0, x / rep_penalty[b], x * rep_penalty[b]), x)
            tok = int(torch.argmax(x).item())
        else:
            p, keep = kept_set_ref(logits[b], temperature[b], top_k[b], top_p[b], srow, rep_penalty[b])
            pk = torch.where(keep, p, torch.zeros_like(p)).double()
            cdf = torch.cumsum(pk, 0)
            draw = u[b] if u is not None else philox_uniform(int(seeds[b]), int(offsets[b]))
            target = draw * cdf[-1].item()
            tok = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype, device=cdf.device), right=True).item())
            tok = min(tok, p.numel() - 1)
            if not keep[tok]:
                nz = torch.nonzero(keep).flatten()
                tok = int(nz[nz <= tok][-1].item()) if (nz <= tok).any() else int(nz[0].item())
        out[b] = tok
        if seen is not None:
            seen[b, tok] = 1
    return out


class SamplerState:
    """Slot-indexed sampling parameters on the device. A request owns one slot for its lifetime."""

    def __init__(self, num_slots: int, vocab_size: int, device, track_seen: bool = False,
                 reserve_pad_slot: bool = False):
        """``reserve_pad_slot`` keeps the last slot out of the free list (``pad_slot``): the padding rows of a
        bucketed batch sample with it (greedy, no penalty), so that they never touch a live request's seen-token
        mask or draw counter."""
        self.num_slots, self.vocab_size, self.device = num_slots, vocab_size, torch.device(device)
        d = self.device
        self.temperature = torch.zeros(num_slots, dtype=torch.float32, device=d)
        self.top_k = torch.zeros(num_slots, dtype=torch.int32, device=d)
        self.top_p = torch.ones(num_slots, dtype=torch.float32, device=d)
        self.rep_penalty = torch.ones(num_slots, dtype=torch.float32, device=d)
        self.seed = torch.zeros(num_slots, dtype=torch.int64, device=d)
        self.offset = torch.zeros(num_slots, dtype=torch.int64, device=d)
        self.seen = torch.zeros((num_slots, vocab_size), dtype=torch.uint8, device=d) if track_seen else None
        # scratch of the kernel: exp(logit - max) per element, written once and read by the later passes
        self._es = (torch.empty((num_slots, vocab_size), dtype=torch.float32, device=d)
                    if torch.device(d).type == "cuda" and vocab_size >= 16384 else None)
        self.pad_slot = num_slots - 1 if reserve_pad_slot else None
        self._free = list(range(num_slots - (2 if reserve_pad_slot else 1), -1, -1))
        self._slot_of: dict[str, int] = {}

    def _escratch(self, rows: int, vocab: int, device):
        if self._es is None or vocab != self._es.shape[1]:
            return None
        if rows > self._es.shape[0]:
            self._es = torch.empty((rows, vocab), dtype=torch.float32, device=device)
        return self._es

    def assign(self, request_id: str, cfg: SamplingConfig, seed: int | None = None,
               prompt_ids: torch.Tensor | None = None, slot: int | None = None) -> int:
        """Bind a request to a slot (a specific one when ``slot`` is given) and load its parameters."""
        if request_id in self._slot_of:
            return self._slot_of[request_id]
        if not self._free:
            raise RuntimeError("sampler: no free slot")
        if slot is not None:
            if slot not in self._free:
                raise RuntimeError(f"sampler: slot {slot} is taken")
            self._free.remove(slot)
            s = slot
        else:
            s = self._free.pop()
        self._slot_of[request_id] = s
        self.temperature[s] = float(cfg.temperature)
        self.top_k[s] = int(cfg.top_k)
        self.top_p[s] = float(cfg.top_p)
        self.rep_penalty[s] = float(cfg.repetition_penalty)
        sd = cfg._seed if cfg._seed is not None else (seed if seed is not None else request_id_to_seed(request_id))
        self.seed[s] = int(sd) & ((1 << 63) - 1)
        self.offset[s] = 0
        if self.seen is not None:
            self.seen[s].zero_()
            if prompt_ids is not None and cfg.repetition_penalty != 1.0:
                self.seen[s, prompt_ids.to(self.device).long().clamp(0, self.vocab_size - 1)] = 1
        return s

    def slot(self, request_id: str) -> int:
        return self._slot_of[request_id]

    def release(self, request_id: str) -> None:
        s = self._slot_of.pop(request_id, None)
        if s is not None:
            self._free.append(s)

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor | None = None,
               advance: bool = True, u: torch.Tensor | None = None) -> torch.Tensor:
        """logits [B, V] (bf16 or fp32), row_slot int32 [B] -> int64 [B]; bumps each used slot's draw counter."""
        B, V = logits.shape
        assert V == self.vocab_size
        if out is None:
            out = torch.empty(B, dtype=torch.int64, device=logits.device)
        if not logits.is_cuda:
            rs = row_slot.tolist()
            seen_rows = self.seen[rs] if self.seen is not None else None
            res = sample_ref(logits, self.temperature[rs].tolist(), self.top_k[rs].tolist(), self.top_p[rs].tolist(),
                             self.rep_penalty[rs].tolist(), self.seed[rs].tolist(), self.offset[rs].tolist(),
                             seen_rows, None if u is None else u.tolist())
            if self.seen is not None:
                self.seen[rs] = seen_rows
            out.copy_(res)
        else:
            assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
            assert row_slot.dtype == torch.int32
            rc = _lib.kernels().mstar_sample(
                ctypes.c_void_p(logits.data_ptr()), ctypes.c_longlong(logits.stride(0)),
                1 if logits.dtype == torch.float32 else 0, int(B), int(V),
                ctypes.c_void_p(self.temperature.data_ptr()), ctypes.c_void_p(self.top_k.data_ptr()),
                ctypes.c_void_p(self.top_p.data_ptr()), ctypes.c_void_p(self.rep_penalty.data_ptr()),
                ctypes.c_void_p(self.seed.data_ptr()), ctypes.c_void_p(self.offset.data_ptr()),
                ctypes.c_void_p(_lib.ptr(self.seen)), ctypes.c_void_p(row_slot.data_ptr()),
                ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(0), ctypes.c_void_p(_lib.ptr(u)),
                ctypes.c_void_p(_lib.ptr(self._escratch(B, V, logits.device))), ctypes.c_void_p(_lib.stream_ptr()))
            _lib.check(rc, "mstar_sample")
        if advance:
            self.offset.index_add_(0, row_slot.long(), torch.ones(B, dtype=torch.int64, device=self.offset.device))
        return out
