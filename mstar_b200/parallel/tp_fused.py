"""Tensor-parallel buffers and fused steps of a decoder over the symmetric heap.

Row-parallel projections (attention output, MLP down) do not all-reduce. Each rank's GEMM writes its PARTIAL result
into a slot of a symmetric region; the kernel that follows in the stream anyway — residual add + RMSNorm — reads each
row as a sum over all ranks' slots (one ``multimem.ld_reduce`` per 16 bytes when the group has an NVLS multicast
object, plain peer loads otherwise) after one flag round. Two slots are used in turn by the call sites of a forward
(site index parity); a slot is rewritten two sites later, after every rank has passed the flag round of the site in
between, so no rank can still be reading it.

The vocabulary is cut by rows over the ranks: the embedding shard lives in the heap and a token's row is loaded from
its owner over NVLink; the output head multiplies by the local shard and the [rows, vocab / W] logit shards are
multicast-stored into every rank's full logits matrix, from which every rank samples the same token (same seed and
draw counter), so no id is ever broadcast.

Reference counterparts: RowParallelLinear / ColumnParallelLinear(gather_output) / VocabParallelEmbedding
(mstar/model/components/distributed/linear.py:105,415, embedding.py:27-116), sampler broadcast
(mstar/utils/sampling.py:281).
"""
from __future__ import annotations

import torch


class TPFusedContext:
    TWO_SHOT_ROWS = 1024      # from this many rows on, the consumer norm reduces row shares and all-gathers them

    def __init__(self, symm, hidden: int, max_tokens: int, *, vocab: int = 0, max_logit_rows: int = 0):
        self.symm, self.hidden, self.max_tokens = symm, hidden, max_tokens
        self.world, self.rank = symm.world, symm.rank
        slot = max_tokens * hidden * 2
        self.vocab = vocab
        self.rows_per_rank = ((vocab + self.world - 1) // self.world + 7) // 8 * 8 if vocab else 0
        logit_bytes = 0
        if vocab and max_logit_rows:
            logit_bytes = max_logit_rows * self.rows_per_rank * 2 * (1 + self.world) + 1024
        self.region = symm.new_region(3 * slot + logit_bytes + 2048)
        self.slot_off = [self.region.alloc(slot), self.region.alloc(slot)]
        self.h_off = self.region.alloc(slot)        # gathered normalised activations of the two-shot form
        self.max_logit_rows = max_logit_rows
        if logit_bytes:
            self.logit_shard_off = self.region.alloc(max_logit_rows * self.rows_per_rank * 2)
            self.logit_full_off = self.region.alloc(max_logit_rows * self.rows_per_rank * self.world * 2)
        self.table_region = None
        self.table_off = 0

    # ---- row-parallel projections ----
    def partial_out(self, site: int, M: int, N: int | None = None) -> torch.Tensor:
        """Where the row-parallel GEMM of call site ``site`` writes its partial [M, N] (this rank's slot)."""
        N = N or self.hidden
        if M > self.max_tokens or N != self.hidden:
            raise ValueError(f"{M} x {N} does not fit the tensor-parallel slots ({self.max_tokens} x {self.hidden})")
        return self.region.view(self.slot_off[site & 1], (M, N), torch.bfloat16)

    def two_shot(self, M: int) -> bool:
        return M >= self.TWO_SHOT_ROWS

    def residual_rows(self, x: torch.Tensor) -> torch.Tensor:
        """The rows of a full [M, hidden] activation that enter the residual stream on this rank: all of them in the
        one-shot form, this rank's row share in the two-shot form."""
        if not self.two_shot(x.shape[0]):
            return x
        a, b = self.symm.row_share(x.shape[0])
        return x[a:b]

    def reduce_norm(self, site: int, M: int, gamma, eps: float, residual, bias=None):
        """(RMSNorm(sum over ranks + bias + residual), sum + bias + residual). For large M the residual is this
        rank's row share and the normalised rows are gathered from all ranks (see ``reduce_residual_norm``)."""
        return self.symm.reduce_residual_norm(self.region, self.slot_off[site & 1], M, self.hidden, gamma, eps,
                                              residual=residual, bias=bias,
                                              h_off=self.h_off if self.two_shot(M) else None)

    # ---- vocabulary-parallel embedding and head ----
    def alloc_table(self) -> torch.Tensor:
        """This rank's [rows_per_rank, hidden] shard of the embedding table, in a symmetric region of its own."""
        nbytes = self.rows_per_rank * self.hidden * 2
        self.table_region = self.symm.new_region(nbytes)
        self.table_off = self.table_region.alloc(nbytes)
        return self.table_region.view(self.table_off, (self.rows_per_rank, self.hidden), torch.bfloat16)

    def shard_rows(self, full: torch.Tensor) -> torch.Tensor:
        """Rows [rank * rows_per_rank, ...) of a [vocab, hidden] matrix, zero-padded to rows_per_rank."""
        a = self.rank * self.rows_per_rank
        part = full[a:a + self.rows_per_rank]
        if part.shape[0] < self.rows_per_rank:
            part = torch.cat([part, part.new_zeros(self.rows_per_rank - part.shape[0], full.shape[1])])
        return part

    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        return self.symm.embed_gather(self.table_region, self.table_off, self.rows_per_rank, self.hidden, ids, self.vocab)

    def logits(self, rows: torch.Tensor, head_shard: torch.Tensor) -> torch.Tensor:
        """[M, vocab] bf16 logits, the same on every rank: local GEMM against the head shard, then every rank's
        shard multicast into every rank's full matrix. The returned tensor is a view with a padded row pitch."""
        from ..ops import gemm
        M = rows.shape[0]
        if M > self.max_logit_rows:
            raise ValueError(f"{M} logit rows exceed the tensor-parallel logits buffer ({self.max_logit_rows})")
        Ns = self.rows_per_rank
        shard = self.region.view(self.logit_shard_off, (M, Ns), torch.bfloat16)
        gemm.linear(rows, head_shard, out=shard)
        self.symm.allgather_cols(self.region, self.logit_shard_off, self.logit_full_off, M, Ns)
        full = self.region.view(self.logit_full_off, (M, Ns * self.world), torch.bfloat16)
        return full[:, :self.vocab]
