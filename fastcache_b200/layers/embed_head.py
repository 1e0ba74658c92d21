"""Vocabulary-parallel embedding and LM head.

Parity: "kv-cache pipeline"/nanovllm/layers/embed_head.py:10-74.  The
vocabulary is padded to a multiple of 64 x tp so any vocabulary size shards
(the reference asserts divisibility), rows outside a rank's shard contribute
zeros that the sum over ranks fills in, and the LM head gathers the shards'
logits on every rank (the reference leaves the gather commented out and
samples from rank 0's shard only).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel import tp as tpmod
from ..utils.context import get_context


def padded_vocab(vocab: int, tp: int, multiple: int = 64) -> int:
    m = multiple * tp
    return -(-vocab // m) * m


# Above this many bytes an embedding table is sharded over the ranks; below it every rank keeps the whole table
# and the lookup needs no collective.  (151936 x 4096 bf16 = 1.2 GB on a 180 GB part.)
REPLICATE_EMBEDDING_BYTES = 8 << 30

_LOCAL_LOGITS = False


def set_local_logits(on: bool) -> bool:
    """While on, `ParallelLMHead` returns this rank's vocabulary shard [B, V / tp] (padding columns included)
    instead of gathering; the sampler then works on the shards (`Sampler.forward_sharded`).  Returns the
    previous setting."""
    global _LOCAL_LOGITS
    prev, _LOCAL_LOGITS = _LOCAL_LOGITS, bool(on)
    return prev


class VocabParallelEmbedding(nn.Module):
    """Token embedding under tensor parallelism.

    `replicate=None` decides by size: a table of at most REPLICATE_EMBEDDING_BYTES is kept whole on every rank,
    which removes the all-reduce the sharded lookup needs (the reference always shards and all-reduces,
    "kv-cache pipeline"/nanovllm/layers/embed_head.py:38-46).  The LM head is always sharded."""

    def __init__(self, num_embeddings: int, embedding_dim: int, replicate: Optional[bool] = None):
        super().__init__()
        self.tp_size = tpmod.get_tp_size()
        self.tp_rank = tpmod.get_tp_rank()
        self.num_embeddings = num_embeddings
        self.padded = padded_vocab(num_embeddings, self.tp_size) if self.tp_size > 1 else num_embeddings
        self.per_rank = self.padded // self.tp_size
        self.vocab_start = self.per_rank * self.tp_rank
        self.vocab_end = self.vocab_start + self.per_rank
        if replicate is None:
            replicate = self.padded * embedding_dim * 2 <= REPLICATE_EMBEDDING_BYTES
        self.replicated = bool(replicate) and self.tp_size > 1 and not isinstance(self, ParallelLMHead)
        rows = self.padded if self.replicated else self.per_rank
        self.weight = nn.Parameter(torch.zeros(rows, embedding_dim), requires_grad=False)
        self.weight.weight_loader = self.weight_loader

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        if loaded.shape[0] == param.data.shape[0] and (self.tp_size == 1 or self.replicated):
            param.data.copy_(loaded)
            return
        lo, hi = (0, self.padded) if self.replicated else (self.vocab_start, self.vocab_end)
        hi = min(hi, loaded.shape[0])
        param.data.zero_()
        if hi > lo:
            param.data[: hi - lo].copy_(loaded[lo:hi])

    def shard_rows(self) -> torch.Tensor:
        """This rank's vocabulary shard of the table (what a tied LM head multiplies with)."""
        return self.weight[self.vocab_start:self.vocab_end] if self.replicated else self.weight

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.replicated:
            return ops.embedding(ids, self.weight, 0)
        y = ops.embedding(ids, self.weight, self.vocab_start)
        if self.tp_size > 1:
            tpmod.tp_all_reduce(y)
        return y


class ParallelLMHead(VocabParallelEmbedding):
    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        ctx = get_context()
        if ctx.logits_indices is not None:
            hidden = hidden.index_select(0, ctx.logits_indices)
        elif ctx.is_prefill and ctx.cu_seqlens_q is not None:
            hidden = hidden.index_select(0, (ctx.cu_seqlens_q[1:] - 1).long())
        logits = ops.linear(hidden.contiguous(), self.weight)
        if self.tp_size > 1:
            if _LOCAL_LOGITS:
                return logits
            logits = tpmod.tp_all_gather(logits, dim=-1)
        return logits[:, : self.num_embeddings]
