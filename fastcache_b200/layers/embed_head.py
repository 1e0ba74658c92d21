"""Vocabulary-parallel embedding and LM head.

Parity: "kv-cache pipeline"/nanovllm/layers/embed_head.py:10-74.  The
vocabulary is padded to a multiple of 64 x tp so any vocabulary size shards
(the reference asserts divisibility), rows outside a rank's shard contribute
zeros that the sum over ranks fills in, and the LM head gathers the shards'
logits on every rank (the reference leaves the gather commented out and
samples from rank 0's shard only).
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..parallel import tp as tpmod
from ..utils.context import get_context


def padded_vocab(vocab: int, tp: int, multiple: int = 64) -> int:
    m = multiple * tp
    return -(-vocab // m) * m


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        self.tp_size = tpmod.get_tp_size()
        self.tp_rank = tpmod.get_tp_rank()
        self.num_embeddings = num_embeddings
        self.padded = padded_vocab(num_embeddings, self.tp_size) if self.tp_size > 1 else num_embeddings
        self.per_rank = self.padded // self.tp_size
        self.vocab_start = self.per_rank * self.tp_rank
        self.vocab_end = self.vocab_start + self.per_rank
        self.weight = nn.Parameter(torch.zeros(self.per_rank, embedding_dim), requires_grad=False)
        self.weight.weight_loader = self.weight_loader

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        if loaded.shape[0] == param.data.shape[0] and self.tp_size == 1:
            param.data.copy_(loaded)
            return
        lo = self.vocab_start
        hi = min(self.vocab_end, loaded.shape[0])
        param.data.zero_()
        if hi > lo:
            param.data[: hi - lo].copy_(loaded[lo:hi])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
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
            logits = tpmod.tp_all_gather(logits, dim=-1)
        return logits[:, : self.num_embeddings]
