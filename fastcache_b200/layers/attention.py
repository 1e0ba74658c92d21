"""Paged attention layer.

Parity: nanovllm/layers/attention.py:42-79 — store the new K/V rows in the
paged pool by slot, then causal varlen attention for prefill and paged
single-row attention for decode.  Here the q/k RMSNorm (Qwen3), the rotary
embedding and the pool store are one fused op, and prefill attention always
reads K/V through the block table, which covers prefix-cache hits without a
second code path.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..utils.context import get_context


class Attention(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, scale: float, num_kv_heads: int, layer_idx: int = 0):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.layer_idx = layer_idx
        # bound by the model runner to this layer's slice of the pool:
        # [num_blocks, num_kv_heads, block_size, head_dim]
        self.k_cache: Optional[torch.Tensor] = None
        self.v_cache: Optional[torch.Tensor] = None

    def forward(self, qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
                eps: float = 1e-6, fused_qkv=None) -> torch.Tensor:
        """`fused_qkv = (x, qkv_weight)` instead of `qkv`: the projection runs here, fused with the
        rope / norm / store kernel."""
        ctx = get_context()
        if self.k_cache is None:
            raise RuntimeError("attention layer used before the KV pool was bound")
        if fused_qkv is not None:
            q = ops.linear_rope_qknorm_store(fused_qkv[0], fused_qkv[1], positions, cos_sin, self.num_heads,
                                             self.num_kv_heads, self.head_dim, q_norm_weight, k_norm_weight, eps,
                                             self.k_cache, self.v_cache, ctx.slot_mapping)
        else:
            q = ops.rope_qknorm_store(qkv, positions, cos_sin, self.num_heads, self.num_kv_heads, self.head_dim,
                                      q_norm_weight, k_norm_weight, eps, self.k_cache, self.v_cache,
                                      ctx.slot_mapping)
        if ctx.is_prefill:
            if ctx.window_q is not None:
                ctx.window_q["q"][self.layer_idx] = q.index_select(0, ctx.window_q["indices"])
            o = ops.prefill_attention(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.cu_seqlens_q,
                                      ctx.context_lens, self.scale, ctx.max_seqlen_q)
        else:
            o = ops.decode_attention(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.context_lens,
                                     self.scale, ctx.attn_workspace)
        return o.reshape(-1, self.num_heads * self.head_dim)


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """Scatter new K / V rows `[T, Hkv, D]` into the paged pool `[blocks, Hkv, block, D]` by slot
    (slot = block * block_size + offset; negative slots are skipped).

    The reference launches a Triton kernel for this (nanovllm/layers/attention.py:10-39).  The
    engine here never stores on its own: the rows are written by the fused rope / q-k-norm / store
    kernel.  This function is the stand-alone form for callers that fill a pool themselves (tests,
    cache import); it is index arithmetic plus two indexed copies on whatever device the pool is on."""
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    bs = k_cache.shape[2]
    blk, off = slots // bs, slots % bs
    k_cache[blk, :, off] = key[valid].to(k_cache.dtype)
    v_cache[blk, :, off] = value[valid].to(v_cache.dtype)
