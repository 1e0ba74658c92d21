"""Step metadata shared by the layers of one forward pass.

Parity: nanovllm/utils/context.py:6-28 (a process-global record of
prefill/decode metadata).  Fields here describe the paged layout directly:
`kv_lens` is the number of rows each request has in the pool after this step's
store, for prefill and decode alike.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch


@dataclass
class Context:
    is_prefill: bool = False
    cu_seqlens_q: Optional[torch.Tensor] = None
    cu_seqlens_k: Optional[torch.Tensor] = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: Optional[torch.Tensor] = None
    context_lens: Optional[torch.Tensor] = None     # kv rows per request (decode and prefill)
    block_tables: Optional[torch.Tensor] = None
    # rows of the flattened batch whose hidden state feeds the LM head
    logits_indices: Optional[torch.Tensor] = None
    # SnapKV: when set, attention layers stash the last `window` rotated queries
    # of every request here, keyed by layer index
    window_q: Any = None
    obs_window: int = 0
    attn_workspace: Any = None
    tp: Any = None


_CONTEXT = Context()


def get_context() -> Context:
    return _CONTEXT


def set_context(is_prefill: bool, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=0, max_seqlen_k=0,
                slot_mapping=None, context_lens=None, block_tables=None, logits_indices=None,
                window_q=None, obs_window=0, attn_workspace=None, tp=None) -> Context:
    global _CONTEXT
    _CONTEXT = Context(is_prefill, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                       slot_mapping, context_lens, block_tables, logits_indices, window_q,
                       obs_window, attn_workspace, tp)
    return _CONTEXT


def reset_context() -> None:
    global _CONTEXT
    _CONTEXT = Context()
