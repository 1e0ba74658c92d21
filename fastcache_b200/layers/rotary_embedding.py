"""Rotary position tables (reference: nanovllm/layers/rotary_embedding.py:20-73).

The rotation itself is fused with the q/k RMSNorm and the KV-pool store in
`ops.rope_qknorm_store`; this module owns the cos|sin table.  Linear and
"llama3" frequency scaling are supported in the table (the reference asserts
`rope_scaling is None`).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ..ops import reference as ref


class RotaryEmbedding(nn.Module):
    def __init__(self, head_size: int, rotary_dim: int, max_position: int, base: float,
                 rope_scaling: Optional[dict] = None):
        super().__init__()
        if rotary_dim != head_size:
            raise ValueError("partial rotary is not supported")
        self.head_size = head_size
        inv = 1.0 / (base ** (torch.arange(0, head_size, 2, dtype=torch.float32) / head_size))
        if rope_scaling:
            kind = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
            factor = float(rope_scaling.get("factor", 1.0))
            if kind == "linear":
                inv = inv / factor
            elif kind == "llama3":
                lo = float(rope_scaling.get("low_freq_factor", 1.0))
                hi = float(rope_scaling.get("high_freq_factor", 4.0))
                orig = float(rope_scaling.get("original_max_position_embeddings", 8192))
                wavelen = 2 * math.pi / inv
                smooth = ((orig / wavelen) - lo) / (hi - lo)
                scaled = torch.where(wavelen > orig / lo, inv / factor, inv)
                mid = (wavelen <= orig / lo) & (wavelen >= orig / hi)
                inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
            elif kind not in ("default", None):
                raise ValueError(f"rope scaling {kind!r} is not supported")
        t = torch.arange(max_position, dtype=torch.float32)
        freqs = torch.outer(t, inv)
        self.register_buffer("cos_sin_cache", torch.cat([freqs.cos(), freqs.sin()], dim=-1), persistent=False)

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        """Standalone rotation of [T, H, D] tensors (used by tests and vision-free paths)."""
        cs = self.cos_sin_cache[positions.long()]
        half = self.head_size // 2
        cos, sin = cs[:, None, :half], cs[:, None, half:]
        q = ref._rotate(query.float(), cos, sin).to(query.dtype)
        k = ref._rotate(key.float(), cos, sin).to(key.dtype)
        return q, k


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half (neox) rotation of `x [..., D]` by `cos`, `sin` `[..., D / 2]`, computed in fp32
    (nanovllm/layers/rotary_embedding.py:7-17)."""
    return ref._rotate(x.float(), cos.float(), sin.float()).to(x.dtype)


_ROPE_CACHE: dict = {}


def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float,
             rope_scaling: Optional[dict] = None) -> RotaryEmbedding:
    key = (head_size, rotary_dim, max_position, float(base),
           tuple(sorted(rope_scaling.items())) if rope_scaling else None, str(torch.get_default_device()))
    if key not in _ROPE_CACHE:
        _ROPE_CACHE[key] = RotaryEmbedding(head_size, rotary_dim, max_position, base, rope_scaling)
    return _ROPE_CACHE[key]
