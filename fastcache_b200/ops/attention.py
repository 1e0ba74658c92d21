"""CUDA attention wrappers."""
from __future__ import annotations


from .loader import ext


def decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale, workspace=None):
    """`workspace` may carry {"splits": n, "max_ctx": n} chosen by the runner so the
    launch shape is fixed under CUDA-graph capture."""
    splits = 0
    max_ctx = 0
    if isinstance(workspace, dict):
        splits = int(workspace.get("splits", 0))
        max_ctx = int(workspace.get("max_ctx", 0))
    return ext().decode_attention(q, k_cache, v_cache, block_tables, context_lens, float(scale), splits, max_ctx)
