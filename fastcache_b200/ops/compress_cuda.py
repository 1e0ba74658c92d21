"""CUDA side of in-pool compression: eviction (score -> top-k -> compaction) and CCM merge."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .loader import ext


def _batch_meta(pool: torch.Tensor, block_tables: List[Sequence[int]], kv_lens: Sequence[int]):
    bs = pool.shape[4]
    need = [-(-n // bs) for n in kv_lens]
    width = max(1, max(need))
    bt = np.zeros((len(kv_lens), width), dtype=np.int32)
    for i, (t, n) in enumerate(zip(block_tables, need)):
        bt[i, :n] = np.asarray(t[:n], dtype=np.int32)
    dev = pool.device
    bt_d = torch.from_numpy(bt).pin_memory().to(dev, non_blocking=True)
    lens_d = torch.tensor(list(kv_lens), dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
    return bt_d, lens_d


def _torch_scores(pool, block_tables, kv_lens, method, window_q, params, stride) -> torch.Tensor:
    """Scores for the methods without a dedicated kernel: the PyTorch statement, on the device."""
    from ..compress.inpool import _rows
    from ..compress.scorers import NEEDS_QUERIES, score_keys
    L, _, _, H, _, D = pool.shape
    out = torch.full((len(kv_lens), L, H, stride), float("-inf"), dtype=torch.float32, device=pool.device)
    for i, (bt, n) in enumerate(zip(block_tables, kv_lens)):
        blocks = torch.as_tensor(list(bt), dtype=torch.long, device=pool.device)
        for layer in range(L):
            k = _rows(pool[layer, 0], blocks, n).permute(1, 0, 2)
            v = _rows(pool[layer, 1], blocks, n).permute(1, 0, 2)
            q = None
            if method in NEEDS_QUERIES:
                wq = window_q[i] if window_q is not None else None
                if wq is None or layer not in wq:
                    raise ValueError(f"{method} needs the observation-window queries of layer {layer}")
                q = wq[layer].permute(1, 0, 2)
            out[i, layer, :, :n] = score_keys(method, k, v, q, **params)
    return out


def evict_cuda(pool: torch.Tensor, block_tables: List[Sequence[int]], kv_lens: Sequence[int], method: str,
               n_kepts: Sequence[int], window_q: Optional[List[Optional[Dict[int, torch.Tensor]]]],
               params: dict) -> List[int]:
    e = ext()
    dev = pool.device
    bt_d, lens_d = _batch_meta(pool, block_tables, kv_lens)
    kept = [max(1, min(int(k), int(n))) for k, n in zip(n_kepts, kv_lens)]
    kept_d = torch.tensor(kept, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
    status = e.status_tensor(dev.index if dev.index is not None else torch.cuda.current_device())
    max_len = int(max(kv_lens))
    scores = None
    if method in ("knorm", "knorm_ref"):
        scores = e.knorm_scores(pool, bt_d, lens_d, max_len, 1 if method == "knorm_ref" else 0, status)
    elif method == "snapkv" and window_q is not None and all(wq is not None for wq in window_q) \
            and min(kv_lens) > int(params.get("window", 64)):
        from .snapkv import snapkv_scores_cuda
        scores = snapkv_scores_cuda(pool, bt_d, lens_d, max_len, window_q, params, status)
    elif method == "expected_attention" and window_q is not None and all(wq is not None for wq in window_q):
        from .snapkv import stack_window_queries
        qw = stack_window_queries(window_q, pool.shape[0])
        if qw is not None and pool.shape[5] in (64, 128):
            scores = e.expected_attention_scores(pool, bt_d, lens_d, max_len, qw, int(params.get("n_sink", 4)), status)
    elif method == "streaming_llm":
        scores = e.position_scores(pool, lens_d, max_len, int(params.get("n_sink", 4)))
    if scores is None:
        stride = (max_len + 3) // 4 * 4
        p = dict(params)
        if method == "uniform":
            p.pop("n_kept", None)
            scores = torch.full((len(kv_lens), pool.shape[0], pool.shape[3], stride), float("-inf"),
                                dtype=torch.float32, device=dev)
            from ..compress.scorers import uniform
            for i, (n, k) in enumerate(zip(kv_lens, kept)):
                dummy = torch.empty(pool.shape[3], n, 1, device=dev)
                scores[i, :, :, :n] = uniform(dummy, n_kept=k)[None]
        else:
            scores = _torch_scores(pool, block_tables, kv_lens, method, window_q, p, stride)
    e.select_compact(pool, scores, bt_d, lens_d, kept_d, status)
    return kept


def ccm_compress_cuda(pool, block_tables, kv_lens, image_lens, w, layer_start=0, layer_end=None,
                      dst_block_tables=None) -> None:
    from .ccm_cuda import ccm_compress
    ccm_compress(pool, block_tables, kv_lens, image_lens, w, layer_start, layer_end, dst_block_tables)
