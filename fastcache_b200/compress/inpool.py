"""Compression that operates directly on the paged KV pool.

The reference extracts a request's KV from the pool into HuggingFace-format
tensors with per-layer, per-block Python loops, runs the compressor and copies
the result back block by block ("kv-cache pipeline"/nanovllm/engine/
llava_model_runner.py:908-996).  Here both merge compression (CCM) and
eviction read rows through the block table and write the shorter result into
the *leading rows of the same blocks*, so the tail blocks can be freed; no
intermediate per-request tensors exist on the GPU path.

Pool layout: `[L, 2, num_blocks, Hkv, block_size, D]` (index 1: 0 = K, 1 = V); inside a block
the rows of one head are contiguous.

In-place safety: every output row index is <= the index of each input row it
depends on.  The CUDA kernels give each (request, head, layer, K|V) to one
thread block that walks the rows in ascending order and reads a tile
completely before writing it, so no row is overwritten before it is read.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .ccm import PackedCCMWeights, ccm_segment_len
from .scorers import NEEDS_QUERIES, score_keys, select_keep


def _rows(pool_lkv: torch.Tensor, block_ids: torch.Tensor, n: int) -> torch.Tensor:
    """[n, Hkv, D] rows of one (layer, K|V) slice of the pool."""
    nb = -(-n // pool_lkv.shape[2])
    return pool_lkv[block_ids[:nb]].permute(0, 2, 1, 3).reshape(-1, pool_lkv.shape[1], pool_lkv.shape[3])[:n]


def _write_rows(pool_lkv: torch.Tensor, block_ids: torch.Tensor, rows: torch.Tensor) -> None:
    n = rows.shape[0]
    bs = pool_lkv.shape[2]
    r = torch.arange(n, device=rows.device)
    pool_lkv[block_ids[r // bs], :, r % bs] = rows.to(pool_lkv.dtype)


# ----------------------------------------------------------------- CCM merge
def _ccm_segment(x: torch.Tensor, w: PackedCCMWeights, layer: int, bank: int) -> torch.Tensor:
    """x [S, H, D] -> [S_c, H, D]"""
    S, H, D = x.shape
    f = w.factor
    s = S // f
    if S == 0 or s < w.min_seq_len:
        return x
    z = x[: s * f].reshape(s, f, H, D).permute(0, 2, 1, 3).reshape(s, H, f * D)
    y = w.mlp(z, layer, bank).to(x.dtype)
    return torch.cat([y, x[s * f:]], dim=0) if S > s * f else y


def ccm_compress_reference(kv_pool: torch.Tensor, block_table: Sequence[int], kv_len: int, image_len: int,
                           w: PackedCCMWeights, layer_start: int = 0, layer_end: Optional[int] = None,
                           weight_layer_offset: int = 0, dst_block_table: Optional[Sequence[int]] = None) -> int:
    """PyTorch statement of the fused kernel for one request.  Returns the new row count.  With
    `dst_block_table` the result goes to those blocks and the request's own rows stay as they are."""
    L = kv_pool.shape[0]
    layer_end = L if layer_end is None else layer_end
    blocks = torch.as_tensor(block_table, dtype=torch.long, device=kv_pool.device)
    out_blocks = blocks if dst_block_table is None else \
        torch.as_tensor(dst_block_table, dtype=torch.long, device=kv_pool.device)
    if w.single_segment:
        image_len = 0
    image_len = max(0, min(image_len, kv_len))
    new_len = kv_len
    for layer in range(layer_start, layer_end):
        wl = layer - weight_layer_offset
        for kv in (0, 1):
            rows = _rows(kv_pool[layer, kv], blocks, kv_len).clone()
            img = _ccm_segment(rows[:image_len], w, wl, 2 + kv)
            txt = _ccm_segment(rows[image_len:], w, wl, kv)
            out = torch.cat([img, txt], dim=0)
            new_len = out.shape[0]
            _write_rows(kv_pool[layer, kv], out_blocks, out)
    return new_len


def ccm_compress_in_pool(kv_pool: torch.Tensor, block_tables: List[Sequence[int]], kv_lens: Sequence[int],
                         image_lens: Sequence[int], w: PackedCCMWeights, layer_start: int = 0,
                         layer_end: Optional[int] = None,
                         dst_block_tables: Optional[List[Sequence[int]]] = None) -> List[int]:
    """Compress a batch of requests in place (or, with `dst_block_tables`, into a second set of blocks per
    request, leaving the source rows untouched).  Returns the new row count per request."""
    if w.single_segment:
        image_lens = [0] * len(kv_lens)
    new_lens = [ccm_segment_len(min(i, n), w.factor, w.min_seq_len) +
                ccm_segment_len(n - min(i, n), w.factor, w.min_seq_len)
                for n, i in zip(kv_lens, image_lens)]
    if kv_pool.is_cuda:
        from ..ops.compress_cuda import ccm_compress_cuda
        ccm_compress_cuda(kv_pool, block_tables, kv_lens, image_lens, w, layer_start, layer_end, dst_block_tables)
        return new_lens
    for k, (bt, n, i) in enumerate(zip(block_tables, kv_lens, image_lens)):
        ccm_compress_reference(kv_pool, bt, n, i, w, layer_start, layer_end,
                               dst_block_table=None if dst_block_tables is None else dst_block_tables[k])
    return new_lens


# ------------------------------------------------------------------- eviction
def evict_reference(kv_pool: torch.Tensor, block_table: Sequence[int], kv_len: int, method: str,
                    n_kept: int, window_q: Optional[Dict[int, torch.Tensor]] = None,
                    params: Optional[dict] = None) -> int:
    """Score -> per-head top-k -> compaction into the leading rows, every layer.

    window_q: {layer: [w, Hq, D]} rotated trailing queries of this request.
    """
    params = params or {}
    blocks = torch.as_tensor(block_table, dtype=torch.long, device=kv_pool.device)
    n_kept = max(1, min(n_kept, kv_len))
    for layer in range(kv_pool.shape[0]):
        k = _rows(kv_pool[layer, 0], blocks, kv_len).clone()           # [S, H, D]
        v = _rows(kv_pool[layer, 1], blocks, kv_len).clone()
        q = None
        if method in NEEDS_QUERIES:
            if window_q is None or layer not in window_q:
                raise ValueError(f"{method} needs the observation-window queries of layer {layer}")
            q = window_q[layer].permute(1, 0, 2)
        scores = score_keys(method, k.permute(1, 0, 2), v.permute(1, 0, 2), q, n_kept=n_kept, **params)
        idx = select_keep(scores, n_kept)                              # [H, n_kept]
        gather = idx.t()[:, :, None].expand(-1, -1, k.shape[-1])       # [n_kept, H, D]
        _write_rows(kv_pool[layer, 0], blocks, torch.gather(k, 0, gather))
        _write_rows(kv_pool[layer, 1], blocks, torch.gather(v, 0, gather))
    return n_kept


def _window_slice(wq: Optional[Dict[int, torch.Tensor]], first: int, last: int) -> Optional[Dict[int, torch.Tensor]]:
    """Observation-window queries of layers [first, last), keyed from 0 like the pool slice they go with."""
    if wq is None:
        return None
    return {l - first: q for l, q in wq.items() if first <= l < last}


def evict_in_pool(kv_pool: torch.Tensor, block_tables: List[Sequence[int]], kv_lens: Sequence[int],
                  method: str, n_kepts: Sequence[int], window_q: Optional[List[Optional[Dict[int, torch.Tensor]]]] = None,
                  params: Optional[dict] = None, layer_start: int = 0, layer_end: Optional[int] = None) -> List[int]:
    """Evict in place in layers [layer_start, layer_end) only (all layers by default).  `kv_lens` are the row
    counts before eviction; a caller that works through the layers in chunks passes the same original counts
    for every chunk, because the other layers' rows are untouched by a chunk."""
    L = kv_pool.shape[0]
    layer_end = L if layer_end is None else min(layer_end, L)
    if layer_start > 0 or layer_end < L:
        # the layer index is the outermost dimension of the pool, so a range of layers is a contiguous pool
        kv_pool = kv_pool[layer_start:layer_end]
        if window_q is not None:
            window_q = [_window_slice(wq, layer_start, layer_end) for wq in window_q]
    if kv_pool.is_cuda:
        from ..ops.compress_cuda import evict_cuda
        return evict_cuda(kv_pool, block_tables, kv_lens, method, n_kepts, window_q, params or {})
    out = []
    for i, (bt, n, nk) in enumerate(zip(block_tables, kv_lens, n_kepts)):
        wq = window_q[i] if window_q is not None else None
        out.append(evict_reference(kv_pool, bt, n, method, nk, wq, params))
    return out
