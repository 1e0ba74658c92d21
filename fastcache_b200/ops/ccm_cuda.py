"""CUDA entry of the in-pool CCM merge."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .compress_cuda import _batch_meta
from .loader import ext

_TILE_ROWS = 128


def heads_per_tile(num_kv_heads: int, kv_lens: Sequence[int], image_lens: Sequence[int], factor: int,
                   min_seq_len: int, single_segment: bool) -> int:
    """How many KV heads share one 128-row tile of the fused kernel.

    The MLP weights are shared by all heads, so a tile may hold 128 / G output rows of G heads.  With G = 1 a
    segment of n rows costs ceil(n / f / 128) tiles per head, most of them nearly empty when segments are short
    (a 576-row image segment at factor 4 gives 144 output rows: one full tile and one with 16 rows).  The count of
    tiles over the whole launch is minimised; ties go to the smaller G (longer runs of rows per head)."""
    best, best_cost = 1, None
    for g in (1, 2, 4, 8):
        if num_kv_heads % g:
            continue
        rows = _TILE_ROWS // g
        cost = 0
        for n, img in zip(kv_lens, image_lens):
            img = 0 if single_segment else max(0, min(int(img), int(n)))
            for seg in (img, int(n) - img):
                out = seg // factor
                if seg > 0 and out >= min_seq_len:
                    cost += -(-out // rows)
        cost *= num_kv_heads // g
        if best_cost is None or cost < best_cost:
            best, best_cost = g, cost
    return best


def ccm_compress(pool: torch.Tensor, block_tables: List[Sequence[int]], kv_lens: Sequence[int],
                 image_lens: Sequence[int], w, layer_start: int = 0, layer_end: Optional[int] = None,
                 dst_block_tables: Optional[List[Sequence[int]]] = None) -> None:
    """`dst_block_tables`: blocks that receive the compressed rows (the source rows then stay as they are)."""
    L = pool.shape[0]
    layer_end = L if layer_end is None else min(layer_end, L)
    D = pool.shape[5]
    if D != 128 or w.w1.dtype != torch.bfloat16 or w.factor > 8:
        # shapes the tcgen05 kernel is not built for: the PyTorch statement on the device
        from ..compress.inpool import ccm_compress_reference
        for k, (bt, n, i) in enumerate(zip(block_tables, kv_lens, image_lens)):
            ccm_compress_reference(pool, bt, n, i, w, layer_start, layer_end,
                                   dst_block_table=None if dst_block_tables is None else dst_block_tables[k])
        return
    e = ext()
    dev = pool.device
    bt_d, lens_d = _batch_meta(pool, block_tables, kv_lens)
    img_d = torch.tensor(list(image_lens), dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
    status = e.status_tensor(dev.index if dev.index is not None else torch.cuda.current_device())
    g = heads_per_tile(pool.shape[3], kv_lens, image_lens, int(w.factor), int(w.min_seq_len), bool(w.single_segment))
    dst_d = None
    if dst_block_tables is not None:
        import numpy as np
        dst = np.zeros(tuple(bt_d.shape), dtype=np.int32)
        for k, t in enumerate(dst_block_tables):
            t = list(t)[: dst.shape[1]]
            dst[k, : len(t)] = t
        dst_d = torch.from_numpy(dst).pin_memory().to(dev, non_blocking=True)
    e.ccm_compress(pool, bt_d, lens_d, img_d, w.w1, w.b1, w.w2, w.b2, w.w3, w.b3, int(layer_start), int(layer_end),
                   int(layer_start), int(w.factor), int(w.min_seq_len), bool(w.single_segment), status, g, dst_d)
