"""CUDA entry of the in-pool CCM merge."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .compress_cuda import _batch_meta
from .loader import ext


def ccm_compress(pool: torch.Tensor, block_tables: List[Sequence[int]], kv_lens: Sequence[int],
                 image_lens: Sequence[int], w, layer_start: int = 0, layer_end: Optional[int] = None) -> None:
    L = pool.shape[0]
    layer_end = L if layer_end is None else min(layer_end, L)
    D = pool.shape[5]
    if D != 128 or w.w1.dtype != torch.bfloat16 or w.factor > 8:
        # shapes the tcgen05 kernel is not built for: the PyTorch statement on the device
        from ..compress.inpool import ccm_compress_reference
        for bt, n, i in zip(block_tables, kv_lens, image_lens):
            ccm_compress_reference(pool, bt, n, i, w, layer_start, layer_end)
        return
    e = ext()
    dev = pool.device
    bt_d, lens_d = _batch_meta(pool, block_tables, kv_lens)
    img_d = torch.tensor(list(image_lens), dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
    status = e.status_tensor(dev.index if dev.index is not None else torch.cuda.current_device())
    e.ccm_compress(pool, bt_d, lens_d, img_d, w.w1, w.b1, w.w2, w.b2, w.w3, w.b3, int(layer_start), int(layer_end),
                   int(layer_start), int(w.factor), int(w.min_seq_len), bool(w.single_segment), status)
