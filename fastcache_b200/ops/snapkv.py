"""Scoring kernels that read the observation-window queries (csrc/snapkv.cu, csrc/scores.cu)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .loader import ext


def stack_window_queries(window_q: List[Optional[Dict[int, torch.Tensor]]], L: int) -> Optional[torch.Tensor]:
    """[n_seq, L, w, Hq, D] from the per-request {layer: [w, Hq, D]} dicts; None when the requests carry
    different window lengths or miss a layer (the caller then uses the PyTorch statement)."""
    if any(wq is None or len(wq) < L for wq in window_q):
        return None
    w = window_q[0][0].shape[0]
    for wq in window_q:
        if any(wq[l].shape[0] != w for l in range(L)):
            return None
    if w < 2:
        return None
    return torch.stack([torch.stack([wq[l] for l in range(L)]) for wq in window_q]).contiguous()


def snapkv_scores_cuda(pool: torch.Tensor, bt_d: torch.Tensor, lens_d: torch.Tensor, max_len: int,
                       window_q: List[Optional[Dict[int, torch.Tensor]]], params: dict,
                       status: torch.Tensor) -> Optional[torch.Tensor]:
    """Scores [n_seq, L, Hkv, stride] for `select_compact`, or None when the shapes are outside what the
    kernel takes (the caller then scores with the PyTorch statement): every request must carry the same
    window length w (a multiple of 16, shorter than the request), with (Hq / Hkv) * w <= 256."""
    L, Hkv, D = pool.shape[0], pool.shape[3], pool.shape[5]
    window = int(params.get("window", 64))
    kernel_size = int(params.get("kernel_size", 5))
    if D not in (64, 128) or kernel_size % 2 == 0:
        return None
    qw = stack_window_queries(window_q, L)
    if qw is None:
        return None
    w, Hq = qw.shape[2], qw.shape[3]
    if w % 16 != 0 or w > window or Hq % Hkv != 0 or (Hq // Hkv) * w > 256:
        return None
    return ext().snapkv_scores(pool, bt_d, lens_d, int(max_len), qw, kernel_size, float(D) ** -0.5, status)
