"""Row-parallel GEMM + sum over ranks + residual add + RMSNorm as one call.

The decoder layers never see a bare all-reduce: the pattern "row-parallel
projection, reduce, add the residual, normalise for the next projection"
occurs twice per layer ("kv-cache pipeline"/nanovllm/layers/linear.py:216-220
followed by nanovllm/layers/layernorm.py:29-41 in the reference) and is
routed here.  Depending on where the data lives this becomes

  * tp == 1:           GEMM kernel, then the add+RMSNorm kernel
  * tp > 1 on CUDA:    the fused kernels of `fastcache_b200.parallel.symm`
                       (one-shot all-reduce+add+norm for decode-size inputs,
                       GEMM + reduce-scatter + add + norm for prefill sizes)
  * tp > 1 elsewhere:  GEMM, library all-reduce, add+RMSNorm (CPU/gloo tests
                       and the library baseline)
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from . import tp as tpmod

_FUSED_COMM = None      # set by parallel.symm.enable() on CUDA ranks


def set_fused_comm(comm) -> None:
    global _FUSED_COMM
    _FUSED_COMM = comm


def get_fused_comm():
    return _FUSED_COMM


def row_linear_reduce_add_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                               residual: torch.Tensor, norm_weight: torch.Tensor, eps: float
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (rms_norm(residual + sum_ranks(x @ weight.T)), new residual)."""
    tp = tpmod.get_tp_size()
    if tp > 1 and tpmod.get_tp_rank() != 0:
        bias = None
    if tp > 1 and x.is_cuda and _FUSED_COMM is not None:
        return _FUSED_COMM.row_linear_reduce_add_norm(x, weight, bias, residual, norm_weight, eps)
    if tp == 1 and x.is_cuda:
        return ops.linear_add_rms_norm(x, weight, bias, residual, norm_weight, eps)
    y = ops.linear(x, weight, bias)
    if tp > 1:
        tpmod.tp_all_reduce(y)
    return ops.add_rms_norm(y, residual, norm_weight, eps)
