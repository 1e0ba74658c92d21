"""Megatron-style sharded linear layers.

Parity: "kv-cache pipeline"/nanovllm/layers/linear.py:34-220 — Replicated,
Column, MergedColumn (gate|up packed), QKV (q|k|v packed, heads split over
ranks) and Row-parallel (input dim split, bias on rank 0, sum over ranks).
Loaders take full HuggingFace tensors and cut the local shard; a tensor that
already has the local shape is copied as is.

Differences by design:
  * KV heads are replicated when there are fewer of them than ranks (the
    reference requires divisibility), so a 4-KV-head model runs at TP=8.
  * `RowParallelLinear.forward` returns the *partial* product when
    `reduce_results=False`; the decoder layers use that and hand the reduction
    to the fused reduce + residual + RMSNorm kernels.
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..parallel import tp as tpmod


def divide(a: int, b: int) -> int:
    if a % b:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


class LinearBase(nn.Module):
    def __init__(self, in_local: int, out_local: int, bias: bool):
        super().__init__()
        self.tp_size = tpmod.get_tp_size()
        self.tp_rank = tpmod.get_tp_rank()
        self.weight = nn.Parameter(torch.empty(out_local, in_local), requires_grad=False)
        self.weight.weight_loader = self.weight_loader
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_local), requires_grad=False)
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        raise NotImplementedError

    def forward(self, x: torch.Tensor, act: str = "none") -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, act)


def _copy(dst: torch.Tensor, src: torch.Tensor) -> None:
    if dst.shape != src.shape:
        raise ValueError(f"shape mismatch: parameter {tuple(dst.shape)} vs checkpoint {tuple(src.shape)}")
    dst.copy_(src)


class ReplicatedLinear(LinearBase):
    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        super().__init__(input_size, output_size, bias)

    def weight_loader(self, param, loaded, shard_id=None):
        _copy(param.data, loaded)


class ColumnParallelLinear(LinearBase):
    """Output features split over ranks."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        tp = tpmod.get_tp_size()
        self.output_size = output_size
        super().__init__(input_size, divide(output_size, tp), bias)

    def weight_loader(self, param, loaded, shard_id=None):
        local = param.data.shape[0]
        if loaded.shape[0] != local:
            loaded = loaded.narrow(0, self.tp_rank * local, local)
        _copy(param.data, loaded)


class MergedColumnParallelLinear(LinearBase):
    """Several column-parallel projections of the same input in one weight."""

    def __init__(self, input_size: int, output_sizes: List[int], bias: bool = False):
        tp = tpmod.get_tp_size()
        self.output_sizes = list(output_sizes)
        self.local_sizes = [divide(s, tp) for s in output_sizes]
        super().__init__(input_size, sum(self.local_sizes), bias)

    def weight_loader(self, param, loaded, shard_id=None):
        if shard_id is None:
            _copy(param.data, loaded)
            return
        idx = int(shard_id)
        off = sum(self.local_sizes[:idx])
        size = self.local_sizes[idx]
        if loaded.shape[0] != size:
            loaded = loaded.narrow(0, self.tp_rank * size, size)
        _copy(param.data.narrow(0, off, size), loaded)


class QKVParallelLinear(LinearBase):
    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: Optional[int] = None, bias: bool = False):
        tp = tpmod.get_tp_size()
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.head_size = head_size
        self.total_num_heads = total_num_heads
        self.total_num_kv_heads = total_num_kv_heads
        self.num_heads = divide(total_num_heads, tp)
        if total_num_kv_heads >= tp:
            self.num_kv_heads = divide(total_num_kv_heads, tp)
            self.kv_replicas = 1
        else:
            self.num_kv_heads = 1
            self.kv_replicas = divide(tp, total_num_kv_heads)
        out = (self.num_heads + 2 * self.num_kv_heads) * head_size
        super().__init__(hidden_size, out, bias)

    def weight_loader(self, param, loaded, shard_id=None):
        if shard_id is None:
            _copy(param.data, loaded)
            return
        q_sz = self.num_heads * self.head_size
        kv_sz = self.num_kv_heads * self.head_size
        if shard_id == "q":
            off, size, src = 0, q_sz, self.tp_rank * q_sz
        else:
            off = q_sz + (kv_sz if shard_id == "v" else 0)
            size = kv_sz
            src = (self.tp_rank // self.kv_replicas) * kv_sz
        if loaded.shape[0] != size:
            loaded = loaded.narrow(0, src, size)
        _copy(param.data.narrow(0, off, size), loaded)


class RowParallelLinear(LinearBase):
    """Input features split over ranks; the products are summed over ranks."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, reduce_results: bool = True):
        tp = tpmod.get_tp_size()
        self.reduce_results = reduce_results
        super().__init__(divide(input_size, tp), output_size, bias)

    def weight_loader(self, param, loaded, shard_id=None):
        if param.data.dim() == 1:                    # bias: whole vector, applied on rank 0 only
            _copy(param.data, loaded)
            return
        local = param.data.shape[1]
        if loaded.shape[1] != local:
            loaded = loaded.narrow(1, self.tp_rank * local, local)
        _copy(param.data, loaded)

    def forward(self, x: torch.Tensor, act: str = "none") -> torch.Tensor:
        bias = self.bias if self.tp_rank == 0 else None
        y = ops.linear(x, self.weight, bias, act)
        if self.reduce_results and self.tp_size > 1:
            tpmod.tp_all_reduce(y)
        return y
