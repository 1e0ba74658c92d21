"""Symmetric-memory staging buffers and the fused communication path.

Each rank allocates two activation staging buffers and a small flag array in
symmetric memory (`torch.distributed._symmetric_memory`: CUDA VMM allocations
whose peer mappings and NVSwitch multicast address are exchanged over the
process group once).  The kernels in csrc/comm.cu then read and write peers'
buffers directly over NVLink; NCCL is left with bootstrap, small control
messages and the library baseline.

`FusedComm.row_linear_reduce_add_norm` is what the decoder layers call for
"row-parallel GEMM -> sum over ranks -> + residual -> RMSNorm" when the tensors
are on a CUDA device and tensor parallelism is on.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops.loader import ext
from . import fused as fused_mod
from . import tp as tpmod

MAX_SLOTS = 512
MAX_WORLD = 8


class FusedComm:
    def __init__(self, max_tokens: int, hidden: int, device: torch.device, use_multimem: Optional[bool] = None,
                 one_shot_max_tokens: int = 512):
        import torch.distributed._symmetric_memory as symm_mem
        if not tpmod.is_tp_initialized():
            raise RuntimeError("tensor parallelism is not initialised")
        self.world, self.rank = tpmod.get_tp_size(), tpmod.get_tp_rank()
        if self.world > MAX_WORLD:
            raise ValueError(f"fused communication supports up to {MAX_WORLD} ranks")
        self.device = device
        self.hidden = hidden
        self.max_tokens = max_tokens
        self.one_shot_max_tokens = min(one_shot_max_tokens, max_tokens)
        group = tpmod.get_tp_group()
        name = group.group_name
        self._symm = symm_mem
        self.bufs = [symm_mem.empty((max_tokens, hidden), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.flags = symm_mem.empty((MAX_SLOTS * MAX_WORLD,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.handles = [symm_mem.rendezvous(b, name) for b in self.bufs]
        self.flag_handle = symm_mem.rendezvous(self.flags, name)
        mc = [int(getattr(h, "multicast_ptr", 0) or 0) for h in self.handles]
        if use_multimem is None:
            use_multimem = os.environ.get("FC_MULTIMEM", "0") == "1"
        self.use_multimem = bool(use_multimem and all(mc))
        index = device.index if device.index is not None else torch.cuda.current_device()
        ext().comm_init(self.rank, self.world, [int(p) for p in self.handles[0].buffer_ptrs],
                        [int(p) for p in self.handles[1].buffer_ptrs],
                        [int(p) for p in self.flag_handle.buffer_ptrs], mc[0], mc[1], index)
        self.status = ext().status_tensor(index)
        self.cur = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def begin_forward(self) -> None:
        """Every forward pass starts on staging buffer 0 and makes an even number of calls,
        so consecutive passes (eager or replayed from a graph) keep alternating buffers."""
        self.cur = 0

    def row_linear_reduce_add_norm(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                                   residual: torch.Tensor, norm_weight: torch.Tensor, eps: float
                                   ) -> Tuple[torch.Tensor, torch.Tensor]:
        T = x.shape[0]
        if T > self.one_shot_max_tokens:
            return self._large(x, weight, bias, residual, norm_weight, eps)
        buf = self.cur
        self.cur ^= 1
        staging = self.bufs[buf][:T]
        ops.linear(x, weight, bias, out=staging)           # partial sums land in symmetric memory
        ops._n()
        y = ext().allreduce_add_rmsnorm(buf, residual, norm_weight, float(eps), self.use_multimem, self.status)
        return y, residual

    def _large(self, x, weight, bias, residual, norm_weight, eps):
        # prefill-size inputs: library all-reduce until the GEMM + reduce-scatter kernel takes over
        y = ops.linear(x, weight, bias)
        tpmod.tp_all_reduce(y)
        return ops.add_rms_norm(y, residual, norm_weight, eps)

    def close(self) -> None:
        ext().comm_shutdown()


def enable(max_tokens: int, hidden: int, device: torch.device, **kw) -> FusedComm:
    comm = FusedComm(max_tokens, hidden, device, **kw)
    fused_mod.set_fused_comm(comm)
    return comm


def disable() -> None:
    comm = fused_mod.get_fused_comm()
    if comm is not None:
        comm.close()
    fused_mod.set_fused_comm(None)
