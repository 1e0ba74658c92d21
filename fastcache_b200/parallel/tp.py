"""Tensor-parallel process group plumbing.

Parity: nanovllm/utils/tp.py:32-197 — `init_tensor_parallel(tp_size, rank,
backend)`, in-place sum all-reduce, all-gather, broadcast, barrier, cleanup
and the vLLM-style size/rank aliases.  One process drives one GPU; the group
is created from the torchrun environment.  NCCL (or gloo on CPU) is used for
bootstrap, for the library baseline and for small control messages; the
per-layer reductions of the model go through the fused kernels in
`fastcache_b200.parallel.fused` when symmetric memory is available.
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional

import torch
import torch.distributed as dist

_TP_SIZE = 1
_TP_RANK = 0
_TP_GROUP: Optional[dist.ProcessGroup] = None
_OWNS_PG = False


def init_tensor_parallel(tp_size: int = 1, rank: Optional[int] = None, backend: Optional[str] = None,
                         timeout_s: float = 600.0) -> None:
    """Join the tensor-parallel group.  With tp_size == 1 this is a no-op."""
    global _TP_SIZE, _TP_RANK, _TP_GROUP, _OWNS_PG
    if tp_size <= 1:
        _TP_SIZE, _TP_RANK, _TP_GROUP = 1, 0, None
        return
    if rank is None:
        rank = int(os.environ.get("RANK", os.environ.get("LOCAL_RANK", 0)))
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda and backend == "nccl":
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if use_cuda and backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend, rank=rank, world_size=tp_size,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
        _OWNS_PG = True
    world = dist.get_world_size()
    if world != tp_size:
        raise ValueError(f"world size {world} differs from tp_size {tp_size}: this engine has no "
                         "data-parallel replicas inside one process group")
    _TP_GROUP = dist.group.WORLD
    _TP_SIZE = tp_size
    _TP_RANK = dist.get_rank()


def cleanup_tensor_parallel() -> None:
    global _TP_SIZE, _TP_RANK, _TP_GROUP, _OWNS_PG
    if _OWNS_PG and dist.is_initialized():
        dist.destroy_process_group()
    _TP_SIZE, _TP_RANK, _TP_GROUP, _OWNS_PG = 1, 0, None, False


def is_tp_initialized() -> bool:
    return _TP_SIZE > 1


def get_tp_device() -> torch.device:
    """The device this rank computes on (reference nanovllm/utils/tp.py:102-104)."""
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def get_tp_size() -> int:
    return _TP_SIZE


def get_tp_rank() -> int:
    return _TP_RANK


def get_tp_group():
    return _TP_GROUP


def tp_all_reduce(t: torch.Tensor) -> torch.Tensor:
    if _TP_SIZE > 1:
        dist.all_reduce(t, group=_TP_GROUP)
    return t


def tp_all_gather(t: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if _TP_SIZE == 1:
        return t
    parts: List[torch.Tensor] = [torch.empty_like(t) for _ in range(_TP_SIZE)]
    dist.all_gather(parts, t.contiguous(), group=_TP_GROUP)
    return torch.cat(parts, dim=dim)


def tp_broadcast(t: torch.Tensor, src: int = 0) -> torch.Tensor:
    if _TP_SIZE > 1:
        dist.broadcast(t, src=src, group=_TP_GROUP)
    return t


def tp_barrier() -> None:
    if _TP_SIZE > 1:
        dist.barrier(group=_TP_GROUP)


# vLLM-style names used by model code written against the reference
def get_tensor_model_parallel_world_size() -> int:
    return _TP_SIZE


def get_tensor_model_parallel_rank() -> int:
    return _TP_RANK
