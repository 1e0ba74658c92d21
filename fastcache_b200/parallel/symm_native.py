"""Symmetric buffers from this package's own runtime (csrc/symm.cpp).

`rendezvous_buffers(shapes, dtype, device, group)` gives every rank of the tensor-parallel group the same list of
buffers, each with the addresses of all ranks' copies (peer pointers, usable from kernels with plain loads and
stores over NVLink) and, where the system has NVSwitch multicast, one multicast address per buffer for
multimem.* instructions.  The allocation is one CUDA virtual-memory allocation per rank that holds all the
buffers; it is exported as a POSIX file descriptor, and the descriptors travel between the ranks' processes over
Unix-domain sockets (`socket.send_fds`), the socket paths and sizes over the torch.distributed group.  The
reference has no counterpart (its collectives are NCCL calls, nanovllm/utils/tp.py:112-186).

`FusedComm` uses these buffers by default and falls back to `torch.distributed._symmetric_memory` when the
runtime cannot be brought up (old driver, no peer access), or when FC_SYMM=torch.
"""
from __future__ import annotations

import os
import socket
import tempfile
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops.loader import ext


@dataclass
class SymmBuffer:
    tensor: torch.Tensor                      # this rank's copy
    buffer_ptrs: List[int]                    # address of every rank's copy, by rank
    multicast_ptr: int = 0                    # 0: no multicast on this system


@dataclass
class SymmSegment:
    """One allocation per rank with all buffers inside; keeps the mappings alive."""
    size: int
    local_va: int
    peer_vas: List[int]
    mc_handle: int = 0
    mc_va: int = 0
    buffers: List[SymmBuffer] = field(default_factory=list)
    _keep: list = field(default_factory=list)

    def close(self) -> None:
        e = ext()
        self.buffers.clear()
        self._keep.clear()
        if self.mc_va:
            e.symm_free(self.mc_va)
        if self.mc_handle:
            e.multicast_release(self.mc_handle)
        for va in set(self.peer_vas):
            e.symm_free(va)
        self.peer_vas, self.mc_va, self.mc_handle = [], 0, 0


def _tensor_at(address: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device, owner) -> torch.Tensor:
    """A tensor over memory this package mapped itself (`owner` keeps the mapping alive)."""
    numel = 1
    for s in shape:
        numel *= int(s)
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Span:
        # the CUDA array interface is how a foreign allocation becomes a tensor without a copy
        __cuda_array_interface__ = {"shape": (numel * itemsize,), "typestr": "|u1", "data": (int(address), False),
                                    "version": 3, "strides": None}

    span = _Span()
    span.owner = owner
    flat = torch.as_tensor(span, device=device)
    return flat.view(dtype).view(*shape)


_SOCKET_TIMEOUT_S = 60.0


def _exchange_fds(my_fd: int, rank: int, world: int, group) -> List[int]:
    """Every rank receives every rank's descriptor (its own is returned as given).  Each rank listens on a
    Unix socket, sends its descriptor to every peer (a connect succeeds as soon as the peer listens, the message
    fits the socket buffer) and then accepts world - 1 connections; the first byte of a message names its sender.
    All socket calls have a time limit, so a peer that never shows up is an error, not a hang."""
    tmp = tempfile.mkdtemp(prefix=f"fc_symm_{os.getpid()}_")
    path = os.path.join(tmp, "fd.sock")
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.settimeout(_SOCKET_TIMEOUT_S)
    srv.bind(path)
    srv.listen(world)
    paths: List[Optional[str]] = [None] * world
    dist.all_gather_object(paths, path, group=group)
    fds = [-1] * world
    fds[rank] = my_fd
    try:
        for r in range(1, world):
            out = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            out.settimeout(_SOCKET_TIMEOUT_S)
            out.connect(paths[(rank + r) % world])
            socket.send_fds(out, [bytes([rank])], [my_fd])
            out.close()
        for _ in range(world - 1):
            conn, _ = srv.accept()
            conn.settimeout(_SOCKET_TIMEOUT_S)
            msg, got, _, _ = socket.recv_fds(conn, 16, 1)
            conn.close()
            if not msg or not got:
                raise RuntimeError("a peer closed its socket without sending a descriptor")
            fds[msg[0]] = got[0]
    finally:
        srv.close()
        try:
            os.unlink(path)
            os.rmdir(tmp)
        except OSError:
            pass
    return fds


def rendezvous_buffers(shapes: Sequence[Tuple[Sequence[int], torch.dtype]], device: torch.device, group,
                       want_multicast: bool = True) -> SymmSegment:
    """Collective over `group`: allocate, exchange, map.  `shapes`: (shape, dtype) per buffer, the same on every
    rank.  Raises RuntimeError when the runtime cannot be brought up on some rank (every rank then raises)."""
    e = ext()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    index = device.index if device.index is not None else torch.cuda.current_device()
    err: Optional[str] = None
    seg: Optional[SymmSegment] = None
    fds: List[int] = []
    try:
        gran = int(e.symm_granularity(index, world))
        offsets, total = [], 0
        for shape, dtype in shapes:
            n = torch.empty((), dtype=dtype).element_size()
            for s in shape:
                n *= int(s)
            offsets.append(total)
            total += -(-n // 256) * 256
        size = -(-max(total, 1) // gran) * gran
        local_va, fd = e.symm_alloc(size, index)
        fds.append(fd)
    except Exception as exc:                                  # noqa: BLE001 - reported to every rank below
        err = f"rank {rank}: {type(exc).__name__}: {exc}"
    errs: List[Optional[str]] = [None] * world
    dist.all_gather_object(errs, err, group=group)
    if any(errs):
        raise RuntimeError("symmetric-memory runtime unavailable: " + "; ".join(x for x in errs if x))
    peer_vas: List[int] = []
    try:
        all_fds = _exchange_fds(fd, rank, world, group)
        peer_vas = [local_va if r == rank else int(e.symm_import(all_fds[r], size, index)) for r in range(world)]
        for r, f in enumerate(all_fds):
            if r != rank:
                e.symm_close_fd(f)
    except Exception as exc:                                  # noqa: BLE001 - reported to every rank below
        err = f"rank {rank}: {type(exc).__name__}: {exc}"
    dist.all_gather_object(errs, err, group=group)
    if any(errs):
        for va in set(peer_vas) | {int(local_va)}:
            e.symm_free(va)
        e.symm_close_fd(fd)
        raise RuntimeError("symmetric-memory runtime unavailable: " + "; ".join(x for x in errs if x))
    seg = SymmSegment(size=size, local_va=int(local_va), peer_vas=peer_vas)
    # ---- multicast (NVLS): rank 0 creates the object, every rank adds its device, then binds its memory.  After
    # every step the ranks agree on whether all of them succeeded, so that none waits at a barrier for a rank that
    # gave up; without multicast the peer pointers still work and multimem is simply off.
    def all_ok(problem: Optional[str]) -> bool:
        got: List[Optional[str]] = [None] * world
        dist.all_gather_object(got, problem, group=group)
        return not any(got)

    if all_ok(None if (want_multicast and e.multicast_supported(index)) else "no multicast"):
        mc_handle, mc_fd, problem = 0, -1, None
        try:
            if rank == 0:
                mc_handle, mc_fd = e.multicast_create(size, world)
        except Exception as exc:                              # noqa: BLE001
            problem = str(exc)
        if all_ok(problem):
            got_fd = _exchange_fds_from_root(mc_fd, rank, world, group)
            try:
                if got_fd < 0:
                    raise RuntimeError("the multicast descriptor did not arrive")
                if rank != 0:
                    mc_handle = int(e.multicast_import(got_fd))
                e.multicast_add_device(mc_handle, index)
            except Exception as exc:                          # noqa: BLE001
                problem = str(exc)
            e.symm_close_fd(got_fd)
            if all_ok(problem):                               # every device is added: memory may be bound now
                try:
                    seg.mc_va = int(e.multicast_bind(mc_handle, seg.local_va, size, index))
                    seg.mc_handle = int(mc_handle)
                except Exception as exc:                      # noqa: BLE001
                    problem = str(exc)
                if not all_ok(problem):
                    seg.mc_va = 0
    e.symm_close_fd(fd)
    for (shape, dtype), off in zip(shapes, offsets):
        t = _tensor_at(seg.local_va + off, shape, dtype, device, seg)
        seg.buffers.append(SymmBuffer(t, [va + off for va in peer_vas], seg.mc_va + off if seg.mc_va else 0))
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    return seg


def _exchange_fds_from_root(fd: int, rank: int, world: int, group) -> int:
    """Rank 0's descriptor to every other rank; returns the received descriptor (rank 0: its own), -1 when the
    exchange failed on this rank (the caller's next agreement step tells the others)."""
    tmp = tempfile.mkdtemp(prefix=f"fc_symm_mc_{os.getpid()}_")
    path = os.path.join(tmp, "fd.sock")
    srv = None
    if rank != 0:
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.settimeout(_SOCKET_TIMEOUT_S)
        srv.bind(path)
        srv.listen(1)
    paths: List[Optional[str]] = [None] * world
    dist.all_gather_object(paths, path, group=group)
    got = fd
    try:
        if rank == 0:
            for r in range(1, world):
                out = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                out.settimeout(_SOCKET_TIMEOUT_S)
                out.connect(paths[r])
                socket.send_fds(out, [b"m"], [fd])
                out.close()
        else:
            conn, _ = srv.accept()
            conn.settimeout(_SOCKET_TIMEOUT_S)
            _, fds, _, _ = socket.recv_fds(conn, 16, 1)
            conn.close()
            got = fds[0] if fds else -1
    except OSError:
        got = -1
    finally:
        if srv is not None:
            srv.close()
            try:
                os.unlink(path)
            except OSError:
                pass
        try:
            os.rmdir(tmp)
        except OSError:
            pass
    return got
