"""Symmetric-memory staging buffers and the fused communication paths.

Each rank allocates its buffers in symmetric memory: CUDA virtual-memory allocations whose peer
mappings and NVSwitch multicast address are exchanged once at start-up, by this package's own
runtime (`symm_native.py` + csrc/symm.cpp) or, as a fallback, `torch.distributed._symmetric_memory`.  The kernels in csrc/comm.cu and csrc/gemm_tp.cu then read and write the
peers' buffers directly over NVLink; NCCL is left with bootstrap, small control messages and the
library baseline.

`FusedComm.row_linear_reduce_add_norm` is what the decoder layers call for "row-parallel GEMM ->
sum over ranks -> + residual -> RMSNorm":

  * decode-size inputs (T <= one_shot_max_tokens): the GEMM writes its partial sums into a
    symmetric buffer and ONE kernel does flag exchange + all-reduce (peer loads or
    multimem.ld_reduce) + residual add + RMSNorm; the residual stream stays replicated.
  * prefill-size inputs: ONE kernel does GEMM + reduce-scatter (peer stores from the epilogue) +
    residual add + RMSNorm on the owned rows + the send half of the all-gather; the residual
    stream is sharded by token rows between layers.  The next column-parallel GEMM
    (`gathered_linear`) waits per chunk for the rows to land and runs while later chunks arrive.
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
DEFAULT_AR_PUSH = "1"           # peers' rows are pushed before the flag exchange (FC_AR_PUSH=0: fetched after it)
DEFAULT_RUNTIME = "torch"       # "native": this package's own allocator and handle exchange (FC_SYMM overrides)
MAX_WORLD = 8


class FusedComm:
    def __init__(self, one_shot_tokens: int, hidden: int, device: torch.device, max_tokens: int = 0,
                 use_multimem: Optional[bool] = None):
        if not tpmod.is_tp_initialized():
            raise RuntimeError("tensor parallelism is not initialised")
        self.world, self.rank = tpmod.get_tp_size(), tpmod.get_tp_rank()
        if self.world > MAX_WORLD:
            raise ValueError(f"fused communication supports up to {MAX_WORLD} ranks")
        self.device, self.hidden = device, hidden
        self.one_shot_max_tokens = one_shot_tokens
        group = tpmod.get_tp_group()
        name = group.group_name
        index = device.index if device.index is not None else torch.cuda.current_device()
        bf16 = torch.bfloat16

        # ---- the symmetric buffers: one-shot all-reduce staging (two, used in alternation) and flags, the sampler's
        # candidate tables, and for prefill sizes the reduce-scatter staging, the gathered activations and their flags
        self.max_tokens = 0
        self.tp_multicast = False
        self.epoch = 0
        self._gather = None                 # (epoch, chunk_rows, T) of the rows now arriving in xg
        # form of the decode-size all-reduce (FC_AR_FORM): "push" (default: every rank stores its row into a slot of
        # every peer's buffer before the flag exchange), "pull" (rows fetched after it), "twoshot" (the owner of a
        # row sums it inside the switch and publishes it with one multicast store; needs multicast addresses)
        form = os.environ.get("FC_AR_FORM", "")
        if not form:
            form = "push" if os.environ.get("FC_AR_PUSH", DEFAULT_AR_PUSH) == "1" else "pull"
        if form not in ("push", "pull", "twoshot"):
            raise ValueError("FC_AR_FORM must be push, pull or twoshot")
        if one_shot_tokens > MAX_SLOTS and form != "pull":
            form = "pull"                  # one CTA per token row: at most MAX_SLOTS rows
        slots = {"pull": 1, "push": self.world, "twoshot": max(2, self.world)}[form]
        shapes = [((one_shot_tokens * slots, hidden), bf16), ((one_shot_tokens * slots, hidden), bf16),
                  ((MAX_SLOTS * MAX_WORLD,), torch.int32), ((ext().sample_cells_per_rank(),), torch.int64)]
        if max_tokens > one_shot_tokens:
            per_rank = -(-max_tokens // self.world)
            self.chunk_max = -(-per_rank // 128) * 128
            self.max_tokens = max_tokens
            shapes += [((self.world * self.chunk_max, hidden), bf16), ((self.chunk_max * self.world, hidden), bf16),
                       ((2 * MAX_WORLD + (self.chunk_max // 128) * MAX_WORLD,), torch.int32)]
        tensors, ptrs, mc = self._symmetric(shapes, device, group, name)
        self.bufs, self.flags, self.cells = tensors[:2], tensors[2], tensors[3]
        if use_multimem is None:
            use_multimem = os.environ.get("FC_MULTIMEM", "0") == "1"
        self.has_multicast = bool(mc[0] and mc[1])
        if form == "twoshot" and not self.has_multicast:
            form = "push"                  # no NVSwitch multicast on this set of GPUs
        self.ar_form = form
        self.push = form == "push"
        self.use_multimem = bool(use_multimem and self.has_multicast and form == "pull")
        ext().comm_init(self.rank, self.world, ptrs[0], ptrs[1], ptrs[2], mc[0], mc[1], index,
                        one_shot_tokens if form == "push" else 0, one_shot_tokens if form == "twoshot" else 0)
        ext().sample_exchange_init(ptrs[3])
        self.status = ext().status_tensor(index)
        self.cur = 0
        if self.max_tokens:
            self.stage, self.xg, self.tp_flags = tensors[4], tensors[5], tensors[6]
            # the row-parallel prefill GEMM sums through the switch when both buffers have multicast addresses
            self.tp_multicast = bool(mc[4] and mc[5])
            ext().tp_init(self.rank, self.world, ptrs[4], ptrs[5], ptrs[6], self.chunk_max,
                          self.chunk_max * self.world, hidden, index, self.chunk_max // 128,
                          int(mc[4] or 0), int(mc[5] or 0))
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _symmetric(self, shapes, device, group, group_name):
        """Zeroed symmetric buffers: (this rank's tensors, per buffer the address on every rank, per buffer the
        multicast address or 0).  This package's own runtime (CUDA virtual memory + file descriptors over Unix
        sockets, `parallel/symm_native.py`) unless FC_SYMM=torch or it cannot be brought up; then
        `torch.distributed._symmetric_memory`."""
        self.runtime = "native"
        self._segment = None
        if os.environ.get("FC_SYMM", DEFAULT_RUNTIME) != "torch":
            try:
                from . import symm_native
                seg = symm_native.rendezvous_buffers(shapes, device, group)
                self._segment = seg
                return ([b.tensor for b in seg.buffers], [list(b.buffer_ptrs) for b in seg.buffers],
                        [int(b.multicast_ptr) for b in seg.buffers])
            except RuntimeError as exc:          # raised on every rank together
                print(f"[fastcache_b200] own symmetric-memory runtime unavailable ({exc}); using torch's")
        import torch.distributed._symmetric_memory as symm_mem
        self.runtime = "torch"
        tensors, ptrs, mc = [], [], []
        for shape, dtype in shapes:
            t = symm_mem.empty(tuple(shape), dtype=dtype, device=device)
            t.zero_()
            tensors.append(t)
        torch.cuda.synchronize(device)
        self._handles = [symm_mem.rendezvous(t, group_name) for t in tensors]
        for h in self._handles:
            ptrs.append([int(p) for p in h.buffer_ptrs])
            mc.append(int(getattr(h, "multicast_ptr", 0) or 0))
        return tensors, ptrs, mc

    # ------------------------------------------------------------------ forward hooks
    def begin_forward(self) -> None:
        """Every forward pass starts on staging buffer 0 and makes an even number of one-shot calls,
        so consecutive passes (eager or replayed from a graph) keep alternating buffers."""
        self.cur = 0
        self._gather = None

    def finish_forward(self, hidden: torch.Tensor) -> torch.Tensor:
        """The last normalised activations may still be arriving: order the stream after them."""
        if self._gather is not None and hidden.data_ptr() == self.xg.data_ptr():
            ext().wait_gathered(self._gather[0], self.status)
            ops._n()
            self._gather = None
        return hidden

    def own_rows(self, buf: int, T: int) -> torch.Tensor:
        """Where this rank's partial rows [T, hidden] of staging buffer `buf` go before `allreduce_add_rmsnorm`
        (the push form keeps one slot per source rank in every buffer)."""
        first = self.rank * self.one_shot_max_tokens if self.push else 0
        return self.bufs[buf][first:first + T]

    def chunk_rows_for(self, T: int) -> int:
        return -(-(-(-T // self.world)) // 128) * 128

    # --------------------------------------------------------------------- the fused unit
    def row_linear_reduce_add_norm(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                                   residual: torch.Tensor, norm_weight: torch.Tensor, eps: float
                                   ) -> Tuple[torch.Tensor, torch.Tensor]:
        T = x.shape[0]
        if T <= self.one_shot_max_tokens:
            buf = self.cur
            self.cur ^= 1
            x2 = x if x.stride(-1) == 1 else x.contiguous()
            ops._n()
            # one kernel where the shape allows: GEMM, then the GEMM's CTAs finish their token rows into the
            # staging buffer, exchange flags with the peers, reduce, add the residual and normalise
            y = ext().linear_allreduce_add_rmsnorm(x2, weight, bias, buf, residual, norm_weight, float(eps),
                                                   self.use_multimem, self.status)
            return y, residual
        if bias is not None or T > self.max_tokens or weight.shape[0] != self.hidden:
            return self._library(x, weight, bias, residual, norm_weight, eps)
        chunk = self.chunk_rows_for(T)
        lo = min(T, self.rank * chunk)
        hi = min(T, lo + chunk)
        if residual.shape[0] == T and not getattr(residual, "_fc_shard", False):
            # first call of the pass: keep only the rows this rank owns (the residual stream is
            # sharded by token rows until the end of the pass)
            residual = residual[lo:hi].contiguous()
            residual._fc_shard = True
        self.epoch += 1
        ops._n()
        ext().gemm_rs_add_norm(x, weight, residual, norm_weight, float(eps), chunk, self.epoch, self.status, 0)
        self._gather = (self.epoch, chunk, T)
        return self.xg[:T], residual

    def gathered_linear(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                        act: str = "none") -> Optional[torch.Tensor]:
        """Column-parallel GEMM whose input is the gathered buffer that is still filling up.
        Returns None when the caller should run the plain GEMM: `x` is another tensor, or the
        projection has a bias / activation, in which case the stream is first ordered after the
        arrival of all rows."""
        g = self._gather
        if g is None or x.data_ptr() != self.xg.data_ptr():
            return None
        ops._n()
        swiglu = act == "swiglu" and weight.shape[0] % 256 == 0
        if bias is not None or (act != "none" and not swiglu) or x.shape[0] != g[2] or not x.is_contiguous():
            ext().wait_gathered(g[0], self.status)
            self._gather = None
            return None
        return ext().gemm_after_gather(x, weight, g[1], g[0], self.status, 0, swiglu)

    def sample(self, local_logits: torch.Tensor, temperatures: torch.Tensor, seed: int, vocab_offset: int,
               vocab_size: int) -> torch.Tensor:
        """[B + 1] int64: the tokens (the same on every rank) and this rank's device status code."""
        ops._n()
        return ext().sample_exchange(local_logits, temperatures, int(seed) & 0x7FFFFFFF, int(vocab_offset),
                                     int(vocab_size), self.status)

    def _library(self, x, weight, bias, residual, norm_weight, eps):
        y = ops.linear(x, weight, bias)
        tpmod.tp_all_reduce(y)
        return ops.add_rms_norm(y, residual, norm_weight, eps)

    def close(self) -> None:
        ext().comm_shutdown()
        seg, self._segment = getattr(self, "_segment", None), None
        if seg is not None:
            torch.cuda.synchronize(self.device)
            self.bufs, self.flags, self.cells = [], None, None
            self.stage = self.xg = self.tp_flags = None
            seg.close()


def enable(one_shot_tokens: int, hidden: int, device: torch.device, **kw) -> FusedComm:
    comm = FusedComm(one_shot_tokens, hidden, device, **kw)
    fused_mod.set_fused_comm(comm)
    return comm


def disable() -> None:
    comm = fused_mod.get_fused_comm()
    if comm is not None:
        comm.close()
    fused_mod.set_fused_comm(None)
