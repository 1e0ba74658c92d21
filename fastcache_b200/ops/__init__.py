"""Op entry points.

Each function runs the hand-written sm_100a kernel when its tensors live on a
CUDA device and the PyTorch statement in `reference.py` otherwise.  There is
no backend registry: the device of the data decides, and a CUDA tensor without
the compiled extension is an error, never a silent fallback.

`COUNTERS["launches"]` counts kernels of this package launched from Python
(the model runner adds the kernels inside CUDA graphs per replay).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import reference as ref
from .loader import ext, ext_available  # noqa: F401

COUNTERS = {"launches": 0}


def _n(k: int = 1) -> None:
    COUNTERS["launches"] += k


def rms_norm(x, weight, eps):
    if x.is_cuda:
        _n()
        return ext().rms_norm(x, weight, float(eps))
    return ref.rms_norm(x, weight, eps)


def add_rms_norm(x, residual, weight, eps) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (normed, new_residual).  On CUDA `residual` is updated in place."""
    if x.is_cuda:
        _n()
        y = ext().add_rms_norm(x, residual, weight, float(eps))
        return y, residual
    return ref.add_rms_norm(x, residual, weight, eps)


def layer_norm(x, weight, bias, eps):
    if x.is_cuda:
        _n()
        return ext().layer_norm(x.contiguous(), weight, bias, float(eps))
    return ref.layer_norm(x, weight, bias, eps)


def silu_and_mul(x):
    if x.is_cuda:
        _n()
        return ext().silu_and_mul(x)
    return ref.silu_and_mul(x)


def linear(x, weight, bias=None, act: str = "none", out: Optional[torch.Tensor] = None):
    """y = act(x @ weight.T + bias).  weight is [N, K] as in nn.Linear."""
    if x.is_cuda:
        from ..parallel.fused import get_fused_comm
        comm = get_fused_comm()
        if comm is not None and getattr(comm, "_gather", None) is not None and out is None:
            # x may be the gathered activation buffer that is still filling up over NVLink
            y = comm.gathered_linear(x, weight, bias, act)
            if y is not None:
                return y
        from .gemm import gemm
        _n(2 if act == "swiglu" else 1)
        return gemm(x, weight, bias, act, out)
    y = ref.linear(x, weight, bias, act)
    if out is not None:
        out.copy_(y)
        return out
    return y


def linear_add_rms_norm(x, weight, bias, residual, norm_weight, eps) -> Tuple[torch.Tensor, torch.Tensor]:
    """residual += x @ weight.T (+ bias); returns (RMSNorm(residual), residual).  On CUDA the split-K
    partial sums of a decode-size GEMM are reduced inside the norm kernel (two launches in all)."""
    if x.is_cuda:
        _n(2)
        y = ext().linear_add_rms_norm(x, weight, bias, residual, norm_weight, float(eps))
        return y, residual
    return ref.add_rms_norm(ref.linear(x, weight, bias), residual, norm_weight, eps)


def linear_silu_mul(x, weight):
    """silu(x @ Wg.T) * (x @ Wu.T) for weight = [Wg; Wu]."""
    if x.is_cuda:
        _n(2)
        return ext().linear_silu_mul(x, weight)
    return ref.silu_and_mul(ref.linear(x, weight))


def rope_qknorm_store(qkv, positions, cos_sin, num_q_heads, num_kv_heads, head_dim,
                      q_norm_weight, k_norm_weight, eps, k_cache, v_cache, slot_mapping):
    if qkv.is_cuda:
        _n()
        return ext().rope_qknorm_store(qkv, positions, cos_sin, num_q_heads, num_kv_heads, head_dim,
                                       q_norm_weight, k_norm_weight, float(eps), k_cache, v_cache,
                                       slot_mapping)
    return ref.rope_qknorm_store(qkv, positions, cos_sin, num_q_heads, num_kv_heads, head_dim,
                                 q_norm_weight, k_norm_weight, eps, k_cache, v_cache, slot_mapping)


def linear_rope_qknorm_store(x, weight, positions, cos_sin, num_q_heads, num_kv_heads, head_dim,
                             q_norm_weight, k_norm_weight, eps, k_cache, v_cache, slot_mapping):
    """`rope_qknorm_store(x @ weight.T, ...)`.  On CUDA with head_dim 128 the rope kernel also reduces the
    split-K partial sums of a decode-size GEMM (two launches in all)."""
    if x.is_cuda and head_dim == 128 and slot_mapping is not None:
        _n(2)
        return ext().linear_rope_qknorm_store(x, weight, positions, cos_sin, num_q_heads, num_kv_heads, head_dim,
                                              q_norm_weight, k_norm_weight, float(eps), k_cache, v_cache,
                                              slot_mapping)
    return rope_qknorm_store(linear(x, weight), positions, cos_sin, num_q_heads, num_kv_heads, head_dim,
                             q_norm_weight, k_norm_weight, eps, k_cache, v_cache, slot_mapping)


def prefill_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, scale,
                      max_q_len: int = 0, impl: int = 0):
    """Causal attention of new tokens over the paged cache.  `impl`: 0 picks the kernel (the two-tile
    tcgen05 kernel for head_dim 128 and more than 64 query rows), 1 forces the mma.sync kernel, 2 the
    one-tile tcgen05 kernel, 3 the two-tile tcgen05 kernel."""
    if q.is_cuda:
        _n()
        return ext().prefill_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens,
                                       float(scale), int(max_q_len), int(impl))
    return ref.prefill_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, kv_lens, scale)


def decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale, workspace=None):
    if q.is_cuda:
        from .attention import decode_attention as _dec
        _n()
        return _dec(q, k_cache, v_cache, block_tables, context_lens, scale, workspace)
    return ref.decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale)


def dense_attention(q, k, v, scale, key_mask=None, impl: int = 0):
    """impl (CUDA only): 0 = tcgen05 kernel where the strides allow it, 1 = the mma.sync kernel, 2 = tcgen05 or raise."""
    if q.is_cuda:
        _n()
        return ext().dense_attention(q, k, v, float(scale), key_mask, int(impl))
    return ref.dense_attention(q, k, v, scale, key_mask)


def embedding(ids, weight, vocab_start: int = 0):
    if weight.is_cuda:
        _n()
        return ext().embedding(ids, weight, int(vocab_start))
    return ref.embedding(ids, weight, vocab_start)


def sample(logits, temperatures, noise=None, seed: int = 0, with_status: bool = False, vocab_offset: int = 0,
           v_limit: int = -1):
    """Tokens [B].  `with_status` (CUDA): [B + 1], the last entry is the device status code (0 = clean), so the
    host learns about a kernel wait that ran out with the tokens it reads back anyway."""
    if logits.is_cuda and noise is None:
        _n()
        return ext().sample(logits, temperatures, int(seed) & 0x7FFFFFFF, bool(with_status), int(vocab_offset),
                            int(v_limit))
    if noise is None:
        # drawn from the step's seed, not from the process-wide generator: tensor-parallel ranks on the CPU then
        # make the same draw from their (identical) gathered logits
        g = torch.Generator(device=logits.device).manual_seed(int(seed) & 0x7FFFFFFF)
        noise = torch.empty(logits.shape, dtype=torch.float32, device=logits.device).exponential_(1, generator=g)
    out = ref.sample(logits, temperatures, noise)
    if with_status:
        out = torch.cat([out, out.new_zeros(1)])
    return out
