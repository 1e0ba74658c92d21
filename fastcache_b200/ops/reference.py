"""Plain PyTorch statements of every op in this package.

These run on any device and are the numerical oracle for the sm_100a kernels
(tests compare each kernel against the fp32 result of the function of the same
name here) and the execution path on CPU.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ norms
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps)).to(x.dtype) * weight


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                 eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """residual' = x + residual (rounded to x.dtype); y = rms_norm(residual')."""
    s = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(s, weight, eps), s


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


# ------------------------------------------------------------- activations
def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    gate, up = x.chunk(2, dim=-1)
    return (F.silu(gate.float()) * up.float()).to(x.dtype)


def gelu(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    return F.gelu(x.float(), approximate=approximate).to(x.dtype)


def quick_gelu(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.sigmoid(1.702 * xf)).to(x.dtype)


# ------------------------------------------------------------------- GEMM
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: str = "none") -> torch.Tensor:
    y = F.linear(x, weight, bias)
    if act == "relu":
        y = F.relu(y)
    elif act == "gelu":
        y = gelu(y)
    elif act == "gelu_tanh":
        y = gelu(y, "tanh")
    elif act == "quick_gelu":
        y = quick_gelu(y)
    elif act == "swiglu":
        y = silu_and_mul(y)
    elif act != "none":
        raise ValueError(act)
    return y


# ------------------------------------------------------------------- rope
def build_cos_sin_cache(head_dim: int, max_pos: int, base: float,
                        device=None) -> torch.Tensor:
    """[max_pos, head_dim] fp32: first half cos, second half sin (neox layout)."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv)
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1)


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x [T, H, D] fp32, cos/sin [T, 1, D/2]
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def rope_qknorm_store(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                      num_q_heads: int, num_kv_heads: int, head_dim: int,
                      q_norm_weight: Optional[torch.Tensor], k_norm_weight: Optional[torch.Tensor],
                      eps: float, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                      slot_mapping: Optional[torch.Tensor]) -> torch.Tensor:
    """Per-head q/k RMSNorm (optional) -> neox rotary -> scatter K,V rows into
    the paged pool.  Returns rotated q [T, Hq, D].

    qkv: [T, (Hq + 2 Hkv) * D] packed q | k | v
    k_cache / v_cache: [num_blocks, Hkv, block_size, D] (head-major inside a block, so the
    rows of one head are contiguous); slot = block * block_size + offset, negative slots
    are skipped.
    """
    T = qkv.shape[0]
    qd, kd = num_q_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :qd].reshape(T, num_q_heads, head_dim)
    k = qkv[:, qd:qd + kd].reshape(T, num_kv_heads, head_dim)
    v = qkv[:, qd + kd:].reshape(T, num_kv_heads, head_dim)
    if q_norm_weight is not None:
        q = rms_norm(q, q_norm_weight, eps)
    if k_norm_weight is not None:
        k = rms_norm(k, k_norm_weight, eps)
    cs = cos_sin[positions.long()]
    cos, sin = cs[:, None, : head_dim // 2], cs[:, None, head_dim // 2:]
    q = _rotate(q.float(), cos, sin).to(qkv.dtype)
    k = _rotate(k.float(), cos, sin).to(qkv.dtype)
    if k_cache is not None and slot_mapping is not None:
        valid = slot_mapping >= 0
        slots = slot_mapping[valid].long()
        bs = k_cache.shape[2]
        blk, off = slots // bs, slots % bs
        k_cache[blk, :, off] = k[valid].to(k_cache.dtype)
        v_cache[blk, :, off] = v[valid].to(v_cache.dtype)
    return q.contiguous()


# -------------------------------------------------------------- attention
def gather_paged(cache: torch.Tensor, block_table: torch.Tensor, length: int) -> torch.Tensor:
    """Rows [0, length) of one request from the pool: [length, Hkv, D]."""
    block_size = cache.shape[2]
    nb = -(-length // block_size)
    rows = cache[block_table[:nb].long()].permute(0, 2, 1, 3).reshape(nb * block_size, cache.shape[1],
                                                                       cache.shape[3])
    return rows[:length]


def _sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal_offset: Optional[int]):
    # q [Sq, Hq, D], k/v [Sk, Hkv, D] -> [Sq, Hq, D], fp32 math
    Sq, Hq, D = q.shape
    Sk, Hkv, _ = k.shape
    g = Hq // Hkv
    qf = q.float().view(Sq, Hkv, g, D).permute(1, 2, 0, 3)          # [Hkv, g, Sq, D]
    kf = k.float().permute(1, 0, 2)[:, None]                        # [Hkv, 1, Sk, D]
    vf = v.float().permute(1, 0, 2)[:, None]
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale              # [Hkv, g, Sq, Sk]
    if causal_offset is not None:
        qi = torch.arange(Sq, device=q.device)[:, None] + causal_offset
        ki = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)                                         # [Hkv, g, Sq, D]
    return o.permute(2, 0, 1, 3).reshape(Sq, Hq, D)


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_tables: torch.Tensor, cu_seqlens_q: torch.Tensor,
                      kv_lens: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal attention of new query rows over the paged K/V of their request.

    q: [T, Hq, D] (requests concatenated, boundaries in cu_seqlens_q).  Request i
    has kv_lens[i] rows in the pool, of which the last q_len_i belong to these
    queries (the K/V of the new rows were stored before this call).
    """
    out = torch.empty_like(q)
    cu = cu_seqlens_q.tolist()
    kl = kv_lens.tolist()
    for i in range(len(kl)):
        s, e = cu[i], cu[i + 1]
        if e == s:
            continue
        k = gather_paged(k_cache, block_tables[i], kl[i])
        v = gather_paged(v_cache, block_tables[i], kl[i])
        out[s:e] = _sdpa(q[s:e], k, v, scale, kl[i] - (e - s)).to(q.dtype)
    return out


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, context_lens: torch.Tensor, scale: float) -> torch.Tensor:
    """One query row per request over its paged K/V.  q: [B, Hq, D]."""
    out = torch.empty_like(q)
    cl = context_lens.tolist()
    for i, n in enumerate(cl):
        if n <= 0:
            out[i] = 0
            continue
        k = gather_paged(k_cache, block_tables[i], n)
        v = gather_paged(v_cache, block_tables[i], n)
        out[i:i + 1] = _sdpa(q[i:i + 1], k, v, scale, None).to(q.dtype)
    return out


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Non-causal attention for vision towers.  q/k/v: [B, S, H, D]; key_mask [B, Sk] bool (True = keep)."""
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if key_mask is not None:
        s = s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
    o = torch.matmul(torch.softmax(s, dim=-1), vf)
    return o.permute(0, 2, 1, 3).to(q.dtype).contiguous()


# ----------------------------------------------------------- embed / sample
def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Rows of a (vocab-sharded) table; ids outside the shard give zeros."""
    local = ids.long() - vocab_start
    ok = (local >= 0) & (local < weight.shape[0])
    out = F.embedding(local.clamp(0, weight.shape[0] - 1), weight)
    return out * ok[:, None].to(out.dtype)


def sample(logits: torch.Tensor, temperatures: torch.Tensor, noise: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy where temperature == 0, else Gumbel-max style exponential race.

    `noise` (same shape as logits, Exp(1) samples) can be passed for
    reproducible tests; the reference draws it inside
    (nanovllm/layers/sampler.py:10-17).
    """
    lf = logits.float()
    greedy = lf.argmax(dim=-1)
    t = temperatures.float().clamp_min(1e-10)[:, None]
    probs = torch.softmax(lf / t, dim=-1)
    if noise is None:
        noise = torch.empty_like(probs).exponential_(1)
    picked = (probs / noise.clamp_min(1e-10)).argmax(dim=-1)
    return torch.where(temperatures == 0, greedy, picked)
