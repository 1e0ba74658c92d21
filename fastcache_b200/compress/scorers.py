"""KV-row importance scores and the keep-set selection built on them.

The reference delegates scoring to the external `kvpress` package in its
HuggingFace harness (utils_ccm/utils_compress.py:200-349) and has a partial
native restatement in the engine (nanovllm/kernels/kvpress_compressor.py:
169-251: streaming_llm, knorm (largest head-mean norm, shared indices) and
random; every other method degrades to uniform striding there).  This module
implements the published algorithms directly:

  knorm               score = -||k||  per (kv head, row)                (Devoto et al.)
  knorm_ref           score = +mean_heads ||k||, shared by heads        (reference engine variant)
  snapkv              softmax attention of the last `window` queries over the
                      earlier keys, mean over window and GQA group, 1-D average
                      pool (kernel k, same padding); window rows always kept
  expected_attention  exp(mu.k/sqrt(d) + k^T Sigma k / (2d)) * ||v|| with the mean and
                      covariance of the observed queries; `n_sink` rows always kept
  tova                attention of the last query, mean over heads (shared indices)
  observed_attention  mean attention over all observed queries (H2O-style)
  streaming_llm       `n_sink` first rows + the most recent rows
  random / uniform    random subset / uniform stride
All scores are fp32 `[Hkv, S]`, higher = keep.  `select_keep` turns them into
sorted row indices per head.  Kept rows are the original rotated keys.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F

NEG = float("-inf")
POS = float("inf")


def n_kept_for(seq_len: int, ratio: float) -> int:
    """Rows kept at eviction ratio `ratio` (nanovllm/kernels/kvpress_compressor.py:192-198)."""
    return max(1, int(seq_len * (1.0 - ratio)))


def ratio_from_factor(factor: float) -> float:
    return 1.0 - 1.0 / float(factor)


# ----------------------------------------------------------------- scorers
def knorm(keys, values=None, queries=None, **kw):
    return -keys.float().norm(dim=-1)


def knorm_ref(keys, values=None, queries=None, **kw):
    s = keys.float().norm(dim=-1).mean(dim=0, keepdim=True)
    return s.expand(keys.shape[0], -1).contiguous()


def _window_attention(keys: torch.Tensor, queries: torch.Tensor) -> torch.Tensor:
    """Causal softmax attention of the trailing queries.  keys [Hkv,S,D], queries [Hq,w,D] -> [Hq,w,S]."""
    Hkv, S, D = keys.shape
    Hq, w, _ = queries.shape
    g = Hq // Hkv
    k = keys.float().repeat_interleave(g, dim=0)
    s = torch.matmul(queries.float(), k.transpose(-1, -2)) / math.sqrt(D)
    qpos = torch.arange(S - w, S, device=keys.device)[:, None]
    kpos = torch.arange(S, device=keys.device)[None, :]
    s = s.masked_fill(kpos > qpos, NEG)
    return torch.softmax(s, dim=-1)


def snapkv(keys, values=None, queries=None, window: int = 64, kernel_size: int = 5, **kw):
    if queries is None:
        raise ValueError("snapkv needs the observation-window queries")
    Hkv, S, D = keys.shape
    w = min(window, queries.shape[1], S)
    queries = queries[:, -w:]
    attn = _window_attention(keys, queries)                       # [Hq, w, S]
    votes = attn[..., : S - w].mean(dim=1)                        # [Hq, S-w]
    votes = votes.view(Hkv, -1, S - w).mean(dim=1)                # GQA group mean
    if S - w > 0 and kernel_size > 1:
        votes = F.avg_pool1d(votes[:, None, :], kernel_size, stride=1, padding=kernel_size // 2,
                             count_include_pad=True)[:, 0, : S - w]
    scores = torch.full((Hkv, S), POS, dtype=torch.float32, device=keys.device)
    scores[:, : S - w] = votes
    return scores


def tova(keys, values=None, queries=None, **kw):
    if queries is None:
        raise ValueError("tova needs the last query")
    Hkv, S, D = keys.shape
    attn = _window_attention(keys, queries[:, -1:])[:, 0]          # [Hq, S]
    s = attn.mean(dim=0, keepdim=True).expand(Hkv, -1).contiguous()
    s[:, -1] = POS
    return s


def observed_attention(keys, values=None, queries=None, **kw):
    if queries is None:
        raise ValueError("observed_attention needs queries")
    Hkv, S, D = keys.shape
    attn = _window_attention(keys, queries)                        # [Hq, w, S]
    w = queries.shape[1]
    # each key is visible to a different number of the observed queries
    seen = (torch.arange(S, device=keys.device)[None, :] <=
            torch.arange(S - w, S, device=keys.device)[:, None]).sum(dim=0).clamp_min(1)
    s = attn.sum(dim=1) / seen
    return s.view(Hkv, -1, S).mean(dim=1)


def expected_attention(keys, values=None, queries=None, n_sink: int = 4, **kw):
    if queries is None or values is None:
        raise ValueError("expected_attention needs queries and values")
    Hkv, S, D = keys.shape
    Hq = queries.shape[0]
    g = Hq // Hkv
    q = queries.float().reshape(Hkv, g * queries.shape[1], D)
    mu = q.mean(dim=1)                                             # [Hkv, D]
    qc = q - mu[:, None, :]
    cov = torch.matmul(qc.transpose(1, 2), qc) / max(1, q.shape[1] - 1)   # [Hkv, D, D]
    kf = keys.float()
    lin = torch.einsum("hsd,hd->hs", kf, mu) / math.sqrt(D)
    quad = torch.einsum("hsd,hde,hse->hs", kf, cov, kf) / (2.0 * D)
    logit = lin + quad
    logit = logit - logit.max(dim=-1, keepdim=True).values
    s = torch.exp(logit) * values.float().norm(dim=-1)
    s[:, : min(n_sink, S)] = POS
    return s


def streaming_llm(keys, values=None, queries=None, n_sink: int = 4, **kw):
    Hkv, S, _ = keys.shape
    s = torch.arange(S, dtype=torch.float32, device=keys.device)[None, :].expand(Hkv, -1).contiguous()
    s[:, : min(n_sink, S)] = POS
    return s


def random_scores(keys, values=None, queries=None, seed: int = 0, **kw):
    Hkv, S, _ = keys.shape
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = torch.rand(S, generator=g).to(keys.device)
    return s[None, :].expand(Hkv, -1).contiguous()


def uniform(keys, values=None, queries=None, n_kept: Optional[int] = None, **kw):
    """Uniform striding (what the reference engine does for methods it has no code for)."""
    Hkv, S, _ = keys.shape
    n = n_kept or max(1, S // 2)
    idx = torch.linspace(0, S - 1, n, device=keys.device).round().long()
    s = torch.zeros(S, dtype=torch.float32, device=keys.device)
    s[idx] = 1.0
    return s[None, :].expand(Hkv, -1).contiguous()


SCORERS: Dict[str, Callable] = {
    "knorm": knorm, "knorm_ref": knorm_ref, "snapkv": snapkv, "expected_attention": expected_attention,
    "tova": tova, "observed_attention": observed_attention, "h2o": observed_attention,
    "streaming_llm": streaming_llm, "random": random_scores, "uniform": uniform,
}
NEEDS_QUERIES = {"snapkv", "expected_attention", "tova", "observed_attention", "h2o"}
SHARED_INDICES = {"knorm_ref", "tova", "streaming_llm", "random", "uniform"}


def score_keys(method: str, keys: torch.Tensor, values: Optional[torch.Tensor] = None,
               queries: Optional[torch.Tensor] = None, **params) -> torch.Tensor:
    """keys/values [Hkv, S, D], queries [Hq, w, D] (rotated, trailing rows of the prompt) -> [Hkv, S]."""
    try:
        fn = SCORERS[method]
    except KeyError:
        raise ValueError(f"unknown scoring method {method!r}; have {sorted(SCORERS)}") from None
    return fn(keys, values, queries, **params)


def select_keep(scores: torch.Tensor, n_kept: int) -> torch.Tensor:
    """Indices of the `n_kept` best rows per head, ascending.  scores [Hkv, S] -> int64 [Hkv, n_kept].

    Ties are broken toward the later row (recency), deterministically.
    """
    Hkv, S = scores.shape
    n_kept = max(1, min(int(n_kept), S))
    s = scores.float().clone()
    s = torch.where(torch.isposinf(s), torch.full_like(s, 3.0e38), s)
    # stable descending sort on (score, position): flip so later rows win ties
    order = torch.argsort(s.flip(-1), dim=-1, descending=True, stable=True)
    idx = (S - 1) - order[:, :n_kept]
    return idx.sort(dim=-1).values
