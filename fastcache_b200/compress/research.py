"""The reference's remaining v1 compressors and cache containers (research code paths).

Parity: utils_ccm/module_ccm_v11.py:35-127 (`LLaMAKVCacheSampler`, `CompressibleCache`),
:347-521 (`MAEEncoder`, `CompressedKVCache`, `CompressedDecoder`, `CompressedDecoder_OnlyMLP`),
:1063-1279 (`CrossModelKVCompressor`, `CrossModelRealKVCompressor`).  None of them is on the
serving path of the reference's engine; they operate on HuggingFace-layout caches
(`[(K, V)] * layers`, each `[B, H, S, D]`).  They are plain PyTorch here as well and run on any
device; the engine's in-pool compressors live in `ccm.py` / `inpool.py`.

Differences from the reference, on purpose:
  * the cross-model compressors merge a trailing group of fewer than `compression_factor` rows by
    repeating its last row up to a full group (the reference reshapes the remainder to one row of
    the wrong width, which only works when the remainder is zero);
  * `CompressibleCache` is self-contained (lists of tensors) instead of a subclass of
    `transformers.DynamicCache`, whose fields changed between major versions.
"""
from __future__ import annotations

import copy
import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

KV = Tuple[torch.Tensor, torch.Tensor]


# ------------------------------------------------------------------------ sampler
class LLaMAKVCacheSampler:
    """Keep the `recent_size` newest rows plus the most attended older rows.

    Older rows are ranked by the softmax attention that the newest key of the LAST layer, used as a
    query, pays to every key, averaged over batch and heads.  The same row set is applied to all layers."""

    def __init__(self, recent_size: int = 128, device: Optional[str] = None):
        self.recent_size = int(recent_size)
        self.device = device

    def importance(self, past_key_values: Sequence[KV]) -> torch.Tensor:
        k = past_key_values[-1][0].float()                          # [B, H, S, D]
        q = k[:, :, -1:, :]
        scores = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(k.shape[-1])
        return torch.softmax(scores, dim=-1).mean(dim=(0, 1, 2))    # [S]

    def hybrid_sampling(self, past_key_values: Sequence[KV], num_samples: int):
        S = past_key_values[0][0].shape[2]
        dev = past_key_values[0][0].device
        n_recent = min(self.recent_size, S)
        recent = torch.arange(S - n_recent, S, device=dev)
        extra = min(num_samples - n_recent, S - n_recent)
        if extra > 0:
            imp = self.importance(past_key_values).to(dev).clone()
            imp[S - n_recent:] = -1.0                               # already kept
            older = torch.topk(imp, k=extra).indices
            idx = torch.sort(torch.cat([older, recent])).values
        else:
            idx = recent
        out = tuple((k.index_select(2, idx), v.index_select(2, idx)) for k, v in past_key_values)
        return out, idx


# ------------------------------------------------------------------------- caches
class CompressibleCache:
    """Per-layer KV lists whose reported length can be pinned (`set_seen_tokens`) so that position ids
    keep counting original tokens after the stored rows were compressed."""

    def __init__(self) -> None:
        self.key_cache: List[torch.Tensor] = []
        self.value_cache: List[torch.Tensor] = []
        self._seen_tokens = -1

    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    def set_seen_tokens(self, seen_tokens: int) -> None:
        self._seen_tokens = int(seen_tokens)

    def __len__(self) -> int:
        return len(self.key_cache)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int) -> KV:
        while len(self.key_cache) <= layer_idx:
            self.key_cache.append(key_states.new_zeros(0))
            self.value_cache.append(value_states.new_zeros(0))
        if self.key_cache[layer_idx].numel() == 0:
            self.key_cache[layer_idx], self.value_cache[layer_idx] = key_states, value_states
        else:
            self.key_cache[layer_idx] = torch.cat([self.key_cache[layer_idx], key_states], dim=-2)
            self.value_cache[layer_idx] = torch.cat([self.value_cache[layer_idx], value_states], dim=-2)
        if layer_idx == 0 and self._seen_tokens >= 0:
            self._seen_tokens += key_states.shape[-2]
        return self.key_cache[layer_idx], self.value_cache[layer_idx]

    def get_actual_seq_length(self, layer_idx: int = 0) -> int:
        if len(self.key_cache) <= layer_idx or self.key_cache[layer_idx].numel() == 0:
            return 0
        return int(self.key_cache[layer_idx].shape[-2])

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen_tokens if self._seen_tokens >= 0 else self.get_actual_seq_length(layer_idx)

    def to_legacy_cache(self) -> Tuple[KV, ...]:
        return tuple(zip(self.key_cache, self.value_cache))

    @classmethod
    def from_legacy_cache(cls, past: Sequence[KV]) -> "CompressibleCache":
        c = cls()
        for i, (k, v) in enumerate(past):
            c.update(k, v, i)
        return c

    def clone(self) -> "CompressibleCache":
        new = copy.copy(self)
        new.key_cache = [k.clone().detach() for k in self.key_cache]
        new.value_cache = [v.clone().detach() for v in self.value_cache]
        return new


class CompressedKVCache:
    """Append-only per-layer store of compressed K/V (`[B, H, S, D]`)."""

    def __init__(self, num_layers: int, num_heads: int, head_dim: int, device="cpu"):
        self.num_layers, self.num_heads, self.head_dim, self.device = num_layers, num_heads, head_dim, device
        self.reset()

    def reset(self) -> None:
        self.key_cache: List[Optional[torch.Tensor]] = [None] * self.num_layers
        self.value_cache: List[Optional[torch.Tensor]] = [None] * self.num_layers

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int) -> KV:
        k, v = self.key_cache[layer_idx], self.value_cache[layer_idx]
        self.key_cache[layer_idx] = key_states if k is None else torch.cat([k, key_states], dim=2)
        self.value_cache[layer_idx] = value_states if v is None else torch.cat([v, value_states], dim=2)
        return self.key_cache[layer_idx], self.value_cache[layer_idx]

    def get(self) -> List[KV]:
        return list(zip(self.key_cache, self.value_cache))


# --------------------------------------------------------------- encoder / decoder
def flatten_kv(kv_cache: Sequence[KV]) -> torch.Tensor:
    """[(K, V)] * L with K, V `[B, H, S, D]` -> `[B, L * S, 2 * H * D]` (K and V features side by side)."""
    rows = []
    for k, v in kv_cache:
        kv = torch.cat([k, v], dim=-1)                               # [B, H, S, 2D]
        rows.append(kv.permute(0, 2, 1, 3).reshape(k.shape[0], k.shape[2], -1))
    return torch.cat(rows, dim=1)


class MAEEncoder(nn.Module):
    """Transformer encoder over every (layer, position) KV row, with a class token that is dropped again."""

    def __init__(self, input_dim: int, hidden_dim: int, num_layers: int, kv_dim: int, nhead: int = 8):
        super().__init__()
        self.projection = nn.Linear(kv_dim, input_dim)
        layer = nn.TransformerEncoderLayer(d_model=input_dim, nhead=nhead, dim_feedforward=hidden_dim,
                                           batch_first=True)
        self.transformer = nn.TransformerEncoder(layer, num_layers=num_layers)
        self.cls_token = nn.Parameter(torch.randn(1, 1, input_dim))

    def forward(self, kv_cache: Sequence[KV]) -> torch.Tensor:
        x = self.projection(flatten_kv(kv_cache))
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1), x], dim=1)
        return self.transformer(x)[:, 1:]


class _PoolingDecoder(nn.Module):
    """Shared tail: split `[B, L * S, hidden]` by layer, average-pool S to the compressed length,
    project to K and V features, reshape to `[B, H, S', D]` pairs."""

    def _decode(self, x: torch.Tensor, num_llm_layers: int, compressed_len: Optional[int], feature_dim: int):
        B, total, _ = x.shape
        per_layer = total // num_llm_layers
        n_out = compressed_len if compressed_len is not None else max(1, per_layer // self.compression_ratio)
        out = []
        for xl in torch.split(x[:, :per_layer * num_llm_layers], per_layer, dim=1):
            pooled = F.adaptive_avg_pool1d(xl.transpose(1, 2), n_out).transpose(1, 2)      # [B, S', hidden]
            kv = self.output_projection(pooled)                                            # [B, S', 2 * out]
            kv = kv.reshape(B, n_out, -1, feature_dim).permute(0, 2, 1, 3)                 # [B, H, S', 2D]
            k, v = torch.split(kv, feature_dim // 2, dim=3)
            out.append((k, v))
        return out


class CompressedDecoder(_PoolingDecoder):
    def __init__(self, input_dim: int, hidden_dim: int, output_dim: int, compression_ratio: int, num_layers: int,
                 num_heads: int, num_llm_layers: int):
        super().__init__()
        self.compression_ratio, self.num_layers, self.num_llm_layers = compression_ratio, num_layers, num_llm_layers
        self.num_heads, self.head_dim = num_heads, output_dim // num_heads
        self.input_projection = nn.Linear(input_dim, hidden_dim)
        layer = nn.TransformerEncoderLayer(d_model=hidden_dim, nhead=num_heads, batch_first=True)
        self.transformer_compressor = nn.TransformerEncoder(layer, num_layers=num_layers)
        self.output_projection = nn.Linear(hidden_dim, output_dim * 2)

    def forward(self, x: torch.Tensor, compressed_len: Optional[int] = None):
        """x: `[B, L * S, F]` with F = 2 * head_dim (one head's K|V features per row group)."""
        h = self.transformer_compressor(self.input_projection(x))
        return self._decode(h, self.num_llm_layers, compressed_len, x.shape[-1])

    def compress_with_len(self, x: torch.Tensor, compressed_len: int):
        return self.forward(x, compressed_len)


class CompressedDecoder_OnlyMLP(_PoolingDecoder):
    def __init__(self, input_dim: int, hidden_dim: int, output_dim: int, compression_ratio: int, num_layers: int,
                 num_heads: int):
        super().__init__()
        self.compression_ratio, self.num_layers, self.num_heads = compression_ratio, num_layers, num_heads
        self.input_projection = nn.Linear(input_dim, hidden_dim)
        self.output_projection = nn.Linear(hidden_dim, output_dim * 2)

    def forward(self, x: torch.Tensor, compressed_len: Optional[int] = None):
        return self._decode(self.input_projection(x), self.num_layers, compressed_len, x.shape[-1])


# ------------------------------------------------------------------- cross-model
class CrossModelKVCompressor(nn.Module):
    """Map the cache of a source model onto a target model with fewer layers and shorter sequences.

    Target layer t reads a learned soft mixture of all source layers (a small MLP of t / T followed by
    a softmax), then a per-target-layer MLP merges every `compression_factor` consecutive rows of a
    head (`heads_ratio` source heads at once in the `Real` variant) into one row of `tgt_dim` features."""

    heads_merge = False

    def __init__(self, src_config, tgt_config, compression_factor: int = 2, device=None, tgt_dim: int = 64):
        super().__init__()
        self.src_layers, self.tgt_layers = src_config.num_hidden_layers, tgt_config.num_hidden_layers
        self.src_heads, self.tgt_heads = src_config.num_key_value_heads, tgt_config.num_key_value_heads
        self.heads_ratio = max(1, self.src_heads // self.tgt_heads) if self.heads_merge else 1
        self.src_dim = getattr(src_config, "head_dim", None) or src_config.hidden_size // src_config.num_attention_heads
        self.tgt_dim = tgt_dim
        self.compression_factor = int(compression_factor)
        self.layer_map_net = nn.Sequential(nn.Linear(1, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU(),
                                           nn.Linear(64, self.src_layers))
        in_dim = self.src_dim * self.compression_factor * self.heads_ratio
        self.compressors = nn.ModuleList(
            nn.Sequential(nn.Linear(in_dim, self.src_dim), nn.ReLU(), nn.Linear(self.src_dim, self.tgt_dim))
            for _ in range(self.tgt_layers))
        if device is not None:
            self.to(device)

    def layer_mixture(self, tgt_layer: int) -> torch.Tensor:
        t = torch.tensor([[tgt_layer / self.tgt_layers]], dtype=torch.float32,
                         device=self.layer_map_net[0].weight.device)
        return F.softmax(self.layer_map_net(t).squeeze(0), dim=0)

    def _merge(self, x: torch.Tensor, mlp: nn.Module) -> torch.Tensor:
        B, H, S, D = x.shape
        f = self.compression_factor
        pad = (-S) % f
        if pad:
            x = torch.cat([x, x[:, :, -1:, :].expand(B, H, pad, D)], dim=2)
        n = x.shape[2] // f
        x = x.reshape(B, H, n, f * D)
        if self.heads_ratio > 1:                                    # [B, Ht, ratio, n, f*D] -> [B, Ht, n, ratio*f*D]
            x = x.reshape(B, H // self.heads_ratio, self.heads_ratio, n, f * D).permute(0, 1, 3, 2, 4)
            x = x.reshape(B, H // self.heads_ratio, n, -1)
        return mlp(x)

    def forward(self, src_kv_cache: Sequence[KV]) -> List[KV]:
        ks = torch.stack([k for k, _ in src_kv_cache]).float()      # [Ls, B, H, S, D]
        vs = torch.stack([v for _, v in src_kv_cache]).float()
        out = []
        for t in range(self.tgt_layers):
            w = self.layer_mixture(t).view(-1, 1, 1, 1, 1)
            k, v = (w * ks).sum(0), (w * vs).sum(0)
            out.append((self._merge(k, self.compressors[t]), self._merge(v, self.compressors[t])))
        return out


class CrossModelRealKVCompressor(CrossModelKVCompressor):
    heads_merge = True


# ----------------------------------------------------------------- small helpers
class PositionalEncoding(nn.Module):
    """Additive sinusoidal positions for `[S, B, d_model]` inputs (utils_ccm/module_ccm_v11.py:333-345)."""

    def __init__(self, d_model: int, max_len: int = 5000):
        super().__init__()
        pos = torch.arange(max_len, dtype=torch.float32)[:, None]
        div = torch.exp(torch.arange(0, d_model, 2, dtype=torch.float32) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : d_model // 2]
        self.register_buffer("pe", pe[:, None, :])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.pe[: x.size(0)]


def logits_to_onehot(logits: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """One-hot of the arg-max along `dim` (utils_ccm/module_ccm_v11.py:2050-2053)."""
    return F.one_hot(logits.argmax(dim=dim), num_classes=logits.size(dim))


def count_true_segments_with_zeros(bool_tensor: torch.Tensor) -> List[int]:
    """Lengths of the pieces a 1-D mask falls into when cut after every False: each piece is a run
    of True values plus the False that ends it; the last piece has no closing False
    (utils_ccm/module_ccm_v11.py:2055-2064).  [T, T, F, T] -> [3, 1]; all True -> [len]."""
    flags = bool_tensor.bool().tolist()
    out, run = [], 0
    for f in flags:
        run += 1
        if not f:
            out.append(run)
            run = 0
    out.append(run)
    return out
