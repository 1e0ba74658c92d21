"""Eviction front ends with the reference's class names.

Parity:
  * KVPressCompressor / KVPressConfig   nanovllm/kernels/kvpress_compressor.py:35-336 — engine-side
    compressor object: `compressor(kv_cache, it_len) -> kv_cache` on HF-format tensors, `n_kept =
    max(1, int(S * (1 - ratio)))`.  The reference implements streaming_llm, knorm (largest head-mean
    norm, shared indices) and random natively and strides uniformly for every other method; here
    every method runs its published algorithm (compress/scorers.py).  `reference_variants=True`
    selects the reference's own knorm variant for like-for-like comparisons.
  * ScorerPressWithTime and the *PressWithTime wrappers, `press_select`, `exec_compression_methods`
    utils_ccm/utils_compress.py:200-411 — timing wrappers around the external `kvpress` presses that
    hook HuggingFace attention modules.  Here a "press" is a callable on HF-format KV that records its
    own device time (CUDA events when the tensors are on a GPU, so the time is real, not the
    unsynchronised host time the reference accumulates).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .scorers import NEEDS_QUERIES, n_kept_for, score_keys, select_keep

KV = List[Tuple[torch.Tensor, torch.Tensor]]


@dataclass
class KVPressConfig:
    method: str = "streaming_llm"
    compression_ratio: float = 0.5          # share of rows dropped
    n_sink: int = 4
    window_size: int = 64
    kernel_size: int = 5
    reference_variants: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)


class KVPressCompressor:
    def __init__(self, method: str = "streaming_llm", compression_ratio: float = 0.5, config: Any = None,
                 reference_variants: bool = False, **kwargs: Any):
        self.cfg = KVPressConfig(method, compression_ratio, kwargs.pop("n_sink", 4), kwargs.pop("window_size", 64),
                                 kwargs.pop("kernel_size", 5), reference_variants, kwargs)
        self.method_name = method
        self.compression_ratio = compression_ratio
        self.model_config = config
        self.total_time_ms = 0.0
        self.calls = 0

    @property
    def kvpress_available(self) -> bool:          # the algorithms are built in; nothing external is needed
        return True

    def _method(self) -> str:
        if self.cfg.reference_variants and self.method_name == "knorm":
            return "knorm_ref"
        return self.method_name

    def _params(self) -> Dict[str, Any]:
        p = dict(self.cfg.extra)
        m = self._method()
        if m in ("streaming_llm", "expected_attention"):
            p["n_sink"] = self.cfg.n_sink
        if m == "snapkv":
            p.update(window=self.cfg.window_size, kernel_size=self.cfg.kernel_size)
        return p

    def _compress_layer(self, keys: torch.Tensor, values: torch.Tensor, layer_idx: int,
                        queries: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        B, H, S, D = keys.shape
        n_kept = n_kept_for(S, self.compression_ratio)
        if n_kept >= S:
            return keys.contiguous(), values.contiguous()
        method = self._method()
        ks, vs = [], []
        for b in range(B):
            q = queries[b] if queries is not None else None
            m = method if (method not in NEEDS_QUERIES or q is not None) else "uniform"
            s = score_keys(m, keys[b], values[b], q, n_kept=n_kept, **self._params())
            idx = select_keep(s, n_kept)[:, :, None].expand(-1, -1, D)
            ks.append(torch.gather(keys[b], 1, idx))
            vs.append(torch.gather(values[b], 1, idx))
        return torch.stack(ks), torch.stack(vs)

    @torch.no_grad()
    def __call__(self, kv_cache: KV, it_len: Sequence[int] = (0, 0), queries: Optional[List[torch.Tensor]] = None
                 ) -> KV:
        timer = _DeviceTimer(kv_cache[0][0])
        out = [self._compress_layer(k, v, l, None if queries is None else queries[l])
               for l, (k, v) in enumerate(kv_cache)]
        self.total_time_ms += timer.stop()
        self.calls += 1
        return out

    def forward(self, kv_cache: KV, it_len: Optional[Sequence[int]] = None, **kwargs: Any) -> KV:
        """Same call under the name the batched compressors use (kvpress_compressor.py:253-289)."""
        if len(kv_cache) == 0:
            return kv_cache
        return self(kv_cache, it_len or (0, 0), kwargs.get("queries"))

    def get_compressed_length(self, original_length: int) -> int:
        return n_kept_for(original_length, self.compression_ratio)

    @property
    def compression_factor(self) -> float:
        return 1.0 / (1.0 - self.compression_ratio)

    def get_stats(self) -> Dict[str, Any]:
        return {"method": self.method_name, "compression_ratio": self.compression_ratio, "calls": self.calls,
                "total_time_ms": self.total_time_ms}


def create_kvpress_compressor(method: str = "streaming_llm", compression_factor: float = 5, config: Any = None,
                              **kwargs: Any) -> KVPressCompressor:
    """Factor f keeps 1 / f of the rows (kvpress_compressor.py:310-336)."""
    return KVPressCompressor(method, 1.0 - 1.0 / compression_factor, config, **kwargs)


class _DeviceTimer:
    def __init__(self, like: torch.Tensor):
        self.cuda = like.is_cuda
        if self.cuda:
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.a.record()
        else:
            self.t0 = time.perf_counter()

    def stop(self) -> float:
        if self.cuda:
            self.b.record()
            self.b.synchronize()
            return float(self.a.elapsed_time(self.b))
        return (time.perf_counter() - self.t0) * 1e3


class ScorerPressWithTime:
    """A press = method + ratio; calling it compresses HF-format KV and accumulates `totalTime` (seconds)."""
    method = "knorm"

    def __init__(self, compression_ratio: float = 0.5, **kwargs: Any):
        self.compression_ratio = compression_ratio
        self._impl = KVPressCompressor(self.method, compression_ratio, **kwargs)
        self.totalTime = 0.0

    def __call__(self, kv_cache: KV, queries: Optional[List[torch.Tensor]] = None) -> KV:
        before = self._impl.total_time_ms
        out = self._impl(kv_cache, queries=queries)
        self.totalTime += (self._impl.total_time_ms - before) / 1e3
        return out


class StreamingLLMPressWithTime(ScorerPressWithTime):
    method = "streaming_llm"


class RandomPressWithTime(ScorerPressWithTime):
    method = "random"


class SnapKVPressWithTime(ScorerPressWithTime):
    method = "snapkv"


class ExpectedAttentionPressWithTime(ScorerPressWithTime):
    method = "expected_attention"


class KnormPressWithTime(ScorerPressWithTime):
    method = "knorm"


class TOVAPressWithTime(ScorerPressWithTime):
    method = "tova"


_PRESSES = {"StreamingLLM": StreamingLLMPressWithTime, "RandomPress": RandomPressWithTime,
            "SnapKV": SnapKVPressWithTime, "ExpectedAttention": ExpectedAttentionPressWithTime,
            "Knorm": KnormPressWithTime, "TOVA": TOVAPressWithTime}


def press_select(name: str, compression_ratio: float = 0.5, **kw: Any) -> ScorerPressWithTime:
    for key, cls in _PRESSES.items():
        if key.lower() == name.lower() or cls.method == name.lower():
            return cls(compression_ratio, **kw)
    raise ValueError(f"unknown press {name!r}; have {sorted(_PRESSES)}")


def exec_compression_methods(kv_cache: KV, name: str, compression_ratio: float = 0.5,
                             queries: Optional[List[torch.Tensor]] = None, **kw: Any) -> Tuple[KV, float]:
    """Compress with the named press; returns (kv, seconds spent)."""
    press = press_select(name, compression_ratio, **kw)
    out = press(kv_cache, queries)
    return out, press.totalTime


def get_underlying_model(model: Any) -> Any:
    """The transformer stack (the object that owns `.layers`) inside a wrapper model.

    Looks through the attribute names the supported families use (LLaVA: `language_model`,
    MiniCPM: `llm`, plus `llava_model`, `llama_model`, `decoder`) and then through `.model` /
    `.transformer` nesting (reference: utils_ccm/utils_compress.py:351-411).  Raises if nothing with
    layers is found, where the reference goes on with None."""
    seen = set()

    def descend(m: Any, depth: int = 0) -> Any:
        if m is None or id(m) in seen or depth > 4:
            return None
        seen.add(id(m))
        if hasattr(m, "layers"):
            return m
        for inner in ("model", "transformer", "decoder"):
            got = descend(getattr(m, inner, None), depth + 1)
            if got is not None:
                return got
        return None

    for attr in ("language_model", "llava_model", "llama_model", "decoder", "llm"):
        got = descend(getattr(model, attr, None))
        if got is not None:
            return got
    got = descend(model)
    if got is None:
        raise AttributeError(f"no transformer stack with `.layers` found in {type(model).__name__}")
    return got


class TimeTik:
    """Named timers (reference: utils_ccm/utils_compress.py:414-475)."""

    def __init__(self) -> None:
        self._t: Dict[str, float] = {}
        self.totals: Dict[str, float] = {}

    def tik(self, name: str) -> None:
        self._t[name] = time.perf_counter()

    def tok(self, name: str) -> float:
        dt = time.perf_counter() - self._t.pop(name)
        self.totals[name] = self.totals.get(name, 0.0) + dt
        return dt
