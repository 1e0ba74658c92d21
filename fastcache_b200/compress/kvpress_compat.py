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

    def reset_timeCheck(self) -> None:
        self.totalTime = 0.0

    def forward_hook(self, module: Any, input: Any, kwargs: dict, output: Any):
        """Forward hook of a HuggingFace attention layer (`register_forward_hook(..., with_kwargs=True)`):
        once prefill has filled the layer's cache, compress that layer in place and time it on the
        device (the reference's hook accumulates host time without a synchronize,
        utils_ccm/utils_compress.py:209-268).  Decode steps (one query row) pass through."""
        hidden = kwargs.get("hidden_states", input[0] if input else None)
        cache = kwargs.get("past_key_value", kwargs.get("past_key_values"))
        if hidden is None or cache is None or hidden.shape[1] <= 1:
            return output
        li = int(getattr(module, "layer_idx", 0))
        layers = getattr(cache, "layers", None)
        if layers is not None:
            k, v = layers[li].keys, layers[li].values
        else:
            k, v = cache.key_cache[li], cache.value_cache[li]
        (ck, cv), = self([(k, v)])
        if layers is not None:
            layers[li].keys, layers[li].values = ck, cv
        else:
            cache.key_cache[li], cache.value_cache[li] = ck, cv
        return output


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
    """Named accumulating timers plus per-token decode latencies (utils_ccm/utils_compress.py:414-475).

    `timeTik(name)` / `timeTok(name)` bracket a region: its time adds to `timeTable[name]` and its
    count to `timeTimesTable[name]`.  With `pos_tik_check` set, `timeTikPos()` stamps the moment a
    token was produced and `timeTokPos(next_id)` records the time since the stamp `src_id`."""

    def __init__(self) -> None:
        self.timeTable: Dict[str, float] = {}
        self.timeTimesTable: Dict[str, int] = {}
        self.startTimeTable: Dict[str, float] = {}
        self.pos_tik_check = 0
        self.pos_reset()

    @property
    def totals(self) -> Dict[str, float]:
        return self.timeTable

    def timeTik(self, token_name: str = "") -> None:
        self.timeTable.setdefault(token_name, 0.0)
        self.timeTimesTable.setdefault(token_name, 0)
        self.startTimeTable[token_name] = time.perf_counter()

    def timeTok(self, token_name: str = "") -> float:
        dt = time.perf_counter() - self.startTimeTable[token_name]
        self.timeTable[token_name] += dt
        self.timeTimesTable[token_name] += 1
        return dt

    tik, tok = timeTik, timeTok

    def timeTikPos(self) -> None:
        if self.pos_tik_check:
            self.generated_id_time.append(time.perf_counter())

    def timeTokPos(self, next_id: int) -> None:
        if self.pos_tik_check:
            self.generated_pos_latency.append(time.perf_counter() - self.generated_id_time[self.src_id])
            self.src_id = next_id

    def get_token_time(self) -> List[float]:
        return self.generated_pos_latency

    def reset(self) -> None:
        for name in self.timeTable:
            self.timeTable[name], self.timeTimesTable[name] = 0.0, 0

    def report(self) -> str:
        return "\n".join(f"{n}: {self.timeTable[n]:.4f}. {self.timeTimesTable[n]}" for n in self.timeTable)

    def show(self) -> None:
        print(self.report())

    def show_and_reset(self) -> None:
        self.show()
        self.reset()

    def pos_reset(self) -> None:
        self.generated_pos_latency: List[float] = []
        self.generated_id_time: List[float] = []
        self.src_id = 0

    def show_posTik(self) -> None:
        print("generated_pos_latency", self.generated_pos_latency)

    def show_posTik_and_reset(self) -> None:
        self.show_posTik()
        self.pos_reset()
