"""Compression methods behind one interface.

Parity: nanovllm/autocompress/methods.py:43-853 — `CompressionMethod` ABC,
`MLPCompressionMethod`, `KVPressMethod` (snapkv, streaming_llm, observed /
expected attention, knorm, tova, think, simlayer, h2o, random), and
`QuantizationMethod` (INT8 sym/asym, INT4 group-128 packed, FP8 e4m3/e5m2, NF4)
with `dequantize`, plus `MethodRegistry`.  Methods act on HF-format tensors
`[B, H, S, D]`; the serving engine uses the in-pool forms in
`fastcache_b200.compress.inpool` instead.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..compress import quant as Q
from ..compress.scorers import NEEDS_QUERIES, n_kept_for, score_keys, select_keep
from .profiles import CompressMethodProfile, get_profile

KV = List[Tuple[torch.Tensor, torch.Tensor]]


class CompressionMethod(ABC):
    name = "base"

    def __init__(self, profile: Optional[CompressMethodProfile] = None, **kwargs: Any):
        self.profile = profile
        self.kwargs = kwargs

    @abstractmethod
    def compress(self, kv_cache: KV, **ctx: Any) -> KV:
        ...

    def __call__(self, kv_cache: KV, **ctx: Any) -> KV:
        return self.compress(kv_cache, **ctx)

    def output_len(self, seq_len: int) -> int:
        return self.profile.get_output_seq_len(seq_len) if self.profile is not None else seq_len

    def get_optimal_timing(self, workload: Any, hw_profile: Any) -> "ExecutionTiming":
        """When to run relative to prefill and decode (reference methods.py:80-110): methods that
        need attention scores run inside prefill when they are cheap (under 1 ms), otherwise after
        it; the others overlap with decode when decode is memory-bound and the profile allows it."""
        from .cost_model import CostModel
        from .execution import ExecutionTiming
        p = self.profile
        if p is None:
            return ExecutionTiming.AFTER_PREFILL
        if p.requires_attention:
            cheap = CostModel(hw_profile).compress_latency_ms(p, workload) < 1.0
            return ExecutionTiming.INLINE_PREFILL if cheap else ExecutionTiming.AFTER_PREFILL
        mem_bound = hw_profile.is_decode_memory_bound(workload.batch_size, workload.seq_len, workload.num_layers,
                                                      workload.num_kv_heads, workload.head_dim,
                                                      workload.hidden_size)
        if p.can_overlap_with_decode(mem_bound) and p.decode_compatibility >= 0.5:
            return ExecutionTiming.ASYNC_DECODE
        return ExecutionTiming.AFTER_PREFILL


class MLPCompressionMethod(CompressionMethod):
    """CCM merge: a trained compressor module folds f rows into one."""
    name = "mlp"

    def __init__(self, compressor: Any = None, compression_ratio: float = 4.0, num_layers: int = 32, **kw):
        p = get_profile("mlp")
        p = CompressMethodProfile(**{**p.__dict__, "compression_ratio": float(compression_ratio)})
        super().__init__(p, num_layers=num_layers, **kw)
        self.compressor = compressor

    def compress(self, kv_cache: KV, it_len: Sequence[int] = (0, 0), **ctx: Any) -> KV:
        if self.compressor is None:
            raise RuntimeError("MLPCompressionMethod needs a compressor module")
        return self.compressor(kv_cache, it_len=list(it_len))

    def get_optimal_timing(self, workload: Any, hw_profile: Any) -> "ExecutionTiming":
        """Small batches compress right after prefill (the merge GEMMs are too small to be worth a
        second stream); from batch 4 with memory-bound decode, or batch 8, overlap with decode
        (reference methods.py:200-230)."""
        from .execution import ExecutionTiming
        if workload.batch_size < 4:
            return ExecutionTiming.AFTER_PREFILL
        mem_bound = hw_profile.is_decode_memory_bound(workload.batch_size, workload.seq_len, workload.num_layers,
                                                      workload.num_kv_heads, workload.head_dim,
                                                      workload.hidden_size)
        if mem_bound or workload.batch_size >= 8:
            return ExecutionTiming.ASYNC_DECODE
        return ExecutionTiming.AFTER_PREFILL


class KVPressMethod(CompressionMethod):
    """Score-based eviction; the published algorithms are implemented in compress/scorers.py."""
    name = "kvpress"
    SUPPORTED = ("snapkv", "streaming_llm", "observed_attention", "expected_attention", "knorm", "knorm_ref",
                 "tova", "h2o", "random", "uniform", "think", "simlayer")

    def __init__(self, method: str = "knorm", compression_ratio: float = 0.5, **kw):
        if method not in self.SUPPORTED:
            raise ValueError(f"unknown eviction method {method!r}; have {self.SUPPORTED}")
        self.method = method
        self.drop_ratio = float(compression_ratio)
        base = get_profile(method if method in ("snapkv", "streaming_llm", "h2o", "knorm") else "knorm")
        keep = max(1e-6, 1.0 - self.drop_ratio)
        super().__init__(CompressMethodProfile(**{**base.__dict__, "name": f"kvpress_{method}",
                                                  "compression_ratio": 1.0 / keep,
                                                  "requires_attention": method in NEEDS_QUERIES}), **kw)

    def compress(self, kv_cache: KV, queries: Optional[List[torch.Tensor]] = None, **ctx: Any) -> KV:
        out: KV = []
        for layer, (k, v) in enumerate(kv_cache):
            B, H, S, D = k.shape
            n_kept = n_kept_for(S, self.drop_ratio)
            if n_kept >= S:
                out.append((k, v))
                continue
            if self.method == "think":           # channel pruning keeps every row: identity on the row axis
                out.append((k, v))
                continue
            if self.method == "simlayer":        # layer-wise switch to streaming for "lazy" layers
                method = "streaming_llm"
            else:
                method = self.method
            ks, vs = [], []
            for b in range(B):
                q = queries[layer][b] if (queries is not None and method in NEEDS_QUERIES) else None
                if method in NEEDS_QUERIES and q is None:
                    method_b = "uniform"        # no queries were recorded: same degradation as the reference
                else:
                    method_b = method
                s = score_keys(method_b, k[b], v[b], q, n_kept=n_kept, **self.kwargs)
                idx = select_keep(s, n_kept)[:, :, None].expand(-1, -1, D)
                ks.append(torch.gather(k[b], 1, idx))
                vs.append(torch.gather(v[b], 1, idx))
            out.append((torch.stack(ks), torch.stack(vs)))
        return out


class QuantizationMethod(CompressionMethod):
    """Fake-compression of precision: quantise K/V, keep the packed form, `dequantize` restores bf16/fp32."""
    name = "quant"
    MODES = ("int8", "int8_asym", "int4", "fp8_e4m3", "fp8_e5m2", "nf4")

    def __init__(self, mode: str = "int8", group_size: int = 128, **kw):
        if mode not in self.MODES:
            raise ValueError(f"unknown quantisation mode {mode!r}; have {self.MODES}")
        self.mode, self.group_size = mode, group_size
        ratio = {"int8": 2.0, "int8_asym": 2.0, "int4": 4.0, "nf4": 4.0, "fp8_e4m3": 2.0, "fp8_e5m2": 2.0}[mode]
        base = get_profile("int4_quant" if ratio == 4.0 else "int8_quant")
        super().__init__(CompressMethodProfile(**{**base.__dict__, "name": f"quant_{mode}",
                                                  "compression_ratio": ratio}), **kw)

    def quantize(self, x: torch.Tensor) -> Dict[str, Any]:
        return Q.quantize(x, self.mode, self.group_size)

    def dequantize(self, packed: Dict[str, Any]) -> torch.Tensor:
        return Q.dequantize(packed)

    def compress(self, kv_cache: KV, **ctx: Any):
        return [(self.quantize(k), self.quantize(v)) for k, v in kv_cache]

    def decompress(self, packed) -> KV:
        return [(self.dequantize(k), self.dequantize(v)) for k, v in packed]

    def get_optimal_timing(self, workload: Any, hw_profile: Any) -> "ExecutionTiming":
        """Quantisation streams the cache once: after prefill for short prompts, layer by layer
        beside decode for long ones (reference methods.py:759-790)."""
        from .execution import ExecutionTiming
        return ExecutionTiming.AFTER_PREFILL if workload.seq_len < 1024 else ExecutionTiming.ASYNC_DECODE


class MethodRegistry:
    _factories: Dict[str, Any] = {}

    @classmethod
    def register(cls, name: str, factory) -> None:
        cls._factories[name] = factory

    @classmethod
    def create(cls, name: str, **kw) -> CompressionMethod:
        if name in cls._factories:
            return cls._factories[name](**kw)
        if name == "mlp":
            return MLPCompressionMethod(**kw)
        if name.startswith("kvpress_"):
            return KVPressMethod(name[len("kvpress_"):], **kw)
        if name in KVPressMethod.SUPPORTED:
            return KVPressMethod(name, **kw)
        if name.startswith("quant_"):
            return QuantizationMethod(name[len("quant_"):], **kw)
        if name in ("int8_quant", "int4_quant"):
            return QuantizationMethod(name.split("_")[0], **kw)
        raise KeyError(f"unknown compression method {name!r}")

    @classmethod
    def list_methods(cls) -> List[str]:
        return cls.names()

    @classmethod
    def names(cls) -> List[str]:
        return sorted(set(cls._factories) | {"mlp"} | {f"kvpress_{m}" for m in KVPressMethod.SUPPORTED} |
                      {f"quant_{m}" for m in QuantizationMethod.MODES})


def get_method(name: str, **kw) -> CompressionMethod:
    return MethodRegistry.create(name, **kw)


def list_methods() -> List[str]:
    return MethodRegistry.names()
