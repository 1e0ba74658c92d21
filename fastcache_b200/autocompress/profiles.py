"""Compression-method profiles: what kind of work a method is and what it costs.

Parity: nanovllm/autocompress/profiles.py:17-331 (ComputeType, CompressMethodProfile,
built-in profiles mlp / snapkv / streaming_llm / h2o / int4_quant / int8_quant and a
registry).  Latency models here are roofline estimates against a HardwareProfile
instead of fixed A100 guesses: bytes moved / bandwidth for MEMORY methods, FLOPs /
tensor throughput for GEMM methods, the larger of the two for MIXED.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional


class ComputeType(Enum):
    GEMM = "gemm"        # tensor-core bound (CCM MLP merge)
    MEMORY = "memory"    # bandwidth bound (eviction, gather, quantisation)
    MIXED = "mixed"      # attention-score based selection


@dataclass
class CompressMethodProfile:
    name: str
    compute_type: ComputeType
    decode_compatibility: float = 0.5          # 0..1: how well it hides under decode
    latency_params: Dict[str, float] = field(default_factory=lambda: {
        "base_ms": 0.02, "per_token_us": 0.05, "per_batch_scale": 1.0})
    chunkable: bool = False
    min_chunk_size: int = 1
    max_chunk_size: int = 32
    requires_attention: bool = False
    modifies_seq_len: bool = False
    modifies_precision: bool = False
    compression_ratio: float = 1.0             # input rows / output rows (1 = none)
    flops_per_row: float = 0.0                 # per KV row per layer per K|V
    bytes_per_row: float = 0.0
    _custom_latency_fn: Optional[Callable[[int, int], float]] = None

    def estimate_latency(self, seq_len: int, batch_size: int) -> float:
        """Milliseconds for one layer-batch of work on the profile's default assumptions."""
        if self._custom_latency_fn is not None:
            return float(self._custom_latency_fn(seq_len, batch_size))
        p = self.latency_params
        rows = seq_len * batch_size
        return p.get("base_ms", 0.0) + rows * p.get("per_token_us", 0.0) * 1e-3 * p.get("per_batch_scale", 1.0)

    def get_output_seq_len(self, input_seq_len: int) -> int:
        if not self.modifies_seq_len or self.compression_ratio <= 1.0:
            return input_seq_len
        return max(1, int(input_seq_len / self.compression_ratio))

    def can_overlap_with_decode(self, decode_is_memory_bound: bool) -> bool:
        """GEMM work hides under memory-bound decode; memory work competes with it."""
        if self.compute_type is ComputeType.GEMM:
            return decode_is_memory_bound and self.decode_compatibility >= 0.5
        if self.compute_type is ComputeType.MEMORY:
            return (not decode_is_memory_bound) and self.decode_compatibility >= 0.5
        return self.decode_compatibility >= 0.7


def _mlp_profile(ratio: float = 4.0, head_dim: int = 128) -> CompressMethodProfile:
    f = ratio
    flops = 2.0 * head_dim * (head_dim * f + 2 * head_dim) / f      # per input row
    return CompressMethodProfile(
        name="mlp", compute_type=ComputeType.GEMM, decode_compatibility=0.9, chunkable=True,
        min_chunk_size=1, max_chunk_size=8, modifies_seq_len=True, compression_ratio=ratio,
        flops_per_row=flops, bytes_per_row=2.0 * head_dim * (1 + 1 / f),
        latency_params={"base_ms": 0.01, "per_token_us": 0.004, "per_batch_scale": 1.0})


BUILTIN_PROFILES: Dict[str, CompressMethodProfile] = {
    "mlp": _mlp_profile(),
    "snapkv": CompressMethodProfile("snapkv", ComputeType.MIXED, 0.4, requires_attention=True,
                                    modifies_seq_len=True, compression_ratio=2.0, bytes_per_row=512.0,
                                    flops_per_row=2 * 64 * 128,
                                    latency_params={"base_ms": 0.02, "per_token_us": 0.002, "per_batch_scale": 1.0}),
    "streaming_llm": CompressMethodProfile("streaming_llm", ComputeType.MEMORY, 0.8, modifies_seq_len=True,
                                           compression_ratio=2.0, bytes_per_row=512.0,
                                           latency_params={"base_ms": 0.005, "per_token_us": 0.0005,
                                                           "per_batch_scale": 1.0}),
    "knorm": CompressMethodProfile("knorm", ComputeType.MEMORY, 0.6, modifies_seq_len=True, compression_ratio=2.0,
                                   bytes_per_row=768.0,
                                   latency_params={"base_ms": 0.01, "per_token_us": 0.001, "per_batch_scale": 1.0}),
    "h2o": CompressMethodProfile("h2o", ComputeType.MIXED, 0.3, requires_attention=True, modifies_seq_len=True,
                                 compression_ratio=2.0, bytes_per_row=512.0, flops_per_row=2 * 128 * 128,
                                 latency_params={"base_ms": 0.03, "per_token_us": 0.004, "per_batch_scale": 1.0}),
    "int8_quant": CompressMethodProfile("int8_quant", ComputeType.MEMORY, 0.7, chunkable=True,
                                        modifies_precision=True, compression_ratio=2.0, bytes_per_row=384.0,
                                        latency_params={"base_ms": 0.005, "per_token_us": 0.0008,
                                                        "per_batch_scale": 1.0}),
    "int4_quant": CompressMethodProfile("int4_quant", ComputeType.MEMORY, 0.7, chunkable=True,
                                        modifies_precision=True, compression_ratio=4.0, bytes_per_row=320.0,
                                        latency_params={"base_ms": 0.005, "per_token_us": 0.001,
                                                        "per_batch_scale": 1.0}),
}
for _alias, _src in (("expected_attention", "snapkv"), ("observed_attention", "h2o"), ("tova", "snapkv"),
                     ("random", "streaming_llm"), ("knorm_ref", "knorm")):
    _p = BUILTIN_PROFILES[_src]
    BUILTIN_PROFILES[_alias] = CompressMethodProfile(**{**_p.__dict__, "name": _alias})


def register_profile(profile: CompressMethodProfile) -> None:
    BUILTIN_PROFILES[profile.name] = profile


def get_profile(name: str) -> CompressMethodProfile:
    key = name[len("kvpress_"):] if name.startswith("kvpress_") else name
    if key not in BUILTIN_PROFILES:
        raise KeyError(f"unknown compression profile {name!r}; have {sorted(BUILTIN_PROFILES)}")
    return BUILTIN_PROFILES[key]


def list_profiles() -> List[str]:
    return sorted(BUILTIN_PROFILES)
