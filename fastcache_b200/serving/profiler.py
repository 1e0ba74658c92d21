"""Analytic FLOP / byte / operational-intensity model of the serving phases.

Parity: utils_ccm/utils_profiler.py:163-428, :520-908 (LLMIntensityAnalyzer,
LLaVAIntensityAnalyzer, VisionEncoderAnalyzer incl. the KV-compression MLP).  The numbers
are the algorithmic ones (each operand read once, each result written once), which is what
the roofline fractions of the kernels are reported against.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional


@dataclass
class PhaseCost:
    flops: float
    bytes: float

    @property
    def intensity(self) -> float:
        return self.flops / max(self.bytes, 1.0)

    def time_ms(self, tflops: float, gbs: float) -> float:
        return max(self.flops / (tflops * 1e12), self.bytes / (gbs * 1e9)) * 1e3

    def __add__(self, other: "PhaseCost") -> "PhaseCost":
        return PhaseCost(self.flops + other.flops, self.bytes + other.bytes)


class LLMIntensityAnalyzer:
    def __init__(self, hidden: int, layers: int, heads: int, kv_heads: Optional[int] = None,
                 head_dim: Optional[int] = None, ffn: Optional[int] = None, vocab: int = 32000,
                 dtype_bytes: int = 2, tp: int = 1):
        self.h, self.L, self.hq = hidden, layers, heads
        self.hkv = kv_heads or heads
        self.d = head_dim or hidden // heads
        self.ffn = ffn or 4 * hidden
        self.vocab, self.b, self.tp = vocab, dtype_bytes, tp

    def layer_weight_params(self) -> float:
        return (self.h * (self.hq + 2 * self.hkv) * self.d + self.hq * self.d * self.h + 3 * self.h * self.ffn) / self.tp

    def weight_bytes(self) -> float:
        return (self.L * self.layer_weight_params() + self.vocab * self.h / self.tp) * self.b

    def kv_bytes_per_token(self) -> float:
        return 2.0 * self.L * max(1, self.hkv // self.tp) * self.d * self.b

    def prefill(self, batch: int, seq_len: int) -> PhaseCost:
        T = batch * seq_len
        gemm = 2.0 * T * self.L * self.layer_weight_params()
        attn = 4.0 * batch * (self.hq / self.tp) * self.d * seq_len * seq_len / 2 * self.L
        head = 2.0 * batch * self.h * self.vocab / self.tp
        byts = self.weight_bytes() + T * self.kv_bytes_per_token() + 12.0 * T * self.h * self.b * self.L
        return PhaseCost(gemm + attn + head, byts)

    def decode(self, batch: int, context_len: int) -> PhaseCost:
        gemm = 2.0 * batch * (self.L * self.layer_weight_params() + self.h * self.vocab / self.tp)
        attn = 4.0 * batch * (self.hq / self.tp) * self.d * context_len * self.L
        byts = self.weight_bytes() + batch * context_len * self.kv_bytes_per_token()
        return PhaseCost(gemm + attn, byts)

    def compression_mlp(self, batch: int, seq_len: int, factor: int) -> PhaseCost:
        """CCM merge of every layer, K and V: rows/f outputs, (D f -> D -> D -> D) MLP shared by heads."""
        rows = batch * max(1, self.hkv // self.tp) * (seq_len // factor) * self.L * 2
        flops = 2.0 * rows * (self.d * factor * self.d + 2 * self.d * self.d)
        byts = batch * seq_len * self.kv_bytes_per_token() * (1.0 + 1.0 / factor)
        return PhaseCost(flops, byts)

    def eviction(self, batch: int, seq_len: int, keep: float) -> PhaseCost:
        """Key-norm scoring + compaction: read K once for the scores, move the kept K and V rows."""
        kv = batch * seq_len * self.kv_bytes_per_token()
        return PhaseCost(2.0 * batch * seq_len * self.L * max(1, self.hkv // self.tp) * self.d,
                         0.5 * kv + 2.0 * keep * kv)

    def tp_message_bytes(self, tokens: int) -> float:
        """Bytes of one all-reduce payload ([tokens, hidden])."""
        return float(tokens) * self.h * self.b


class VisionEncoderAnalyzer:
    def __init__(self, hidden: int = 1024, layers: int = 24, heads: int = 16, mlp: int = 4096, patches: int = 577,
                 patch: int = 14, dtype_bytes: int = 2):
        self.h, self.L, self.heads, self.mlp, self.n, self.p, self.b = hidden, layers, heads, mlp, patches, patch, dtype_bytes

    def encode(self, images: int) -> PhaseCost:
        T = images * self.n
        gemm = 2.0 * T * self.L * (4 * self.h * self.h + 2 * self.h * self.mlp) + 2.0 * T * 3 * self.p * self.p * self.h
        attn = 4.0 * images * self.n * self.n * self.h * self.L
        byts = self.L * (4 * self.h * self.h + 2 * self.h * self.mlp) * self.b + 10.0 * T * self.h * self.b * self.L
        return PhaseCost(gemm + attn, byts)


class LLaVAIntensityAnalyzer:
    def __init__(self, llm: Optional[LLMIntensityAnalyzer] = None, vision: Optional[VisionEncoderAnalyzer] = None,
                 projector_hidden: int = 4096):
        self.llm = llm or LLMIntensityAnalyzer(4096, 32, 32, 32, 128, 11008, 32064)
        self.vision = vision or VisionEncoderAnalyzer()
        self.proj = projector_hidden

    def projection(self, images: int) -> PhaseCost:
        T = images * (self.vision.n - 1)
        return PhaseCost(2.0 * T * (self.vision.h * self.proj + self.proj * self.proj),
                         (self.vision.h * self.proj + self.proj * self.proj) * 2.0 + 2.0 * T * self.proj * 2)

    def request(self, text_tokens: int = 64, out_tokens: int = 128, factor: int = 0) -> Dict[str, PhaseCost]:
        rows = self.vision.n - 1 + text_tokens
        out = {"vision": self.vision.encode(1), "projection": self.projection(1), "prefill": self.llm.prefill(1, rows)}
        ctx = rows
        if factor > 1:
            out["compress"] = self.llm.compression_mlp(1, rows, factor)
            ctx = rows // factor
        out["decode_per_token"] = self.llm.decode(1, ctx + out_tokens // 2)
        return out
