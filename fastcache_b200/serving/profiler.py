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

    # ---- tensor-driven interface (utils_ccm/utils_profiler.py:294-428): built from a config, fed the step's tensors
    peak_tflops = 1590.0

    @classmethod
    def from_config(cls, config, peak_tflops: float = 1590.0, tp: int = 1):
        """Build the analyzer from a HuggingFace config, a model directory or a config wrapper."""
        w = _as_wrapper(config)
        a = cls(w.hidden_size, w.num_hidden_layers, w.num_attention_heads, w.num_key_value_heads, w.head_dim,
                w.intermediate_size, w.vocab_size, w.dtype_size, tp)
        a.config = w
        a.peak_tflops = peak_tflops
        return a

    def analyze_prefill(self, input_ids, position_ids=None, attention_mask=None) -> Dict:
        B, S = (1, input_ids.shape[0]) if input_ids.dim() == 1 else input_ids.shape
        c = self.prefill(B, S)
        out = B * S * (self.kv_bytes_per_token() + self.h * self.b) + B * self.vocab * self.b
        return _stats(c, B, S, out).report("prefill", self.peak_tflops)

    def analyze_decode(self, input_ids, past_key_values, position_ids=None, attention_mask=None, **_) -> Dict:
        B = 1 if input_ids.dim() == 1 else input_ids.shape[0]
        ctx = int(past_key_values[0][0].shape[2]) if past_key_values else 0
        c = self.decode(B, ctx)
        return _stats(c, B, ctx + 1, B * (self.kv_bytes_per_token() + self.vocab * self.b)).report("decode", self.peak_tflops)


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

    def analyze_vision_encoding(self, batch_size: int = 1) -> ComputeStats:
        c = self.encode(batch_size)
        return _stats(c, batch_size, self.n, batch_size * self.n * self.h * self.b)


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

    # ---- tensor-driven interface (utils_ccm/utils_profiler.py:622-908): built from a config, fed the step's tensors
    @classmethod
    def from_config(cls, config, peak_tflops: float = 1590.0, tp: int = 1):
        w = _as_wrapper(config, LLaVAConfigWrapper)
        v = w.vision_config
        n = (v["image_size"] // v["patch_size"]) ** 2 + 1
        a = cls(LLMIntensityAnalyzer.from_config(w, peak_tflops, tp),
                VisionEncoderAnalyzer(v["hidden_size"], v["num_hidden_layers"], v["num_attention_heads"],
                                      v["intermediate_size"], n, v["patch_size"], w.dtype_size), w.hidden_size)
        a.config = w
        return a

    def analyze_multimodal_prefill(self, input_ids, pixel_values=None, **_) -> Dict:
        B, S = (1, input_ids.shape[0]) if input_ids.dim() == 1 else input_ids.shape
        total, rows = ComputeStats(batch_size=B), S
        if pixel_values is not None:
            n_img = len(pixel_values)
            total = total + self.vision.analyze_vision_encoding(n_img)
            p = self.projection(n_img)
            total = total + _stats(p, n_img, self.vision.n - 1, n_img * (self.vision.n - 1) * self.proj * 2.0)
            rows = S + self.vision.n - 2           # the placeholder token becomes n - 1 feature rows
        c = self.llm.prefill(B, rows)
        total = total + _stats(c, B, rows, B * rows * self.llm.kv_bytes_per_token())
        return total.report("multimodal_prefill", self.llm.peak_tflops)

    def analyze_decode(self, input_ids, past_key_values, **kw) -> Dict:
        return self.llm.analyze_decode(input_ids, past_key_values, **kw)

    def analyze_kv_cache_compression(self, kv_cache, image_len: int, text_len: int,
                                            compression_factor: int = 2) -> Dict:
        """Cost of the merge MLPs over a cache given as per-layer (K, V) of shape [B, H, S, D]: each
        segment of at least `compression_factor` rows is merged, K and V each through a
        (D f -> D -> D -> D) MLP shared by all heads."""
        B, H, _, D = kv_cache[0][0].shape
        b = kv_cache[0][0].element_size()
        f = compression_factor
        weights = (D * f * D + 2 * D * D + 3 * D) * b
        total = ComputeStats(batch_size=B, seq_length=image_len + text_len)
        for _layer in kv_cache:
            for seg in (image_len, text_len):
                if seg < f:
                    continue
                rows = B * H * (seg // f)
                one = ComputeStats(2.0 * rows * (D * f * D + 2 * D * D), rows * D * f * b + weights, rows * D * b, B,
                                   image_len + text_len)
                total = total + one + one           # K and V
        return total.report("kv_cache_compression", self.llm.peak_tflops)


# ------------------------------------------------- types of the tensor-driven interface
# The reference's analyzers are built from a HuggingFace config and take the step's tensors
# (utils_ccm/utils_profiler.py:8-160, :294-428, :520-908).  `from_config` / `analyze_*` of the classes
# above give that interface on top of the shape-driven cost model; these are the types they return and
# the config views they read.  "theoretical_time" uses the peak passed in (the reference hard-codes the
# A100's 312 TFLOP/s).
@dataclass
class ComputeStats:
    flops: float = 0
    memory_read: float = 0
    memory_write: float = 0
    batch_size: int = 1
    seq_length: int = 0

    def __add__(self, other: "ComputeStats") -> "ComputeStats":
        return ComputeStats(self.flops + other.flops, self.memory_read + other.memory_read,
                            self.memory_write + other.memory_write, max(self.batch_size, other.batch_size),
                            max(self.seq_length, other.seq_length))

    @property
    def total_memory(self) -> float:
        return self.memory_read + self.memory_write

    @property
    def compute_intensity(self) -> float:
        return self.flops / self.total_memory if self.total_memory > 0 else 0

    @property
    def per_sample_flops(self) -> float:
        return self.flops / self.batch_size if self.batch_size > 0 else self.flops

    @property
    def per_sample_memory(self) -> float:
        return self.total_memory / self.batch_size if self.batch_size > 0 else self.total_memory

    def report(self, phase: str, peak_tflops: float) -> Dict:
        return {"phase": phase, "batch_size": self.batch_size, "seq_length": self.seq_length, "flops": self.flops,
                "memory_read": self.memory_read, "memory_write": self.memory_write,
                "total_memory": self.total_memory, "compute_intensity": self.compute_intensity,
                "theoretical_time": self.flops / (peak_tflops * 1e12)}


def format_number(number: float, base: int = 1024) -> str:
    units = ["", "K", "M", "G", "T", "P"]
    i = 0
    while number >= base and i < len(units) - 1:
        number, i = number / base, i + 1
    return f"{number:.2f}{units[i]}"


_DTYPE_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "float8_e4m3fn": 1, "int8": 1}


class LLMConfigWrapper:
    """Flat view of a (possibly nested multimodal) HuggingFace config with the fields the cost
    model needs; unknown attributes fall through to the wrapped config."""

    def __init__(self, config):
        self.original_config = config
        text = getattr(config, "text_config", None) or getattr(config, "llm_config", None) or config
        if isinstance(text, dict):
            from types import SimpleNamespace
            text = SimpleNamespace(**text)
        self.hidden_size = text.hidden_size
        self.num_attention_heads = text.num_attention_heads
        self.num_hidden_layers = text.num_hidden_layers
        self.vocab_size = text.vocab_size
        self.intermediate_size = getattr(text, "intermediate_size", 4 * text.hidden_size)
        self.model_type = getattr(text, "model_type", "llama")
        self.num_key_value_heads = getattr(text, "num_key_value_heads", None) or text.num_attention_heads
        self.head_dim = getattr(text, "head_dim", None) or text.hidden_size // text.num_attention_heads
        self.rope_theta = getattr(text, "rope_theta", 10000.0)
        self.max_position_embeddings = getattr(text, "max_position_embeddings", None)
        dt = getattr(config, "torch_dtype", None) or getattr(text, "torch_dtype", None) or getattr(config, "dtype", None)
        self.dtype_size = _DTYPE_BYTES.get(str(dt).replace("torch.", ""), 2)

    @classmethod
    def from_pretrained(cls, model_name_or_path: str):
        from ..config import ModelConfig
        return cls(ModelConfig.from_pretrained(model_name_or_path))

    def __getattr__(self, name: str):
        return getattr(self.__dict__["original_config"], name)


LLMConfig = LLMConfigWrapper


class LLaVAConfigWrapper(LLMConfigWrapper):
    def __init__(self, config):
        super().__init__(config)
        vis = getattr(config, "vision_config", None)
        get = (lambda k, d: vis.get(k, d)) if isinstance(vis, dict) else (lambda k, d: getattr(vis, k, d))
        self.vision_config = {"hidden_size": get("hidden_size", 1024), "num_hidden_layers": get("num_hidden_layers", 24),
                              "num_attention_heads": get("num_attention_heads", 16),
                              "intermediate_size": get("intermediate_size", 4096),
                              "image_size": get("image_size", 336), "patch_size": get("patch_size", 14)}
        self.mm_hidden_size = self.hidden_size


def _as_wrapper(config, cls=LLMConfigWrapper):
    if isinstance(config, LLMConfigWrapper):
        return config
    if isinstance(config, str):
        return cls.from_pretrained(config)
    return cls(config)


def _stats(cost: PhaseCost, batch: int, seq: int, write_bytes: float) -> ComputeStats:
    w = min(write_bytes, cost.bytes)
    return ComputeStats(cost.flops, cost.bytes - w, w, batch, seq)


