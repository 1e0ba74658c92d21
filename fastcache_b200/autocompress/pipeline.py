"""Pipeline orchestration: which strategy runs a method (or a composition of methods).

Parity: nanovllm/autocompress/pipeline.py:44-667 — PipelineStrategy, per-method rules
(the MLP merge goes beside decode when the batch is at least 4 and decode is
memory-bound, or at least 8 regardless), chunk sizes, composed pipelines ordered
MEMORY -> MIXED -> GEMM with a diminishing-returns exponent of 0.8, `execute` hooks and
`analyze_all_methods`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Any, Callable, Dict, List, Optional

from .context import HardwareProfile, WorkloadContext, detect_hardware
from .cost_model import CostModel
from .execution import ExecutionTiming
from .methods import CompressionMethod, get_method
from .profiles import ComputeType, get_profile, list_profiles


class PipelineStrategy(Enum):
    INLINE_PREFILL = auto()
    SYNC_AFTER_PREFILL = auto()
    ASYNC_WITH_DECODE = auto()
    PROGRESSIVE = auto()
    COMPOSED = auto()


@dataclass
class PipelineConfig:
    method: str
    strategy: PipelineStrategy
    timing: ExecutionTiming
    chunk_size: int = 0                      # layers per chunk (0 = whole model at once)
    num_streams: int = 1
    estimated_speedup: float = 1.0
    estimated_compress_ms: float = 0.0
    compression_ratio: float = 1.0
    reason: str = ""
    method_kwargs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ComposedPipelineConfig:
    stages: List[PipelineConfig]
    total_compression_ratio: float
    estimated_speedup: float
    strategy: PipelineStrategy = PipelineStrategy.COMPOSED


_ORDER = {ComputeType.MEMORY: 0, ComputeType.MIXED: 1, ComputeType.GEMM: 2}


class PipelineOrchestrator:
    def __init__(self, hardware: Optional[HardwareProfile] = None, min_speedup: float = 1.05):
        self.hw = hardware or detect_hardware()
        self.cost = CostModel(self.hw)
        self.min_speedup = min_speedup

    def create_pipeline(self, method: str, w: WorkloadContext, **method_kw) -> PipelineConfig:
        p = get_profile(method)
        ratio = method_kw.get("compression_ratio")
        if ratio is not None:
            from .cost_model import _with_ratio
            p = _with_ratio(p, ratio)
        mem_bound = self.hw.is_decode_memory_bound(w.batch_size, w.seq_len, w.num_layers, w.num_kv_heads,
                                                   w.head_dim, w.hidden_size)
        chunk = 0
        if p.requires_attention:
            strategy, timing, overlap = PipelineStrategy.INLINE_PREFILL, ExecutionTiming.INLINE_PREFILL, 0.0
        elif p.compute_type is ComputeType.GEMM and ((w.batch_size >= 4 and mem_bound) or w.batch_size >= 8):
            strategy, timing = PipelineStrategy.ASYNC_WITH_DECODE, ExecutionTiming.ASYNC_DECODE
            overlap = 0.8 * p.decode_compatibility
            if p.chunkable:
                t_layer = self.cost.compress_latency_ms(p, w) / max(1, w.num_layers)
                t_dec = max(self.cost.decode_latency_ms(w), 1e-3)
                chunk = int(max(p.min_chunk_size, min(p.max_chunk_size, round(t_dec / max(t_layer, 1e-6)))))
        elif p.compute_type is ComputeType.MEMORY and p.chunkable and w.seq_len >= 8192:
            strategy, timing, overlap = PipelineStrategy.PROGRESSIVE, ExecutionTiming.AFTER_PREFILL, 0.3
            chunk = p.max_chunk_size
        else:
            strategy, timing, overlap = PipelineStrategy.SYNC_AFTER_PREFILL, ExecutionTiming.AFTER_PREFILL, 0.0
        speedup = self.cost.compute_speedup(method, w, overlap, **({"compression_ratio": ratio} if ratio else {}))
        return PipelineConfig(method, strategy, timing, chunk, 2 if strategy is PipelineStrategy.ASYNC_WITH_DECODE
                              else 1, speedup, self.cost.compress_latency_ms(p, w), p.compression_ratio,
                              "decode is memory-bound: GEMM work hides under it" if strategy is
                              PipelineStrategy.ASYNC_WITH_DECODE else strategy.name.lower(), dict(method_kw))

    def create_composed_pipeline(self, methods: List[str], w: WorkloadContext) -> ComposedPipelineConfig:
        ordered = sorted(methods, key=lambda m: _ORDER[get_profile(m).compute_type])
        stages: List[PipelineConfig] = []
        cur = WorkloadContext(**w.__dict__)
        total_ratio, speedup = 1.0, 1.0
        for i, m in enumerate(ordered):
            cfg = self.create_pipeline(m, cur)
            stages.append(cfg)
            r = cfg.compression_ratio if get_profile(m).modifies_seq_len else 1.0
            total_ratio *= r
            speedup *= max(1.0, cfg.estimated_speedup) ** (0.8 ** i)      # diminishing returns per stage
            cur = WorkloadContext(**{**cur.__dict__, "seq_len": max(1, int(cur.seq_len / r))})
        return ComposedPipelineConfig(stages, total_ratio, speedup)

    # --------------------------------------------------------------- execution
    def execute(self, cfg: PipelineConfig, kv_cache, method: Optional[CompressionMethod] = None,
                on_chunk: Optional[Callable[[int, int], None]] = None, **ctx):
        """Run `cfg` on HF-format tensors.  Chunked strategies call `on_chunk(first_layer, last_layer)`
        between layer groups (the engine interleaves decode steps there)."""
        m = method or get_method(cfg.method, **cfg.method_kwargs)
        if cfg.chunk_size <= 0 or len(kv_cache) <= cfg.chunk_size:
            return m.compress(kv_cache, **ctx)
        out = []
        for a in range(0, len(kv_cache), cfg.chunk_size):
            b = min(len(kv_cache), a + cfg.chunk_size)
            out.extend(self._compress_layers(m, kv_cache, a, b, **ctx))
            if on_chunk is not None:
                on_chunk(a, b)
        return out

    @staticmethod
    def _compress_layers(m: CompressionMethod, kv_cache, a: int, b: int, **ctx):
        comp = getattr(m, "compressor", None)
        if comp is not None and hasattr(comp, "compress_layer_kv"):
            img = int(ctx.get("it_len", (0, 0))[0])
            return [comp.compress_layer_kv(k, v, l, img) for l, (k, v) in zip(range(a, b), kv_cache[a:b])]
        return m.compress(kv_cache[a:b], **ctx)

    def execute_composed(self, cfg: ComposedPipelineConfig, kv_cache, methods: Optional[Dict[str, Any]] = None, **ctx):
        for stage in cfg.stages:
            m = (methods or {}).get(stage.method)
            kv_cache = self.execute(stage, kv_cache, m, **ctx)
        return kv_cache


def create_optimal_pipeline(method: str, batch_size: int, seq_len: int, expected_output_len: int = 128, **kw
                            ) -> PipelineConfig:
    w = WorkloadContext(batch_size=batch_size, seq_len=seq_len, expected_output_len=expected_output_len,
                        **{k: v for k, v in kw.items() if k in WorkloadContext.__dataclass_fields__})
    return PipelineOrchestrator().create_pipeline(method, w)


def analyze_all_methods(w: WorkloadContext, hardware: Optional[HardwareProfile] = None) -> Dict[str, PipelineConfig]:
    o = PipelineOrchestrator(hardware)
    return {m: o.create_pipeline(m, w) for m in list_profiles()}
