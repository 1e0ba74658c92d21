"""Offline planner: workload + method -> ExecutionPlan.

Parity: nanovllm/autocompress/scheduler.py:33-503 (SchedulerConfig,
AutoCompressScheduler.schedule / schedule_multi / analyze, fallback checks,
`auto_schedule`, `analyze_compression`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from .context import HardwareProfile, WorkloadContext, detect_hardware
from .cost_model import CostModel
from .execution import (ChunkingConfig, ExecutionPlan, ExecutionTiming, ParallelismConfig, ParallelismMode)
from .profiles import ComputeType, get_profile


@dataclass
class SchedulerConfig:
    min_speedup: float = 1.05
    min_seq_len: int = 256
    min_output_len: int = 32
    async_min_batch: int = 4
    max_chunk_layers: int = 8
    enable_async: bool = True
    enable_chunking: bool = True
    enable_greenctx: bool = True
    memory_pressure_override: float = 0.9      # compress regardless of speed-up above this occupancy


class AutoCompressScheduler:
    def __init__(self, hardware: Optional[HardwareProfile] = None, config: Optional[SchedulerConfig] = None,
                 cost_model: Optional[CostModel] = None):
        self.hw = hardware or detect_hardware()
        self.cfg = config or SchedulerConfig()
        self.cost = cost_model or CostModel(self.hw)

    def schedule(self, method: str, w: WorkloadContext, **method_kw) -> ExecutionPlan:
        p = get_profile(method)
        cfg = self.cfg
        plan = ExecutionPlan(method=method, chunking=ChunkingConfig(num_layers=w.num_layers))
        forced = w.memory_pressure >= cfg.memory_pressure_override
        if not forced and (w.seq_len < cfg.min_seq_len or w.expected_output_len < cfg.min_output_len):
            plan.should_compress = False
            plan.reason = "sequence or expected output too short"
            return plan.build_steps()
        mem_bound = self.hw.is_decode_memory_bound(w.batch_size, w.seq_len, w.num_layers, w.num_kv_heads,
                                                   w.head_dim, w.hidden_size)
        if p.requires_attention:
            plan.timing = ExecutionTiming.INLINE_PREFILL
        elif cfg.enable_async and p.can_overlap_with_decode(mem_bound) and w.batch_size >= cfg.async_min_batch:
            plan.timing = ExecutionTiming.ASYNC_DECODE
        else:
            plan.timing = ExecutionTiming.AFTER_PREFILL
        overlap = 0.0
        if plan.timing is ExecutionTiming.ASYNC_DECODE:
            overlap = 0.8 * p.decode_compatibility
            plan.parallelism = ParallelismConfig(
                ParallelismMode.ASYNC_STREAM, 1,
                (0.4 if p.compute_type is ComputeType.GEMM else 0.2) if cfg.enable_greenctx else 0.0)
            if cfg.enable_chunking and p.chunkable:
                t_c = self.cost.compress_latency_ms(p, w)
                t_d = max(self.cost.decode_latency_ms(w), 1e-3)
                per_layer = t_c / max(1, w.num_layers)
                layers = int(max(p.min_chunk_size, min(cfg.max_chunk_layers, p.max_chunk_size,
                                                       round(t_d / max(per_layer, 1e-6)))))
                plan.chunking = ChunkingConfig(True, w.num_layers, max(1, layers))
        plan.estimated_compress_ms = self.cost.compress_latency_ms(p, w)
        plan.estimated_speedup = self.cost.compute_speedup(method, w, overlap, **method_kw)
        if plan.estimated_speedup < cfg.min_speedup and not forced:
            plan.should_compress = False
            plan.reason = f"predicted speed-up {plan.estimated_speedup:.3f} below {cfg.min_speedup}"
        else:
            plan.reason = "memory pressure" if forced and plan.estimated_speedup < cfg.min_speedup else "predicted gain"
        return plan.build_steps()

    def schedule_multi(self, methods: List[str], w: WorkloadContext) -> ExecutionPlan:
        plans = [self.schedule(m, w) for m in methods]
        good = [p for p in plans if p.should_compress]
        if not good:
            return plans[0] if plans else ExecutionPlan(should_compress=False).build_steps()
        return max(good, key=lambda p: p.estimated_speedup)

    def analyze(self, method: str, w: WorkloadContext) -> Dict[str, float]:
        p = get_profile(method)
        return {
            "decode_ms": self.cost.decode_latency_ms(w),
            "decode_ms_compressed": self.cost.decode_latency_ms(w, p.get_output_seq_len(w.seq_len)),
            "compress_ms": self.cost.compress_latency_ms(p, w),
            "speedup_sync": self.cost.compute_speedup(method, w, 0.0),
            "speedup_overlapped": self.cost.compute_speedup(method, w, 0.8 * p.decode_compatibility),
            "break_even_output_len": float(self.cost.get_break_even_output_len(method, w)),
            "kv_mb": w.kv_cache_size_mb,
            "kv_mb_compressed": w.estimate_compressed_kv_size_mb(p.compression_ratio),
        }


def auto_schedule(method: str, batch_size: int, seq_len: int, expected_output_len: int = 128, **kw) -> ExecutionPlan:
    w = WorkloadContext(batch_size=batch_size, seq_len=seq_len, expected_output_len=expected_output_len, **kw)
    return AutoCompressScheduler().schedule(method, w)


def analyze_compression(method: str, batch_size: int, seq_len: int, expected_output_len: int = 128, **kw):
    w = WorkloadContext(batch_size=batch_size, seq_len=seq_len, expected_output_len=expected_output_len, **kw)
    return AutoCompressScheduler().analyze(method, w)
