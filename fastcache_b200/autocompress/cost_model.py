"""Roofline cost model: is compressing worth it, and with which configuration?

Parity: nanovllm/autocompress/cost_model.py:25-445 (CalibrationData with JSON
save/load, decode-latency model, sync vs async total-time model,
`compute_speedup`, `find_best_config`, `get_break_even_output_len`,
`should_compress`).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Tuple

from .context import HardwareProfile, WorkloadContext, detect_hardware
from .profiles import CompressMethodProfile, ComputeType, get_profile


@dataclass
class CalibrationData:
    """Measured corrections to the analytic model, keyed by GPU name."""
    gpu_name: str = ""
    decode_scale: float = 1.0
    compress_scale: Dict[str, float] = field(default_factory=dict)
    samples: int = 0
    # raw measurements, keyed "batch,seq_len" and "method,seq_len,batch" (the keys of the
    # reference's JSON file, cost_model.py:45-84); the cost model prefers an exact hit over its formula
    decode_measurements: Dict[str, float] = field(default_factory=dict)
    compress_measurements: Dict[str, float] = field(default_factory=dict)

    def save(self, path: str) -> None:
        with open(path, "w") as fh:
            json.dump(asdict(self), fh, indent=1)

    @classmethod
    def load(cls, path: str) -> "CalibrationData":
        with open(path) as fh:
            blob = json.load(fh)
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in blob.items() if k in known})

    def add_decode_measurement(self, batch_size: int, seq_len: int, latency_ms: float) -> None:
        self.decode_measurements[f"{batch_size},{seq_len}"] = float(latency_ms)

    def add_compress_measurement(self, method: str, seq_len: int, batch_size: int, latency_ms: float) -> None:
        self.compress_measurements[f"{method},{seq_len},{batch_size}"] = float(latency_ms)

    def update_decode(self, predicted_ms: float, measured_ms: float, alpha: float = 0.2) -> None:
        if predicted_ms > 0:
            self.decode_scale = (1 - alpha) * self.decode_scale + alpha * measured_ms / predicted_ms
            self.samples += 1

    def update_compress(self, method: str, predicted_ms: float, measured_ms: float, alpha: float = 0.2) -> None:
        if predicted_ms > 0:
            old = self.compress_scale.get(method, 1.0)
            self.compress_scale[method] = (1 - alpha) * old + alpha * measured_ms / predicted_ms


class CostModel:
    def __init__(self, hardware: Optional[HardwareProfile] = None, calibration: Optional[CalibrationData] = None):
        self.hw = hardware or detect_hardware()
        self.cal = calibration or CalibrationData(gpu_name=self.hw.gpu_name)

    # ------------------------------------------------------------ primitives
    def decode_latency_ms(self, w: WorkloadContext, seq_len: Optional[int] = None) -> float:
        s = w.seq_len if seq_len is None else seq_len
        if w.avg_decode_latency_ms is not None and seq_len is None:
            return w.avg_decode_latency_ms
        hit = self.cal.decode_measurements.get(f"{w.batch_size},{s}")
        if hit is not None:
            return hit
        return self.cal.decode_scale * self.hw.estimate_decode_latency_ms(
            w.batch_size, s, w.num_layers, w.num_kv_heads, w.head_dim, w.hidden_size)

    def compress_latency_ms(self, p: CompressMethodProfile, w: WorkloadContext) -> float:
        """All layers, K and V, whole batch."""
        hit = self.cal.compress_measurements.get(f"{p.name},{w.seq_len},{w.batch_size}")
        if hit is not None:
            return hit
        rows = float(w.batch_size) * w.seq_len * w.num_kv_heads
        units = rows * w.num_layers * 2
        t_mem = units * max(p.bytes_per_row, 2.0 * w.head_dim) / max(self.hw.memory_bandwidth_gbps * 1e9, 1.0)
        t_cmp = units * p.flops_per_row / max(self.hw.fp16_tflops * 1e12 * 0.6, 1.0)
        if p.compute_type is ComputeType.GEMM:
            t = max(t_cmp, t_mem)
        elif p.compute_type is ComputeType.MEMORY:
            t = t_mem
        else:
            t = t_mem + t_cmp
        launch = 0.01 * (1 if p.compute_type is not ComputeType.MIXED else 3)
        return self.cal.compress_scale.get(p.name, 1.0) * (t * 1e3 + launch)

    # names of the reference's model (cost_model.py:172-300)
    def estimate_decode_latency(self, workload: WorkloadContext, compressed: bool = False,
                                compression_ratio: float = 1.0) -> float:
        s = workload.seq_len
        if compressed and compression_ratio > 1.0:
            s = max(1, int(s / compression_ratio))
        return self.decode_latency_ms(workload, s)

    def estimate_compress_latency(self, method: str, workload: WorkloadContext) -> float:
        return self.compress_latency_ms(get_profile(method), workload)

    def estimate_total_time(self, workload: WorkloadContext, method: Optional[str] = None,
                            async_mode: bool = False) -> Tuple[float, Dict[str, float]]:
        """(total ms, breakdown).  Asynchronous compression hides the share of its time that the
        method's profile says can run beside decode."""
        n = int(workload.avg_output_len or workload.expected_output_len)
        if method is None:
            t = self.total_time_ms(None, workload)
            return t, {"compress_ms": 0.0, "decode_ms": t, "output_tokens": n, "overlap": 0.0}
        p = get_profile(method)
        overlap = 0.0
        if async_mode:
            mem_bound = self.hw.is_decode_memory_bound(workload.batch_size, workload.seq_len, workload.num_layers,
                                                       workload.num_kv_heads, workload.head_dim,
                                                       workload.hidden_size)
            overlap = 0.8 * p.decode_compatibility if p.can_overlap_with_decode(mem_bound) else 0.0
        t_c = self.compress_latency_ms(p, workload)
        total = self.total_time_ms(p, workload, overlap)
        return total, {"compress_ms": t_c, "exposed_compress_ms": (1.0 - overlap) * t_c,
                       "decode_ms": total - (1.0 - overlap) * t_c, "output_tokens": n, "overlap": overlap}

    # -------------------------------------------------------------- totals
    def total_time_ms(self, p: Optional[CompressMethodProfile], w: WorkloadContext, overlap: float = 0.0
                      ) -> float:
        """Decode time of `expected_output_len` tokens, plus the part of compression not hidden."""
        n = int(w.avg_output_len or w.expected_output_len)
        if p is None:
            return sum_decode(self, w, w.seq_len, n)
        s_c = p.get_output_seq_len(w.seq_len)
        t_c = self.compress_latency_ms(p, w)
        return (1.0 - overlap) * t_c + sum_decode(self, w, s_c, n)

    def compute_speedup(self, method: str, w: WorkloadContext, overlap: float = 0.0, **kw) -> float:
        p = _with_ratio(get_profile(method), kw.get("compression_ratio"))
        base = self.total_time_ms(None, w)
        return base / max(self.total_time_ms(p, w, overlap), 1e-9)

    def get_break_even_output_len(self, method: str, w: WorkloadContext, **kw) -> int:
        p = _with_ratio(get_profile(method), kw.get("compression_ratio"))
        t_c = self.compress_latency_ms(p, w)
        d0 = self.decode_latency_ms(w, w.seq_len)
        d1 = self.decode_latency_ms(w, p.get_output_seq_len(w.seq_len))
        gain = d0 - d1
        return 10 ** 9 if gain <= 0 else int(t_c / gain) + 1

    def find_best_config(self, methods: List[str], w: WorkloadContext) -> Tuple[Optional[str], float, float]:
        """Returns (method or None, speedup, overlap used)."""
        best: Tuple[Optional[str], float, float] = (None, 1.0, 0.0)
        mem_bound = self.hw.is_decode_memory_bound(w.batch_size, w.seq_len, w.num_layers, w.num_kv_heads,
                                                   w.head_dim, w.hidden_size)
        for m in methods:
            p = get_profile(m)
            overlap = 0.8 * p.decode_compatibility if p.can_overlap_with_decode(mem_bound) else 0.0
            s = self.compute_speedup(m, w, overlap)
            if s > best[1]:
                best = (m, s, overlap)
        return best


def sum_decode(cm: CostModel, w: WorkloadContext, start_len: int, n_tokens: int) -> float:
    """Decode latency grows with the context: integrate with the trapezoid rule."""
    a = cm.decode_latency_ms(w, start_len)
    b = cm.decode_latency_ms(w, start_len + n_tokens)
    return 0.5 * (a + b) * n_tokens


def _with_ratio(p: CompressMethodProfile, ratio: Optional[float]) -> CompressMethodProfile:
    if ratio is None:
        return p
    r = ratio if ratio >= 1.0 else 1.0 / max(1e-6, 1.0 - ratio)     # accepts a drop ratio in (0, 1)
    return CompressMethodProfile(**{**p.__dict__, "compression_ratio": r})


def should_compress(method: str, w: WorkloadContext, min_speedup: float = 1.05,
                    hardware: Optional[HardwareProfile] = None) -> bool:
    return CostModel(hardware).compute_speedup(method, w) >= min_speedup
