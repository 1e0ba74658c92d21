"""Hardware and workload descriptions for the planning code.

Parity: nanovllm/autocompress/context.py:16-380 (GPUArch, HardwareProfile with a
roofline knee and decode-latency estimate, WorkloadContext, a GPU table and
`detect_hardware`).  The table here has a Blackwell entry (the reference labels
every device with compute capability >= 9.0 as Hopper and guesses its bandwidth),
and `detect_hardware` prefers measured peaks from a `MEASURED_PEAKS.json` file when
one is given.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from enum import Enum
from typing import Dict, Optional


class GPUArch(Enum):
    UNKNOWN = "unknown"
    VOLTA = "volta"
    AMPERE = "ampere"
    ADA = "ada"
    HOPPER = "hopper"
    BLACKWELL = "blackwell"


@dataclass
class HardwareProfile:
    gpu_name: str = "Unknown"
    gpu_arch: GPUArch = GPUArch.UNKNOWN
    compute_capability: tuple = (0, 0)
    fp16_tflops: float = 0.0               # dense tensor throughput (bf16/fp16)
    memory_bandwidth_gbps: float = 0.0     # GB/s
    memory_size_gb: float = 0.0
    sm_count: int = 0
    max_threads_per_sm: int = 2048
    l2_mb: float = 0.0
    nvlink_gbps: float = 0.0               # per direction per GPU
    _roofline_intensity: Optional[float] = None

    @property
    def roofline_intensity(self) -> float:
        """FLOP per byte at which a kernel turns compute-bound."""
        if self._roofline_intensity is not None:
            return self._roofline_intensity
        if self.memory_bandwidth_gbps <= 0:
            return 150.0
        return self.fp16_tflops * 1e12 / (self.memory_bandwidth_gbps * 1e9)

    def decode_bytes(self, batch_size: int, seq_len: int, num_layers: int, num_kv_heads: int, head_dim: int,
                     hidden_size: int, dtype_bytes: int = 2, weight_bytes: Optional[float] = None) -> float:
        kv = 2.0 * batch_size * seq_len * num_layers * num_kv_heads * head_dim * dtype_bytes
        if weight_bytes is None:
            weight_bytes = 12.0 * num_layers * hidden_size * hidden_size * dtype_bytes
        return kv + weight_bytes

    def is_decode_memory_bound(self, batch_size: int, seq_len: int, num_layers: int = 32, num_kv_heads: int = 8,
                               head_dim: int = 128, hidden_size: int = 4096) -> bool:
        flops = 2.0 * batch_size * 12.0 * num_layers * hidden_size * hidden_size
        byts = self.decode_bytes(batch_size, seq_len, num_layers, num_kv_heads, head_dim, hidden_size)
        return flops / max(byts, 1.0) < self.roofline_intensity

    def estimate_decode_latency_ms(self, batch_size: int, seq_len: int, num_layers: int = 32,
                                   num_kv_heads: int = 8, head_dim: int = 128, hidden_size: int = 4096) -> float:
        flops = 2.0 * batch_size * 12.0 * num_layers * hidden_size * hidden_size
        byts = self.decode_bytes(batch_size, seq_len, num_layers, num_kv_heads, head_dim, hidden_size)
        t_mem = byts / max(self.memory_bandwidth_gbps * 1e9, 1.0)
        t_cmp = flops / max(self.fp16_tflops * 1e12, 1.0)
        return max(t_mem, t_cmp) * 1e3


@dataclass
class WorkloadContext:
    batch_size: int = 1
    seq_len: int = 512
    expected_output_len: int = 100
    num_layers: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    hidden_size: int = 4096
    memory_used_gb: float = 0.0
    memory_total_gb: float = 0.0
    avg_output_len: Optional[float] = None
    avg_decode_latency_ms: Optional[float] = None

    @property
    def memory_pressure(self) -> float:
        return self.memory_used_gb / self.memory_total_gb if self.memory_total_gb > 0 else 0.0

    @property
    def kv_cache_size_mb(self) -> float:
        return 2.0 * self.batch_size * self.seq_len * self.num_layers * self.num_kv_heads * self.head_dim * 2 / 2 ** 20

    def estimate_compressed_kv_size_mb(self, compression_ratio: float) -> float:
        return self.kv_cache_size_mb / max(compression_ratio, 1.0)

    def get_total_decode_time_ms(self, decode_latency_per_token_ms: float) -> float:
        n = self.avg_output_len if self.avg_output_len is not None else self.expected_output_len
        return n * decode_latency_per_token_ms


_TABLE: Dict[str, HardwareProfile] = {
    "B200": HardwareProfile("NVIDIA B200", GPUArch.BLACKWELL, (10, 0), 2250.0, 7700.0, 180.0, 148, 2048, 126.0, 900.0),
    "H100": HardwareProfile("NVIDIA H100", GPUArch.HOPPER, (9, 0), 989.0, 3350.0, 80.0, 132, 2048, 50.0, 450.0),
    "H200": HardwareProfile("NVIDIA H200", GPUArch.HOPPER, (9, 0), 989.0, 4800.0, 141.0, 132, 2048, 50.0, 450.0),
    "A100": HardwareProfile("NVIDIA A100", GPUArch.AMPERE, (8, 0), 312.0, 2039.0, 80.0, 108, 2048, 40.0, 300.0),
    "A100-40GB": HardwareProfile("NVIDIA A100 40GB", GPUArch.AMPERE, (8, 0), 312.0, 1555.0, 40.0, 108, 2048, 40.0, 300.0),
    "RTX4090": HardwareProfile("RTX 4090", GPUArch.ADA, (8, 9), 330.0, 1008.0, 24.0, 128, 1536, 72.0, 0.0),
    "RTX4080": HardwareProfile("RTX 4080", GPUArch.ADA, (8, 9), 195.0, 717.0, 16.0, 76, 1536, 64.0, 0.0),
    "RTX3090": HardwareProfile("RTX 3090", GPUArch.AMPERE, (8, 6), 142.0, 936.0, 24.0, 82, 1536, 6.0, 0.0),
    "V100": HardwareProfile("V100", GPUArch.VOLTA, (7, 0), 125.0, 900.0, 32.0, 80, 2048, 6.0, 150.0),
}


def get_hardware_profile(name: Optional[str] = None) -> HardwareProfile:
    if name is None:
        return detect_hardware()
    key = name.upper().replace("NVIDIA ", "").replace(" ", "")
    for k, v in _TABLE.items():
        if k.replace("-", "") in key.replace("-", ""):
            return v
    raise KeyError(f"no hardware profile for {name!r}; have {sorted(_TABLE)}")


def _apply_measured(profile: HardwareProfile, path: Optional[str]) -> HardwareProfile:
    if not path or not os.path.exists(path):
        return profile
    try:
        d = json.load(open(path))
        return HardwareProfile(**{**profile.__dict__, "memory_bandwidth_gbps": float(d["hbm_gbs"]),
                                  "fp16_tflops": float(d["bf16_tflops"])})
    except Exception:
        return profile


def detect_hardware(measured_peaks: Optional[str] = None) -> HardwareProfile:
    """Profile of the current CUDA device (a generic estimate on unknown parts, a B200 profile
    when no device is visible so that planning code can run on a CPU box)."""
    try:
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(torch.cuda.current_device())
            try:
                prof = get_hardware_profile(p.name)
            except KeyError:
                cc = (p.major, p.minor)
                arch = (GPUArch.BLACKWELL if cc[0] >= 10 else GPUArch.HOPPER if cc[0] == 9 else
                        GPUArch.ADA if cc == (8, 9) else GPUArch.AMPERE if cc[0] == 8 else GPUArch.VOLTA)
                # clock * SMs * 1024 dense fp16 FMA-pairs per SM per clock on Ampere-class tensor cores
                tf = p.multi_processor_count * 1024 * 2 * 1.5e9 / 1e12
                prof = HardwareProfile(p.name, arch, cc, tf, 25.0 * p.total_memory / 2 ** 30,
                                       p.total_memory / 2 ** 30, p.multi_processor_count)
            prof = HardwareProfile(**{**prof.__dict__, "sm_count": p.multi_processor_count,
                                      "memory_size_gb": p.total_memory / 2 ** 30})
            return _apply_measured(prof, measured_peaks)
    except Exception:
        pass
    return _apply_measured(_TABLE["B200"], measured_peaks)
