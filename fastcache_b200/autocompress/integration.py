"""Glue between the planning code and an engine or a bare compressor.

Parity: nanovllm/autocompress/integration.py:28-501 — CompressionConfig,
AutoCompressManager (decide + run), AsyncCompressionHandle (really asynchronous here:
the work is queued on a side stream and `wait()` joins it), AdaptiveCompressionWrapper
and `analyze_workload`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .context import HardwareProfile, WorkloadContext, detect_hardware
from .execution import ExecutionPlan, get_stream_manager
from .methods import CompressionMethod, get_method
from .scheduler import AutoCompressScheduler, SchedulerConfig


@dataclass
class CompressionConfig:
    method: str = "mlp"
    compression_ratio: float = 4.0
    min_speedup: float = 1.05
    enable_async: bool = True
    enable_chunking: bool = True
    force: bool = False


class AsyncCompressionHandle:
    def __init__(self, fn: Callable[[], Any], stream: Any = None):
        self._fn, self._stream = fn, stream
        self._result: Any = None
        self._event: Any = None
        self._started = False

    def start(self) -> "AsyncCompressionHandle":
        self._started = True
        if self._stream is None:
            self._result = self._fn()
            return self
        import torch
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            self._result = self._fn()
            self._event = torch.cuda.Event()
            self._event.record(self._stream)
        return self

    def is_done(self) -> bool:
        return self._started and (self._event is None or self._event.query())

    def wait(self) -> Any:
        if not self._started:
            self.start()
        if self._event is not None:
            import torch
            torch.cuda.current_stream().wait_event(self._event)
        return self._result


class AutoCompressManager:
    def __init__(self, config: Optional[CompressionConfig] = None, hardware: Optional[HardwareProfile] = None,
                 method: Optional[CompressionMethod] = None, **method_kw):
        self.config = config or CompressionConfig()
        self.hw = hardware or detect_hardware()
        self.scheduler = AutoCompressScheduler(self.hw, SchedulerConfig(
            min_speedup=self.config.min_speedup, enable_async=self.config.enable_async,
            enable_chunking=self.config.enable_chunking))
        self.method = method or get_method(self.config.method, **method_kw)
        self.last_plan: Optional[ExecutionPlan] = None
        self.stats = {"decisions": 0, "compressed": 0, "skipped": 0}

    def plan(self, w: WorkloadContext) -> ExecutionPlan:
        plan = self.scheduler.schedule(self.config.method, w, compression_ratio=self.config.compression_ratio)
        if self.config.force:
            plan.should_compress = True
        self.last_plan = plan
        self.stats["decisions"] += 1
        return plan

    def maybe_compress(self, kv_cache, w: WorkloadContext, **ctx):
        plan = self.plan(w)
        if not plan.should_compress:
            self.stats["skipped"] += 1
            return kv_cache, plan
        self.stats["compressed"] += 1
        return self.method.compress(kv_cache, **ctx), plan

    def compress_async(self, kv_cache, **ctx) -> AsyncCompressionHandle:
        sm = get_stream_manager()
        return AsyncCompressionHandle(lambda: self.method.compress(kv_cache, **ctx), sm.compress).start()


class AdaptiveCompressionWrapper:
    """Wraps a compressor callable: compresses only when the plan predicts a gain."""

    def __init__(self, compressor: Any, manager: Optional[AutoCompressManager] = None, **workload_defaults):
        self.compressor = compressor
        self.manager = manager or AutoCompressManager(CompressionConfig(), method=_Callable(compressor))
        self.defaults = workload_defaults

    def __call__(self, kv_cache, it_len=(0, 0), **kw):
        k0 = kv_cache[0][0]
        w = WorkloadContext(batch_size=k0.shape[0], seq_len=k0.shape[2], num_layers=len(kv_cache),
                            num_kv_heads=k0.shape[1], head_dim=k0.shape[3], **self.defaults)
        out, _ = self.manager.maybe_compress(kv_cache, w, it_len=it_len, **kw)
        return out


class _Callable(CompressionMethod):
    name = "callable"

    def __init__(self, fn):
        super().__init__(None)
        self.fn = fn

    def compress(self, kv_cache, **ctx):
        return self.fn(kv_cache, **{k: v for k, v in ctx.items() if k == "it_len"})


def create_auto_compress_manager(method: str = "mlp", **kw) -> AutoCompressManager:
    cfg_keys = CompressionConfig.__dataclass_fields__
    cfg = CompressionConfig(method=method, **{k: v for k, v in kw.items() if k in cfg_keys})
    return AutoCompressManager(cfg, **{k: v for k, v in kw.items() if k not in cfg_keys})


def wrap_compressor(compressor: Any, **kw) -> AdaptiveCompressionWrapper:
    return AdaptiveCompressionWrapper(compressor, **kw)


def analyze_workload(batch_size: int, seq_len: int, expected_output_len: int = 128, method: str = "mlp", **kw
                     ) -> Dict[str, float]:
    w = WorkloadContext(batch_size=batch_size, seq_len=seq_len, expected_output_len=expected_output_len,
                        **{k: v for k, v in kw.items() if k in WorkloadContext.__dataclass_fields__})
    return AutoCompressScheduler().analyze(method, w)
