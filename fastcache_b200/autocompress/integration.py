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

    is_ready = is_done

    def get_result(self) -> Any:
        """The result if the work has finished, else None (never blocks)."""
        return self._result if self.is_done() else None

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

    # argument-style interface of the reference (integration.py:93-210)
    def get_plan(self, batch_size: int, seq_len: int, expected_output_len: int = 100, num_layers: int = 32,
                 num_kv_heads: int = 8, head_dim: int = 128) -> ExecutionPlan:
        return self.plan(WorkloadContext(batch_size=batch_size, seq_len=seq_len,
                                         expected_output_len=expected_output_len, num_layers=num_layers,
                                         num_kv_heads=num_kv_heads, head_dim=head_dim))

    def should_compress(self, batch_size: int, seq_len: int, expected_output_len: int = 100) -> bool:
        plan = self.get_plan(batch_size, seq_len, expected_output_len)
        return plan.should_compress and plan.estimated_speedup >= self.config.min_speedup

    def execute_sync(self, kv_cache, compressor: Any = None, **kwargs):
        """Run `compressor` (default: this manager's method) on the current stream."""
        fn = compressor if compressor is not None else self.method.compress
        self.stats["compressed"] += 1
        return fn(kv_cache, **kwargs)

    def execute_async(self, kv_cache, compressor: Any = None, chunk_size: int = 4,
                      callback: Optional[Callable[[Any], None]] = None, **kwargs) -> AsyncCompressionHandle:
        """Queue the compression on the compression stream; `callback(result)` runs on the host once
        the work is queued (the device-side completion is what `wait()` joins).  `chunk_size` is taken
        for callers that pass it: layer chunking belongs to the engine's decode pipeline."""
        fn = compressor if compressor is not None else self.method.compress

        def work():
            out = fn(kv_cache, **kwargs)
            if callback is not None:
                callback(out)
            return out

        self.stats["compressed"] += 1
        return AsyncCompressionHandle(work, get_stream_manager().compress).start()

    def get_statistics(self) -> Dict[str, Any]:
        out: Dict[str, Any] = dict(self.stats)
        out["method"] = self.config.method
        if self.last_plan is not None:
            out["last_speedup"] = self.last_plan.estimated_speedup
            out["last_timing"] = self.last_plan.timing.name
        return out


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

    def compress(self, kv_cache, batch_size: Optional[int] = None, seq_len: Optional[int] = None,
                 expected_output_len: int = 100, **kwargs):
        """Same decision with the workload stated by the caller (sizes default to the cache's)."""
        k0 = kv_cache[0][0]
        w = WorkloadContext(batch_size=batch_size or k0.shape[0], seq_len=seq_len or k0.shape[2],
                            expected_output_len=expected_output_len, num_layers=len(kv_cache),
                            num_kv_heads=k0.shape[1], head_dim=k0.shape[3],
                            **{k: v for k, v in self.defaults.items() if k != "expected_output_len"})
        out, _ = self.manager.maybe_compress(kv_cache, w, **kwargs)
        return out

    def get_last_plan(self) -> Optional[ExecutionPlan]:
        return self.manager.last_plan


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
