"""Execution plans: the ordered steps a compression decision turns into.

Parity: nanovllm/autocompress/execution.py:20-500 (ExecutionPlan / ExecutionStep /
StepType, timing and parallelism enums, ChunkingConfig, a callback-driven
PipelineExecutor and a StreamManager with a main and a low-priority stream).
ChunkingConfig takes the layer count from the plan instead of assuming 32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Any, Callable, Dict, List, Optional


class ExecutionTiming(Enum):
    INLINE_PREFILL = auto()     # inside the prefill step (needs attention weights)
    AFTER_PREFILL = auto()      # right after prefill, before the first decode
    ASYNC_DECODE = auto()       # overlapped with decode steps


class ParallelismMode(Enum):
    SYNC = auto()
    ASYNC_STREAM = auto()
    FUSED = auto()


class StepType(Enum):
    PREFILL = auto()
    COMPRESS = auto()
    COMPRESS_CHUNK = auto()
    DECODE = auto()
    SYNC = auto()
    FREE_BLOCKS = auto()


@dataclass
class ParallelismConfig:
    mode: ParallelismMode = ParallelismMode.SYNC
    num_streams: int = 1
    sm_fraction: float = 0.0        # share of SMs given to compression (green context), 0 = shared


@dataclass
class ChunkingConfig:
    enabled: bool = False
    num_layers: int = 32
    layers_per_chunk: int = 4

    @property
    def num_chunks(self) -> int:
        return -(-self.num_layers // max(1, self.layers_per_chunk)) if self.enabled else 1

    def get_layers(self, chunk: int) -> range:
        if not self.enabled:
            return range(self.num_layers)
        a = chunk * self.layers_per_chunk
        return range(a, min(self.num_layers, a + self.layers_per_chunk))

    @classmethod
    def create(cls, num_layers: int = 32, chunk_size: int = 4, interleave: bool = True) -> "ChunkingConfig":
        """Chunked compression of `num_layers` layers, `chunk_size` per step.  `interleave` (decode
        steps between chunks) is how chunked plans are always built here; the flag is accepted for
        callers that pass it."""
        return cls(True, int(num_layers), max(1, int(chunk_size)))

    @property
    def chunk_size(self) -> int:
        return self.layers_per_chunk


@dataclass
class ExecutionStep:
    type: StepType
    name: str = ""
    stream: str = "main"
    chunk: int = -1
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ExecutionPlan:
    method: str = "none"
    timing: ExecutionTiming = ExecutionTiming.AFTER_PREFILL
    parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
    chunking: ChunkingConfig = field(default_factory=ChunkingConfig)
    steps: List[ExecutionStep] = field(default_factory=list)
    should_compress: bool = True
    estimated_speedup: float = 1.0
    estimated_compress_ms: float = 0.0
    reason: str = ""
    estimated_total_time_ms: float = 0.0
    warnings: List[str] = field(default_factory=list)
    debug_info: Dict[str, Any] = field(default_factory=dict)

    @property
    def estimated_compress_latency_ms(self) -> float:
        return self.estimated_compress_ms

    def add_step(self, step: ExecutionStep) -> None:
        self.steps.append(step)

    def add_warning(self, warning: str) -> None:
        self.warnings.append(warning)

    def is_valid(self) -> bool:
        return len(self.steps) > 0 and self.estimated_speedup >= 1.0

    def to_schedule(self) -> List[ExecutionStep]:
        return list(self.steps)

    def summary(self) -> str:
        lines = [f"ExecutionPlan for '{self.method}'",
                 f"  timing       {self.timing.name}",
                 f"  parallelism  {self.parallelism.mode.name} ({self.parallelism.num_streams} stream(s), "
                 f"SM share {self.parallelism.sm_fraction:.2f})",
                 f"  chunking     " + (f"{self.chunking.num_chunks} x {self.chunking.layers_per_chunk} layers"
                                       if self.chunking.enabled else "off"),
                 f"  speedup      {self.estimated_speedup:.2f}x, compression {self.estimated_compress_ms:.2f} ms",
                 f"  steps        " + " -> ".join(st.name or st.type.name for st in self.steps)]
        lines += [f"  warning      {w}" for w in self.warnings]
        if self.reason:
            lines.append(f"  reason       {self.reason}")
        return "\n".join(lines)

    # factories for the four plan shapes (reference execution.py:174-300)
    @classmethod
    def create_sync_plan(cls, method: str, compress_latency_ms: float, speedup: float) -> "ExecutionPlan":
        return cls(method, ExecutionTiming.AFTER_PREFILL, ParallelismConfig(ParallelismMode.SYNC),
                   ChunkingConfig(False), estimated_speedup=speedup,
                   estimated_compress_ms=compress_latency_ms).build_steps()

    @classmethod
    def create_async_plan(cls, method: str, compress_latency_ms: float, speedup: float, chunk_size: int = 4,
                          num_layers: int = 32) -> "ExecutionPlan":
        return cls(method, ExecutionTiming.ASYNC_DECODE, ParallelismConfig(ParallelismMode.ASYNC_STREAM, 1),
                   ChunkingConfig.create(num_layers, chunk_size), estimated_speedup=speedup,
                   estimated_compress_ms=compress_latency_ms).build_steps()

    @classmethod
    def create_inline_plan(cls, method: str, compress_latency_ms: float, speedup: float) -> "ExecutionPlan":
        plan = cls(method, ExecutionTiming.INLINE_PREFILL, ParallelismConfig(ParallelismMode.FUSED),
                   ChunkingConfig(False), estimated_speedup=speedup, estimated_compress_ms=compress_latency_ms)
        # the scores come out of the prefill pass itself; selection and compaction follow on the same stream
        plan.steps = [ExecutionStep(StepType.PREFILL, "prefill+scores", params={"fusion_point": "after_attention"}),
                      ExecutionStep(StepType.COMPRESS, "select+compact"),
                      ExecutionStep(StepType.FREE_BLOCKS, "free"), ExecutionStep(StepType.DECODE, "decode")]
        return plan

    @classmethod
    def create_no_compress_plan(cls) -> "ExecutionPlan":
        return cls("none", should_compress=False, reason="compression not worthwhile").build_steps()

    def build_steps(self) -> "ExecutionPlan":
        s: List[ExecutionStep] = [ExecutionStep(StepType.PREFILL, "prefill")]
        if not self.should_compress:
            s.append(ExecutionStep(StepType.DECODE, "decode"))
        elif self.timing is ExecutionTiming.ASYNC_DECODE and self.chunking.enabled:
            for c in range(self.chunking.num_chunks):
                s.append(ExecutionStep(StepType.DECODE, f"decode[{c}]"))
                s.append(ExecutionStep(StepType.COMPRESS_CHUNK, f"compress[{c}]", "compress", c,
                                       {"layers": list(self.chunking.get_layers(c))}))
            s += [ExecutionStep(StepType.SYNC, "join"), ExecutionStep(StepType.FREE_BLOCKS, "free"),
                  ExecutionStep(StepType.DECODE, "decode")]
        else:
            stream = "compress" if self.parallelism.mode is ParallelismMode.ASYNC_STREAM else "main"
            s.append(ExecutionStep(StepType.COMPRESS, "compress", stream))
            if stream == "compress":
                s.append(ExecutionStep(StepType.SYNC, "join"))
            s += [ExecutionStep(StepType.FREE_BLOCKS, "free"), ExecutionStep(StepType.DECODE, "decode")]
        self.steps = s
        return self


class PipelineExecutor:
    """Walks a plan and calls the handler registered for each step type."""

    def __init__(self) -> None:
        self.handlers: Dict[StepType, Callable[[ExecutionStep], Any]] = {}
        self.trace: List[str] = []

    def on(self, step_type: StepType, fn: Callable[[ExecutionStep], Any]) -> "PipelineExecutor":
        self.handlers[step_type] = fn
        return self

    def run(self, plan: ExecutionPlan) -> List[Any]:
        if not plan.steps:
            plan.build_steps()
        out = []
        for step in plan.steps:
            self.trace.append(step.name)
            fn = self.handlers.get(step.type)
            out.append(fn(step) if fn is not None else None)
        return out

    # step-at-a-time interface (reference execution.py:327-436)
    def register_callback(self, step_type: StepType, callback: Callable[[ExecutionStep], Any]) -> None:
        self.on(step_type, callback)

    def set_plan(self, plan: ExecutionPlan) -> None:
        if not plan.steps:
            plan.build_steps()
        self._plan, self._cursor = plan, 0
        self._latencies_ms: List[float] = []
        self._warnings: List[str] = list(plan.warnings)

    def execute_step(self, step: ExecutionStep) -> bool:
        """Run one step's handler; a handler that raises is recorded as a warning and reported as False."""
        import time
        t0 = time.perf_counter()
        self.trace.append(step.name)
        ok = True
        try:
            fn = self.handlers.get(step.type)
            if fn is not None:
                fn(step)
        except Exception as exc:
            ok = False
            self.__dict__.setdefault("_warnings", []).append(f"{step.name or step.type.name}: {exc}")
        self.__dict__.setdefault("_latencies_ms", []).append((time.perf_counter() - t0) * 1e3)
        return ok

    def execute_all(self) -> bool:
        plan = getattr(self, "_plan", None)
        if plan is None:
            raise RuntimeError("set_plan() first")
        ok = True
        while self._cursor < len(plan.steps):
            ok = self.execute_step(plan.steps[self._cursor]) and ok
            self._cursor += 1
        return ok

    def get_statistics(self) -> Dict[str, Any]:
        lat = self.__dict__.get("_latencies_ms", [])
        return {"total_steps": len(lat), "total_time_ms": sum(lat), "avg_step_time_ms": sum(lat) / max(len(lat), 1),
                "warnings": list(self.__dict__.get("_warnings", []))}


class StreamManager:
    """Main stream plus a lower-priority compression stream (None on CPU)."""

    def __init__(self, device: Optional[Any] = None) -> None:
        self.main = self.compress = None
        try:
            import torch
            if torch.cuda.is_available():
                self.main = torch.cuda.current_stream(device)
                self.compress = torch.cuda.Stream(device=device, priority=0)
        except Exception:
            pass

    def get(self, name: str):
        return self.compress if name == "compress" else self.main

    def join(self) -> None:
        if self.main is not None and self.compress is not None:
            self.main.wait_stream(self.compress)

    # names of the reference's manager (execution.py:450-492); streams are made in the constructor here
    def initialize(self) -> None:
        if self.main is None and self.compress is None:
            self.__init__()

    def get_main_stream(self):
        return self.main

    def get_compress_stream(self):
        return self.compress

    synchronize_compress_to_main = join


_STREAMS: Optional[StreamManager] = None


def get_stream_manager() -> StreamManager:
    global _STREAMS
    if _STREAMS is None:
        _STREAMS = StreamManager()
    return _STREAMS
