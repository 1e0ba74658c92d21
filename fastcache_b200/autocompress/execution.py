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


_STREAMS: Optional[StreamManager] = None


def get_stream_manager() -> StreamManager:
    global _STREAMS
    if _STREAMS is None:
        _STREAMS = StreamManager()
    return _STREAMS
