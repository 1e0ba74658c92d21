"""Tracing of the engine loop: NVTX ranges per phase and a per-step trace with device times.

The reference marks one phase with NVTX (`utils_ccm/../llava_testcon2.6.py:1204`, "prefill_processing"), times
engine steps with CUDA events every `auto_tune_interval` steps (`nanovllm/engine/llava_engine.py:359-386`) and
keeps named wall-clock timers (`utils_ccm/utils_compress.py:414-475`).  Here:

* `nvtx_range(name)` wraps a phase ("prefill", "decode", "compress", "compress_chunk") in an NVTX range when
  ranges are switched on (`enable_nvtx()` or the environment variable FC_NVTX=1), so `ncu --nvtx-include` and
  other NVTX-aware tools can select the launches of one phase.  Off, it costs one attribute test.
* `StepTrace` records one entry per engine step: kind, batch, tokens, pool state, host time and (on a GPU) a
  pair of CUDA events on the engine's stream.  The events are only read when the trace is exported, so recording
  never synchronises the loop.  `to_chrome_trace()` gives the JSON that chrome://tracing and Perfetto read.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional

import torch

_NVTX = os.environ.get("FC_NVTX", "0") not in ("", "0")


def enable_nvtx(on: bool = True) -> None:
    global _NVTX
    _NVTX = bool(on)


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


@dataclass
class StepRecord:
    step: int
    kind: str                      # "prefill" | "decode"
    num_seqs: int
    tokens: int                    # prompt tokens of a prefill step, batch size of a decode step
    free_blocks: int
    total_blocks: int
    compressions: int              # compressions finished so far
    host_start: float              # perf_counter seconds
    host_ms: float = 0.0
    device_ms: Optional[float] = None
    _events: Any = field(default=None, repr=False)

    @property
    def pool_occupancy(self) -> float:
        return 1.0 - self.free_blocks / max(1, self.total_blocks)


class StepTrace:
    """Bounded per-step trace of an engine (`LLMEngine.enable_trace()`)."""

    def __init__(self, capacity: int = 4096, device_timing: bool = True):
        self.records: Deque[StepRecord] = deque(maxlen=int(capacity))
        self.device_timing = bool(device_timing) and torch.cuda.is_available()
        self._t0 = time.perf_counter()

    # -- recording (called by the engine) ---------------------------------------------------------------
    def begin(self, step: int, kind: str, num_seqs: int, tokens: int, free_blocks: int, total_blocks: int,
              compressions: int, stream=None) -> StepRecord:
        rec = StepRecord(step, kind, num_seqs, tokens, free_blocks, total_blocks, compressions, time.perf_counter())
        if self.device_timing:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream) if stream is not None else a.record()
            rec._events = (a, b)
        return rec

    def end(self, rec: StepRecord, stream=None) -> None:
        if rec._events is not None:
            b = rec._events[1]
            b.record(stream) if stream is not None else b.record()
        rec.host_ms = (time.perf_counter() - rec.host_start) * 1e3
        self.records.append(rec)

    # -- export -------------------------------------------------------------------------------------
    def resolve(self) -> None:
        """Reads the device times (waits for the recorded events)."""
        for rec in self.records:
            if rec._events is not None:
                a, b = rec._events
                b.synchronize()
                rec.device_ms = a.elapsed_time(b)
                rec._events = None

    def summary(self) -> Dict[str, Any]:
        self.resolve()
        out: Dict[str, Any] = {"steps": len(self.records)}
        for kind in ("prefill", "decode"):
            rs = [r for r in self.records if r.kind == kind]
            if not rs:
                continue
            host = sum(r.host_ms for r in rs)
            dev = [r.device_ms for r in rs if r.device_ms is not None]
            out[kind] = {"steps": len(rs), "tokens": sum(r.tokens for r in rs), "host_ms": round(host, 3),
                         "device_ms": round(sum(dev), 3) if dev else None,
                         "max_pool_occupancy": round(max(r.pool_occupancy for r in rs), 4)}
        return out

    def to_chrome_trace(self) -> List[Dict[str, Any]]:
        """Events in the Trace Event format: one complete ("X") event per step on a host row and, when device times
        were recorded, one on a device row (placed at the host start of the step)."""
        self.resolve()
        ev: List[Dict[str, Any]] = []
        for r in self.records:
            ts = (r.host_start - self._t0) * 1e6
            args = {"step": r.step, "seqs": r.num_seqs, "tokens": r.tokens, "free_blocks": r.free_blocks,
                    "pool_occupancy": round(r.pool_occupancy, 4), "compressions": r.compressions}
            ev.append({"name": r.kind, "ph": "X", "pid": 0, "tid": 0, "ts": ts, "dur": r.host_ms * 1e3, "args": args})
            if r.device_ms is not None:
                ev.append({"name": r.kind, "ph": "X", "pid": 0, "tid": 1, "ts": ts, "dur": r.device_ms * 1e3,
                           "args": args})
        ev.append({"name": "thread_name", "ph": "M", "pid": 0, "tid": 0, "args": {"name": "host (engine step)"}})
        ev.append({"name": "thread_name", "ph": "M", "pid": 0, "tid": 1, "args": {"name": "device (CUDA events)"}})
        return ev

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"traceEvents": self.to_chrome_trace(), "summary": self.summary()}, f)
