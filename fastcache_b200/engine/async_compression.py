"""Per-request view of compressions that run beside the main stream.

The reference keeps a separate manager object with its own side stream, per-request events and a
lock ("kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:43-205: `CompressionState`,
`AsyncCompressionManager`).  Here the engine owns that state (`LLMEngine._pending`, one
`PendingCompression` per request in flight, `Sequence.compression_state`), because the scheduler,
the block manager and the streams have to agree on it; this class is the same surface over the
engine's state, for callers written against the reference's manager.

Differences from the reference, by design:
  * the compressed length is known on the host as soon as the kernels are launched (it is a
    function of the segment lengths), so `get_effective_kv_len` never has to wait on an event;
  * "complete" is decided on the device: the main stream waits for the side stream's event
    before the request's KV is read or its tail blocks are reused, so no host thread polls;
  * `wait_for_compression` honours its limit (the reference accepts `timeout_ms` and ignores
    it, llava_model_runner.py:168-172).
"""
from __future__ import annotations

import threading
import time
from typing import Iterable, List, Optional

from .sequence import CompressionState, Sequence


class AsyncCompressionManager:
    """State machine NONE -> PENDING -> IN_PROGRESS -> COMPLETED per request id."""

    def __init__(self, engine):
        self.engine = engine
        self._lock = threading.Lock()
        self._queued: dict[int, Sequence] = {}

    # ---------------------------------------------------------------- launching
    def start_async_compression(self, seqs: Iterable[Sequence]) -> List[int]:
        """Launch whole-request compression of `seqs` on a compression stream.

        Returns the ids that were launched (requests that are too short, already compressed or
        finished are skipped, as in the engine's own eager/async policies)."""
        eng = self.engine
        todo = [s for s in seqs if eng._eligible(s)]
        with self._lock:
            for s in todo:
                self._queued[s.seq_id] = s      # reads as PENDING until the kernels are queued
        try:
            eng._launch_async(todo)
        finally:
            with self._lock:
                for s in todo:
                    self._queued.pop(s.seq_id, None)
        return [s.seq_id for s in todo]

    # ------------------------------------------------------------------ queries
    def get_state(self, seq_id: int) -> CompressionState:
        with self._lock:
            if seq_id in self._queued:
                return CompressionState.PENDING
        p = self.engine._pending.get(seq_id)
        if p is not None:
            return CompressionState.IN_PROGRESS
        for s in self._live_sequences():
            if s.seq_id == seq_id:
                return s.compression_state
        return CompressionState.NONE

    def is_compression_complete(self, seq_id: int) -> bool:
        """True when nothing of this request's compression is still running on the device."""
        p = self.engine._pending.get(seq_id)
        if p is None:
            return self.get_state(seq_id) is not CompressionState.PENDING
        if p.seq.hold:                          # layer chunks still to launch
            return False
        return p.event is None or bool(p.event.query())

    def wait_for_compression(self, seq_id: int, timeout_ms: float = 1000.0) -> bool:
        """Block the host until the request's compression has finished or the limit runs out.

        A request compressed in layer chunks advances only with engine steps, so waiting on it
        from outside the step loop returns False at the limit instead of spinning for ever."""
        deadline = time.monotonic() + timeout_ms / 1e3
        while not self.is_compression_complete(seq_id):
            if time.monotonic() >= deadline:
                return False
            time.sleep(2e-4)
        return True

    def wait_all_compressions(self, timeout_ms: float = 10000.0) -> bool:
        ok = True
        for sid in list(self.engine._pending):
            ok = self.wait_for_compression(sid, timeout_ms) and ok
        return ok

    def get_effective_kv_len(self, seq: Sequence) -> int:
        """Rows of KV that attention will read for `seq` (the compressed length once launched)."""
        return int(seq.kv_cache_len)

    # ------------------------------------------------------------------ cleanup
    def finalize(self, seqs: Optional[Iterable[Sequence]] = None) -> None:
        """Make the main stream wait for the finished compressions and free their tail blocks."""
        eng = self.engine
        if seqs is None:
            seqs = [p.seq for p in list(eng._pending.values())]
        eng._finalize_pending(list(seqs))

    def cleanup_seq(self, seq_id: int) -> None:
        with self._lock:
            self._queued.pop(seq_id, None)
        self.engine._pending.pop(seq_id, None)

    def _live_sequences(self):
        sch = self.engine.scheduler
        for q in (getattr(sch, "running", ()), getattr(sch, "waiting", ()),
                  getattr(sch, "compress_queue", ())):
            yield from q
