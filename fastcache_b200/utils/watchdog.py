"""Host-side failure detection: step deadline, rank heartbeats, device status codes.

The reference has no such subsystem: a rank that stops answering hangs every other
rank in its next NCCL collective, and its only defences are try/except fallbacks
(nanovllm/engine/llava_model_runner.py:150-153, :555-565).  Here

  * every device-side wait on a flag or barrier is bounded and leaves a code in a
    status word instead of hanging (`DeviceWaitTimeout` carries that code),
  * `StepWatchdog` arms a deadline around each engine step on a helper thread,
  * `RankHeartbeat` publishes a per-rank counter in a `torch.distributed` store
    and reports peers whose counter stopped moving, so the survivors learn of a
    dead rank on the host *before* they launch the next collective,
  * `LLMEngine.recover()` drops the step in flight and requeues its requests.

Nothing here touches a GPU; all of it is exercised with CPU (gloo) ranks.
"""
from __future__ import annotations

import threading
import time
from contextlib import contextmanager
from typing import Callable, Dict, List, Optional

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free pipeline stage",
    3: "timeout waiting for an accumulator",
    4: "timeout waiting for the epilogue",
    5: "timeout waiting for a flag written by another GPU",
    6: "block-table or slot index out of range (access skipped)",
    7: "timeout at a grid barrier inside a kernel",
}


class DeviceWaitTimeout(RuntimeError):
    """A kernel gave up on a bounded wait (or skipped a bad index) and returned."""

    def __init__(self, code: int):
        self.code = int(code)
        super().__init__(f"device status {self.code}: {STATUS_NAMES.get(self.code & 0xFF, 'unknown')}")


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], age_s: float):
        self.ranks = list(ranks)
        super().__init__(f"no heartbeat from rank(s) {self.ranks} for {age_s:.1f} s")


class StepDeadlineExceeded(RuntimeError):
    pass


class StepWatchdog:
    """Deadline around a unit of work.

        wd = StepWatchdog(deadline_s=30, on_expire=abort_fn)
        with wd.step("decode"):
            engine.step()

    If the block has not finished `deadline_s` after it was entered, `on_expire(label, elapsed)`
    runs on the watchdog thread (typically: abort the process group so that a collective
    returns with an error) and leaving the block raises `StepDeadlineExceeded`."""

    def __init__(self, deadline_s: float, on_expire: Optional[Callable[[str, float], None]] = None,
                 poll_s: float = 0.01):
        self.deadline_s = float(deadline_s)
        self.on_expire = on_expire
        self.poll_s = poll_s
        self.expired: List[str] = []
        self._lock = threading.Lock()
        self._armed: Optional[tuple] = None        # (label, t_start, token)
        self._token = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="fc-step-watchdog", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            with self._lock:
                armed = self._armed
            if armed is None:
                continue
            label, t0, token = armed
            elapsed = time.monotonic() - t0
            if elapsed < self.deadline_s:
                continue
            with self._lock:
                if self._armed is None or self._armed[2] != token:
                    continue
                self._armed = None
                self.expired.append(label)
            if self.on_expire is not None:
                try:
                    self.on_expire(label, elapsed)
                except Exception:          # the callback must not kill the watchdog
                    pass

    @contextmanager
    def step(self, label: str = "step"):
        with self._lock:
            self._token += 1
            token = self._token
            self._armed = (label, time.monotonic(), token)
            n_before = len(self.expired)
        try:
            yield self
        finally:
            with self._lock:
                if self._armed is not None and self._armed[2] == token:
                    self._armed = None
                fired = len(self.expired) > n_before
        if fired:
            raise StepDeadlineExceeded(f"{label} exceeded its {self.deadline_s} s deadline")

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=1.0)


class RankHeartbeat:
    """Per-rank liveness counter in a `torch.distributed` store (TCPStore, FileStore, HashStore).

    Every rank runs a thread that bumps `hb/<rank>` each `period_s`.  `dead_ranks()` returns the
    peers whose counter has not changed for `timeout_s` (measured on the caller's clock, so no
    clock agreement between hosts is needed); `check()` raises `RankFailure` for them.  A rank
    that leaves on purpose calls `leave()` first, which marks it gone immediately."""

    def __init__(self, store, rank: int, world_size: int, period_s: float = 0.2, timeout_s: float = 2.0,
                 autostart: bool = True):
        self.store, self.rank, self.world = store, int(rank), int(world_size)
        self.period_s, self.timeout_s = period_s, timeout_s
        self._seen: Dict[int, tuple] = {}           # rank -> (counter, local time it last changed)
        self._stop = threading.Event()
        self._paused = threading.Event()            # fault injection: stop beating without leaving
        self._count = 0
        self._thread: Optional[threading.Thread] = None
        self.beat()
        if autostart:
            self.start()

    def _key(self, r: int) -> str:
        return f"hb/{r}"

    def beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def start(self) -> None:
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name=f"fc-heartbeat-{self.rank}", daemon=True)
            self._thread.start()

    def _run(self) -> None:
        while not self._stop.wait(self.period_s):
            if not self._paused.is_set():
                try:
                    self.beat()
                except Exception:          # the store went away with the rank that hosted it
                    return

    def pause(self) -> None:
        """Stop beating while the process stays alive (what a hung rank looks like)."""
        self._paused.set()

    def resume(self) -> None:
        self._paused.clear()

    def leave(self) -> None:
        self._stop.set()
        try:
            self.store.set(self._key(self.rank), "gone")
        except Exception:
            pass

    def _read(self, r: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return self.store.get(self._key(r)).decode()
        except Exception:
            return None

    def dead_ranks(self) -> List[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == "gone":
                dead.append(r)
                continue
            prev = self._seen.get(r)
            if prev is None or prev[0] != v:
                self._seen[r] = (v, now)
                continue
            if now - prev[1] > self.timeout_s:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead, self.timeout_s)

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
