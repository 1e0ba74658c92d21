"""Host-side race detector for the paged KV pool: which stream may touch which block, and after what.

The engine launches work that reads and rewrites pool blocks on several CUDA streams (model steps on the main
stream, compression on side streams, possibly on another SM partition).  Nothing on the device checks that a
kernel which reads a block was ordered after the kernel that last wrote it; a missing `wait_event` shows up as
rare wrong tokens.  This module keeps the happens-before relation on the host instead, with one vector clock per
stream:

  * `launch(stream, reads, writes)`   a kernel (or a batch of them) is enqueued on `stream`; it is checked against
                                       the earlier writes (for reads) and the earlier writes and reads (for
                                       writes) of the rows of every block it names
  * `record(event, stream)`           the event carries the stream's clock
  * `wait(stream, event)`             the stream's clock absorbs the event's
  * `wait_stream(stream, other)`      the same for `stream.wait_stream(other)`
  * `synchronize()`                   everything enqueued so far is ordered before everything that follows

A launch that is not ordered after a conflicting earlier one raises `StreamOrderError` (or is collected in
`violations` with `raise_on_violation=False`).  Streams and events are identified by `id()`, so the CUDA objects
themselves, or any stand-ins on a machine without a GPU, can be passed.  The engine drives it when it is built
with `check_streams=True` (or `FC_CHECK_STREAMS=1`); it costs a Python loop over the touched blocks per launch
and is meant for tests and debugging, like the block manager's `check_invariants`.

The reference has no counterpart: it serialises compression with the step loop or relies on stream semantics
unchecked (`nanovllm/engine/llava_engine.py`, `nanovllm/utils/streams.py`).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple, Union


class StreamOrderError(RuntimeError):
    pass


Clock = Dict[int, int]
Access = Union[int, Tuple[int, int, int]]
_WHOLE = 1 << 62


def _merge(into: Clock, other: Clock) -> None:
    for k, v in other.items():
        if into.get(k, 0) < v:
            into[k] = v


class StreamOrderChecker:
    def __init__(self, raise_on_violation: bool = True):
        self.raise_on_violation = raise_on_violation
        self.violations: List[str] = []
        self.launches = 0
        self._clock: Dict[int, Clock] = {}                 # stream -> what it is ordered after
        self._names: Dict[int, str] = {}
        self._events: Dict[int, Tuple[object, Clock]] = {}  # id(event) -> (event kept alive, clock at record time)
        self._floor: Clock = {}                            # ordered before everything (host synchronisation)
        # block -> accesses that a later launch can still conflict with: (write?, stream, tick, first row, end row, what)
        self._hist: Dict[int, List[Tuple[bool, int, int, int, int, str]]] = {}

    # ------------------------------------------------------------------ bookkeeping
    def _key(self, stream) -> int:
        k = 0 if stream is None else id(stream)
        if k not in self._clock:
            self._clock[k] = {}
            self._names[k] = "default" if stream is None else f"stream#{len(self._names)}"
        return k

    def name_stream(self, stream, name: str) -> None:
        self._names[self._key(stream)] = name

    def _knows(self, s: int, other: int, tick: int) -> bool:
        if other == s:
            return True                                    # one stream runs in order
        return max(self._clock[s].get(other, 0), self._floor.get(other, 0)) >= tick

    def _violation(self, msg: str) -> None:
        self.violations.append(msg)
        if self.raise_on_violation:
            raise StreamOrderError(msg)

    # ------------------------------------------------------------------ the four operations
    def launch(self, stream, reads: Iterable[Access] = (), writes: Iterable[Access] = (),
               what: str = "kernel") -> None:
        """`reads` / `writes`: block ids, or (block, first row, end row) for a part of a block."""
        s = self._key(stream)
        tick = self._clock[s].get(s, 0) + 1
        self._clock[s][s] = tick
        self.launches += 1
        for is_write, items in ((False, reads), (True, writes)):
            for item in items:
                b, lo, hi = (item, 0, _WHOLE) if isinstance(item, int) else item
                if hi <= lo:
                    continue
                kept = []
                for rec in self._hist.get(b, ()):
                    r_write, r_s, r_tick, r_lo, r_hi, r_what = rec
                    overlap = r_lo < hi and lo < r_hi
                    if overlap and (is_write or r_write) and not self._knows(s, r_s, r_tick):
                        self._violation(
                            f"{what} on {self._names[s]} {'writes' if is_write else 'reads'} rows [{lo}, "
                            f"{min(hi, 1 << 30)}) of block {b} without being ordered after {r_what} on "
                            f"{self._names[r_s]}, which {'writes' if r_write else 'reads'} rows [{r_lo}, "
                            f"{min(r_hi, 1 << 30)})")
                    # an earlier access inside this one is superseded when whoever is ordered after this launch
                    # is ordered after it too: same stream, or a write that was just checked against it
                    inside = lo <= r_lo and r_hi <= hi
                    if inside and (r_s == s or is_write) and (is_write or not r_write):
                        continue
                    kept.append(rec)
                kept.append((is_write, s, tick, lo, hi, what))
                self._hist[b] = kept

    def record(self, event, stream) -> None:
        s = self._key(stream)
        clock = dict(self._clock[s])
        self._events[id(event)] = (event, clock)

    def wait(self, stream, event) -> None:
        s = self._key(stream)
        entry = self._events.get(id(event))
        if entry is None:
            self._violation(f"{self._names[s]} waits for an event that was never recorded")
            return
        _merge(self._clock[s], entry[1])

    def wait_stream(self, stream, other) -> None:
        s, o = self._key(stream), self._key(other)
        _merge(self._clock[s], self._clock[o])

    def synchronize(self, stream=None) -> None:
        """The host waited for `stream` (None: the whole device)."""
        if stream is None:
            for c in self._clock.values():
                _merge(self._floor, c)
        else:
            _merge(self._floor, self._clock[self._key(stream)])
        if len(self._events) > 4096:                        # events older than a synchronisation carry nothing new
            self._events.clear()

    def forget_blocks(self, blocks: Optional[Iterable[int]] = None) -> None:
        """Drop the history of `blocks` (all of them for None), e.g. after the pool was rebuilt."""
        if blocks is None:
            self._hist.clear()
            return
        for b in blocks:
            self._hist.pop(b, None)
