"""Concurrent serving harness: arrival process, three-stage batching, per-request timing.

Parity with the reference's HuggingFace-based harness:
  * request structs and life cycle            utils_ccm/utils_requests.py:7-127
  * TimestampManager (9 stage timestamps -> queue / process times, TTFT = prefill finish -
    prefill queueing start, TPOT = decode time / generated length, latency, normalised
    latency)                                   utils_ccm/utils_schedule_v11.py:27-193
  * GPUMonitor (sampling thread, CSV)          utils_ccm/utils_schedule_v11.py:196-310
  * DynamicScheduler (prefill and decode priority queues; shorter first with ageing toward
    max_wait_time; prefill goes first but waits for a full batch or max_wait_time; decode batch =
    longest prefix whose cumulative size fits the decode cap)
                                               utils_ccm/utils_schedule_v11.py:431-803
  * KVCachePool (request id -> per-layer (K, V), store / get / release / merge_and_pop / pop)
                                               utils_ccm/utils_kvcachePool.py:22-394
  * ImprovedConcurrentTester, PerformanceMonitor, TestResult (collector + dispatcher threads,
    p50 / p90 / p99, throughput)               scripts/llava_testcon2.6.py:100-222, :385-1695
`ConcurrentTester` drives this package's engine (the HuggingFace-model form of the pipeline, with the
pool and the dynamic scheduler in the loop, is `serving/hf_pipeline.py`).  The engine's
scheduler already has the prefill / compress / decode queues with their batch caps, so this
tester supplies the arrival process, the per-stage batching rule for the caps, timing and
reporting.
"""
from __future__ import annotations

import heapq
import random
import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------ requests
class RequestStatus(Enum):
    PENDING = "pending"
    PREFILLING = "prefilling"
    COMPRESSING = "compressing"
    DECODING = "decoding"
    COMPLETED = "completed"
    FAILED = "failed"


@dataclass
class RequestMetrics:
    arrival: float = 0.0
    prefill_start: float = 0.0
    prefill_end: float = 0.0
    compress_start: float = 0.0
    compress_end: float = 0.0
    decode_start: float = 0.0
    decode_end: float = 0.0
    generated: int = 0
    # life-cycle stamps of the reference's request struct (utils_ccm/utils_requests.py:17-46)
    create_time: float = 0.0
    queue_time: float = 0.0
    start_time: float = 0.0
    complete_time: float = 0.0

    @property
    def wait_time(self) -> float:
        return self.start_time - self.queue_time if self.start_time > 0 else 0.0

    @property
    def prefill_time(self) -> float:
        return self.prefill_end - self.prefill_start if self.prefill_end > 0 else 0.0

    @property
    def decode_time(self) -> float:
        return self.decode_end - self.decode_start if self.decode_end > 0 else 0.0

    @property
    def total_time(self) -> float:
        return self.complete_time - self.create_time if self.complete_time > 0 else 0.0

    @property
    def ttft(self) -> float:
        return self.prefill_end - self.arrival

    @property
    def tpot(self) -> float:
        return (self.decode_end - self.decode_start) / max(1, self.generated)

    @property
    def latency(self) -> float:
        return self.decode_end - self.arrival


@dataclass
class Request:
    request_id: int
    prompt: Any
    max_tokens: int = 64
    image: Any = None
    status: RequestStatus = RequestStatus.PENDING
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    output: List[int] = field(default_factory=list)
    error: Optional[str] = None

    @property
    def input_len(self) -> int:
        return len(self.prompt) if not isinstance(self.prompt, str) else len(self.prompt.split())

    def fail(self, why: Any) -> None:
        self.status, self.error = RequestStatus.FAILED, str(why)
        self.metrics.complete_time = time.time()

    # life-cycle transitions (utils_ccm/utils_requests.py:64-100)
    def __post_init__(self) -> None:
        self.batch_id: Optional[int] = None
        self.result: Any = None
        if not self.metrics.create_time:
            self.metrics.create_time = time.time()

    def enter_queue(self) -> None:
        self.status = RequestStatus.PENDING
        self.metrics.queue_time = time.time()

    def start_processing(self) -> None:
        self.metrics.start_time = time.time()

    def start_prefill(self) -> None:
        self.status = RequestStatus.PREFILLING
        self.metrics.prefill_start = time.time()

    def end_prefill(self) -> None:
        self.metrics.prefill_end = time.time()

    def start_decode(self) -> None:
        self.status = RequestStatus.DECODING
        self.metrics.decode_start = time.time()

    def end_decode(self) -> None:
        self.metrics.decode_end = time.time()

    def complete(self, result: Any = None) -> None:
        self.status, self.result = RequestStatus.COMPLETED, result
        self.metrics.complete_time = time.time()

    def to_dict(self) -> dict:
        m = self.metrics
        return {"request_id": self.request_id, "batch_id": self.batch_id, "status": self.status.value,
                "metrics": {"create_time": m.create_time, "queue_time": m.queue_time, "start_time": m.start_time,
                            "wait_time": m.wait_time, "prefill_time": m.prefill_time,
                            "decode_time": m.decode_time, "total_time": m.total_time},
                "error": self.error}


@dataclass(order=True)
class PrioritizedRequest:
    priority: float
    seq: int
    request: Any = field(compare=False)


PriorityRequest = PrioritizedRequest


# ---------------------------------------------------------------------- timestamps
class TimestampManager:
    STAGES = ("arrival", "prefill_queueing_start", "prefill_start", "prefill_finish", "compress_queueing_start",
              "compress_start", "compress_finish", "decoding_queueing_start", "decoding_start", "decoding_finish")

    def __init__(self) -> None:
        self._t: Dict[int, Dict[str, float]] = {}
        self._lock = threading.Lock()

    def record(self, request_id: int, stage: str, t: Optional[float] = None) -> None:
        with self._lock:
            self._t.setdefault(request_id, {})[stage] = time.perf_counter() if t is None else t

    def get(self, request_id: int) -> Dict[str, float]:
        with self._lock:
            return dict(self._t.get(request_id, {}))

    def analyze(self, request_id: int, generated_len: int = 1) -> Dict[str, float]:
        t = self.get(request_id)

        def span(end: str, *starts: str) -> float:
            """end - first recorded start; 0 when either side was never stamped."""
            if t.get(end) is None:
                return 0.0
            for s0 in starts:
                if t.get(s0) is not None:
                    return t[end] - t[s0]
            return 0.0

        out = {
            "prefill_queue": span("prefill_start", "prefill_queueing_start", "arrival"),
            "prefill_process": span("prefill_finish", "prefill_start"),
            "compress_queue": span("compress_start", "compress_queueing_start", "prefill_finish"),
            "compress_process": span("compress_finish", "compress_start"),
            "decoding_queue": span("decoding_start", "decoding_queueing_start", "prefill_finish"),
            "decoding_process": span("decoding_finish", "decoding_start", "prefill_finish"),
            "ttft": span("prefill_finish", "prefill_queueing_start", "arrival"),
            "latency": span("decoding_finish", "arrival", "prefill_queueing_start"),
        }
        out["tpot"] = out["decoding_process"] / max(1, generated_len)
        out["normalized_latency"] = out["latency"] / max(1, generated_len)
        return out

    # list-of-ids interface of the reference (utils_ccm/utils_schedule_v11.py:35-193); its stage
    # names `compress_queueing`, `decoding_queueing`, `decode_start` map to the names above
    _STAGE_ALIASES = {"compress_queueing": "compress_queueing_start", "decoding_queueing": "decoding_queueing_start",
                      "decode_start": "decoding_start"}

    def create_request(self, request_id_list: Sequence[Any]) -> None:
        with self._lock:
            for rid in request_id_list:
                self._t.setdefault(rid, {})

    def record_timestamp(self, request_id_list: Sequence[Any], stage: str, timestamps: float) -> None:
        stage = self._STAGE_ALIASES.get(stage, stage)
        with self._lock:
            for rid in request_id_list:
                if rid in self._t:
                    self._t[rid][stage] = timestamps

    get_timestamps = get

    def remove_request(self, request_id: Any) -> None:
        with self._lock:
            self._t.pop(request_id, None)

    def calculate_stage_durations(self) -> Dict[str, List[float]]:
        """Per-stage lists over the requests that reached `decoding_finish`."""
        with self._lock:
            ids = [rid for rid, t in self._t.items() if "decoding_finish" in t]
        keys = ("prefill_queue", "prefill_process", "compress_queue", "compress_process", "decoding_queue",
                "decoding_process", "ttft", "tpot", "latency", "normalized_latency")
        out: Dict[str, List[float]] = {k: [] for k in keys}
        out["generated_lens"] = []
        for rid in ids:
            n = int(self.get(rid).get("generated_lens") or 1)
            a = self.analyze(rid, n)
            for k in keys:
                out[k].append(a[k])
            out["generated_lens"].append(n)
        return out

    @staticmethod
    def calculate_average_times(durations: Dict[str, List[float]]) -> Dict[str, float]:
        return {k: (round(sum(v) / len(v), 3) if v else 0) for k, v in durations.items()}

    @staticmethod
    def calculate_generated_lens(durations: Dict[str, List[float]]) -> int:
        return int(sum(durations.get("generated_lens", [])))

    def analyze_timestamps(self) -> Tuple[Dict[str, Any], Dict[str, List[float]]]:
        d = self.calculate_stage_durations()
        return {"average_times": self.calculate_average_times(d),
                "total_generated_lens": self.calculate_generated_lens(d)}, d


# --------------------------------------------------------------------- GPU monitor
class GPUMonitor(threading.Thread):
    """Samples utilisation and memory every `period` seconds, tagged with the current stage."""

    def __init__(self, device_index: int = 0, period: float = 0.05):
        super().__init__(daemon=True)
        self.device_index, self.period = device_index, period
        self.stage = "idle"
        self.samples: List[Dict[str, Any]] = []
        self._halt = threading.Event()

    def run(self) -> None:
        nv = handle = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self.device_index)
        except Exception:
            nv = None
        t0 = time.perf_counter()
        while not self._halt.is_set():
            row: Dict[str, Any] = {"t": time.perf_counter() - t0, "stage": self.stage}
            if nv is not None:
                try:
                    u = nv.nvmlDeviceGetUtilizationRates(handle)
                    m = nv.nvmlDeviceGetMemoryInfo(handle)
                    row.update(gpu_util=u.gpu, mem_util=u.memory, mem_used_gb=m.used / 2 ** 30)
                except Exception:
                    pass
            if torch.cuda.is_available():
                row["torch_allocated_gb"] = torch.cuda.memory_allocated() / 2 ** 30
            self.samples.append(row)
            self._halt.wait(self.period)

    def stop(self) -> List[Dict[str, Any]]:
        self._halt.set()
        self.join(timeout=2)
        return self.samples

    # names of the reference's monitor (utils_ccm/utils_schedule_v11.py:242-306)
    def start_monitoring(self) -> None:
        if not self.is_alive() and not self._halt.is_set():
            self.samples.clear()
            self.start()

    def stop_monitoring(self) -> None:
        if self.is_alive():
            self.stop()

    def set_batch_size(self, batch_size: int) -> None:
        self.batch_size = int(batch_size)

    def accum_state_round(self, state_name: str) -> None:
        """Count one more round of `state_name` (prefill / compress / decoding) and tag samples with it."""
        rounds = self.__dict__.setdefault("state_round", {})
        rounds[state_name] = rounds.get(state_name, 0) + 1
        self.stage = f"{state_name} {rounds[state_name]}"

    def get_state_round_info(self) -> str:
        return self.stage if " " in self.stage else "ready -1"

    def check_gpu_stats(self) -> Dict[str, Any]:
        """The latest sample (empty before the first one)."""
        return dict(self.samples[-1]) if self.samples else {}

    def get_stats(self) -> Dict[str, List[Any]]:
        keys = sorted({k for r in self.samples for k in r})
        return {k: [r.get(k) for r in self.samples] for k in keys}

    def save_stats(self, filename: str) -> None:
        self.to_csv(filename)

    def to_csv(self, path: str) -> None:
        import csv
        keys = sorted({k for r in self.samples for k in r})
        with open(path, "w", newline="") as fh:
            w = csv.DictWriter(fh, fieldnames=keys)
            w.writeheader()
            w.writerows(self.samples)


# -------------------------------------------------------------------- KV cache pool
@dataclass
class KVCacheItem:
    """One request's stored cache with its bookkeeping (utils_ccm/utils_kvcachePool.py:23-30)."""
    request_id: Any
    kv_cache: List[Tuple[torch.Tensor, torch.Tensor]]
    seq_len: int = 0
    created: float = field(default_factory=time.time)


class KVCachePool:
    """Request id -> list of per-layer (K, V) in HF layout [1, H, S, D] (lock protected)."""

    def __init__(self, max_entries: int = 0) -> None:
        self._pool: Dict[int, List[Tuple[torch.Tensor, torch.Tensor]]] = {}
        self._lock = threading.Lock()
        self.max_entries = max_entries
        self.stores = self.releases = 0

    def store_kvcache(self, request_ids: Sequence[int], kv_cache: Sequence[Tuple[torch.Tensor, torch.Tensor]],
                      lengths: Optional[Sequence[int]] = None) -> None:
        """Splits a batch along dim 0 (optionally trimming left padding to `lengths`)."""
        with self._lock:
            for b, rid in enumerate(request_ids):
                entry = []
                for k, v in kv_cache:
                    kb, vb = k[b:b + 1], v[b:b + 1]
                    if lengths is not None:
                        kb, vb = kb[:, :, -lengths[b]:], vb[:, :, -lengths[b]:]
                    entry.append((kb.contiguous(), vb.contiguous()))
                self._pool[rid] = entry
                self.stores += 1

    def get(self, request_id: int):
        with self._lock:
            return self._pool.get(request_id)

    def get_kvcache(self, request_ids):
        """One id -> its entry (or None); a list of ids -> list of entries."""
        if isinstance(request_ids, (list, tuple)):
            return [self.get(r) for r in request_ids]
        return self.get(request_ids)

    def release_kvcache(self, request_ids) -> bool:
        ids = request_ids if isinstance(request_ids, (list, tuple)) else [request_ids]
        return all([self.release(r) for r in ids])

    def pop_kvcache(self, request_id: int):
        with self._lock:
            return self._pool.pop(request_id, None)

    def release(self, request_id: int) -> bool:
        with self._lock:
            self.releases += 1
            return self._pool.pop(request_id, None) is not None

    def clear(self) -> None:
        with self._lock:
            self._pool.clear()

    clear_kvcache = clear

    def merge_and_pop(self, request_ids: Sequence[int]):
        """Concatenate the entries of `request_ids` along the batch dim (left-padding to the longest)."""
        entries = [self.pop_kvcache(r) for r in request_ids]
        entries = [e for e in entries if e is not None]
        if not entries:
            return None, []
        lens = [e[0][0].shape[2] for e in entries]
        S = max(lens)
        merged = []
        for layer in range(len(entries[0])):
            ks, vs = [], []
            for e, n in zip(entries, lens):
                k, v = e[layer]
                if n < S:
                    pad = (0, 0, S - n, 0)
                    k, v = torch.nn.functional.pad(k, pad), torch.nn.functional.pad(v, pad)
                ks.append(k)
                vs.append(v)
            merged.append((torch.cat(ks, 0), torch.cat(vs, 0)))
        return merged, lens

    def get_stats(self) -> Dict[str, Any]:
        with self._lock:
            byts = sum(k.numel() * k.element_size() + v.numel() * v.element_size()
                       for e in self._pool.values() for k, v in e)
            return {"entries": len(self._pool), "bytes": byts, "stores": self.stores, "releases": self.releases}


# ----------------------------------------------------------------- dynamic scheduler
class DynamicScheduler:
    """Two priority queues with the reference's selection rule.

    priority = size * (1 - aged share): shorter requests first, and a request that has waited
    `max_wait_time` gets the top priority.  `select_batch` returns ("prefill" | "decoding", batch):
    prefill wins whenever a prefill is queued, but is held until `max_batch_size` requests are
    queued or `max_wait_time` has passed since the last prefill; a decode batch is the longest prefix
    (in priority order) whose cumulative request sizes stay within `std_batch_threshold_decoding`.
    """

    def __init__(self, max_batch_size: int = 15, std_batch_threshold_decoding: int = 90,
                 max_wait_time: float = 0.5, compress_batch_size: int = 45):
        self.max_batch_size = max_batch_size
        self.std_batch_threshold_decoding = std_batch_threshold_decoding
        self.compress_batch_size = compress_batch_size
        self.max_wait_time = max_wait_time
        self._prefill: List[PrioritizedRequest] = []
        self._decode: List[PrioritizedRequest] = []
        self._n = 0
        self._last_prefill = time.perf_counter()
        self._lock = threading.Lock()
        # kept for interface parity: the reference carries PID gains but leaves the batch size fixed
        self.kp, self.ki, self.kd = 0.5, 0.1, 0.05

    def _priority(self, size: float, arrival: float) -> float:
        waited = time.perf_counter() - arrival
        return size * max(0.0, 1.0 - waited / max(self.max_wait_time, 1e-6))

    def add_prefill(self, request: Any, size: int, arrival: Optional[float] = None) -> None:
        with self._lock:
            self._n += 1
            heapq.heappush(self._prefill, PrioritizedRequest(self._priority(size, arrival or time.perf_counter()),
                                                             self._n, (request, size, arrival or time.perf_counter())))

    def add_decoding(self, request: Any, size: int = 1, arrival: Optional[float] = None) -> None:
        with self._lock:
            self._n += 1
            heapq.heappush(self._decode, PrioritizedRequest(self._priority(size, arrival or time.perf_counter()),
                                                            self._n, (request, size, arrival or time.perf_counter())))

    def qsize(self) -> Tuple[int, int]:
        with self._lock:
            return len(self._prefill), len(self._decode)

    # interface of the reference's scheduler (utils_ccm/utils_schedule_v11.py:532-803)
    def add_request(self, request: Any, request_type: str) -> None:
        """`request.batch` carries the tensors: prefill requests are sized by their prompt length,
        decoding requests by `batch["request_size"]` (how many sequences the group holds)."""
        batch = getattr(request, "batch", None) or {}
        if request_type == "prefill":
            ids = batch.get("input_ids")
            self.add_prefill(request, int(ids.shape[1]) if ids is not None else 1)
        else:
            self.add_decoding(request, int(batch.get("request_size", 1)))

    def update_priorities(self) -> None:
        with self._lock:
            self._reprioritise(self._prefill)
            self._reprioritise(self._decode)

    @staticmethod
    def binary_search_last_le(lst: Sequence[float], x: float) -> int:
        """Index of the last element <= x in an ascending list, -1 if none."""
        import bisect
        return bisect.bisect_right(lst, x) - 1

    def adaptive_batch_size(self, queue_type: str, current_performance: float = 0.0, gpu_stats: Any = None) -> int:
        """Batch cap for the queue.  The reference computes a PID correction and then discards it
        (`new_size = current_size`); the caps are fixed here as well, and the decode cap counts how many
        queued groups fit the decoding threshold."""
        if queue_type == "prefill":
            return self.max_batch_size
        with self._lock:
            sizes = sorted(p.request[1] for p in self._decode)
        total, n = 0, 0
        for sz in sizes:
            if n and total + sz > self.std_batch_threshold_decoding:
                break
            total, n = total + sz, n + 1
        return max(1, n)

    def update_performance(self, metrics: Dict[str, Any]) -> None:
        win = self.__dict__.setdefault("perf_window", [])
        win.append(metrics["batch_size"])
        del win[:-100]

    def get_current_performance(self) -> float:
        win = self.__dict__.get("perf_window") or []
        recent = win[-10:]
        return sum(recent) / len(recent) if recent else 0

    def get_queue_status(self) -> Dict[str, Any]:
        p, d = self.qsize()
        return {"prefill_count": p, "decoding_count": d, "current_mode": self.__dict__.get("current_mode", "prefill")}

    def _reprioritise(self, heap: List[PrioritizedRequest]) -> None:
        items = [PrioritizedRequest(self._priority(p.request[1], p.request[2]), p.seq, p.request) for p in heap]
        heap[:] = items
        heapq.heapify(heap)

    def select_batch(self, now: Optional[float] = None) -> Tuple[Optional[str], List[Any]]:
        now = time.perf_counter() if now is None else now
        with self._lock:
            if self._prefill:
                full = len(self._prefill) >= self.max_batch_size
                waited = now - self._last_prefill >= self.max_wait_time
                if full or waited:
                    self._reprioritise(self._prefill)
                    n = min(self.max_batch_size, len(self._prefill))
                    batch = [heapq.heappop(self._prefill).request[0] for _ in range(n)]
                    self._last_prefill = now
                    self.current_mode = "prefill"
                    return "prefill", batch
                if not self._decode:
                    return None, []
            if self._decode:
                self._reprioritise(self._decode)
                batch, used = [], 0
                while self._decode:
                    size = self._decode[0].request[1]
                    if batch and used + size > self.std_batch_threshold_decoding:
                        break
                    batch.append(heapq.heappop(self._decode).request[0])
                    used += size
                self.current_mode = "decoding"
                return "decoding", batch
        return None, []


# ---------------------------------------------------------------------- monitoring
@dataclass
class TestResult:
    num_requests: int = 0
    completed: int = 0
    failed: int = 0
    wall_s: float = 0.0
    output_tokens: int = 0
    throughput_tok_s: float = 0.0
    request_rate: float = 0.0
    ttft: Dict[str, float] = field(default_factory=dict)
    tpot: Dict[str, float] = field(default_factory=dict)
    latency: Dict[str, float] = field(default_factory=dict)
    compression: Dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.__dict__)


class PerformanceMonitor:
    @staticmethod
    def percentiles(xs: Sequence[float]) -> Dict[str, float]:
        if not xs:
            return {}
        s = sorted(xs)
        pick = lambda q: s[min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))]  # noqa: E731
        return {"mean": sum(s) / len(s), "p50": pick(0.5), "p90": pick(0.9), "p99": pick(0.99), "max": s[-1]}

    # accumulate-then-report interface of the reference's monitor (scripts/llava_testcon2.6.py:100-222):
    # results are filed under "orig" or "comp", one entry per finished batch
    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        blank = lambda: {"latencies": [], "throughputs": [], "memory_usage": [], "request_id": [],  # noqa: E731
                         "request_size": [], "valid_tokens": 0, "success_count": 0, "total_count": 0,
                         "compression_ratios": [], "compression_times": []}
        self.results: Dict[str, Dict[str, Any]] = {"orig": blank(), "comp": blank()}
        self.start_time = time.time()

    def add_result(self, result: Any) -> None:
        """`result`: an object with `method` ("orig" | "comp"), `latency` = (total, ttft, tpot) seconds,
        `throughput`, `memory_usage`, `request_id`, `request_size`, `valid_tokens`, `success`, and for
        "comp" optionally `compression_ratio` / `compression_time`."""
        d = self.results[getattr(result, "method", "orig")]
        for key, attr in (("latencies", "latency"), ("throughputs", "throughput"), ("memory_usage", "memory_usage"),
                          ("request_id", "request_id"), ("request_size", "request_size")):
            d[key].append(getattr(result, attr, 0))
        d["valid_tokens"] += int(getattr(result, "valid_tokens", 0))
        d["success_count"] += int(bool(getattr(result, "success", True)))
        d["total_count"] += 1
        for key, attr in (("compression_ratios", "compression_ratio"), ("compression_times", "compression_time")):
            if getattr(result, attr, None) is not None:
                d[key].append(getattr(result, attr))

    def proc_latencies(self) -> Tuple[List[float], List[float]]:
        """Per-request TTFT and TPOT lists (a batch entry counts once per request in it)."""
        ttft: List[float] = []
        tpot: List[float] = []
        for d in self.results.values():
            for lat, n in zip(d["latencies"], d["request_size"]):
                ttft += [lat[1]] * int(n)
                tpot += [lat[2]] * int(n)
        return ttft, tpot

    def calculate_metrics(self, durations_dict: Optional[Dict[str, List[float]]] = None,
                          system_completion_times: Optional[float] = None) -> Dict[str, Dict[str, float]]:
        """`durations_dict`: {"TTFT": [...], "TPOT": [...]} (default: from the filed results);
        `system_completion_times`: wall seconds of the whole job (default: since `reset`)."""
        if durations_dict is None:
            a, b = self.proc_latencies()
            durations_dict = {"TTFT": a, "TPOT": b}
        wall = system_completion_times if system_completion_times is not None else time.time() - self.start_time
        out: Dict[str, Dict[str, float]] = {}
        for method, d in self.results.items():
            if not d["latencies"] or not durations_dict["TTFT"]:
                continue
            row: Dict[str, float] = {"total_requests": d["total_count"],
                                     "success_rate": 100.0 * d["success_count"] / max(1, d["total_count"]),
                                     "requests_per_second": d["total_count"] / wall if wall > 0 else 0.0}
            for name, xs in (("ttft", durations_dict["TTFT"]), ("tpot", durations_dict["TPOT"])):
                s_ = sorted(xs)
                n = len(s_)
                row.update({f"avg_{name}": sum(s_) / n, f"median_{name}": s_[int(n * 0.5)],
                            f"p90_{name}": s_[int(n * 0.9)], f"p99_{name}": s_[min(int(n * 0.99), n - 1)],
                            f"min_{name}": s_[0], f"max_{name}": s_[-1]})
            mem, thr = d["memory_usage"], d["throughputs"]
            row["avg_memory_usage"] = sum(mem) / max(1, len(mem))
            row["avg_throughput"] = d["valid_tokens"] / (wall + 1e-5)
            mean_thr = sum(thr) / max(1, len(thr))
            row["throughput_stddev"] = (sum((t - mean_thr) ** 2 for t in thr) / (len(thr) - 1)) ** 0.5 \
                if len(thr) > 1 else 0.0
            if method == "comp" and d["compression_ratios"]:
                row["avg_compression_ratio"] = sum(d["compression_ratios"]) / len(d["compression_ratios"])
                ct = d["compression_times"]
                row["avg_compression_time"] = sum(ct) / len(ct) if ct else 0.0
            out[method] = row
        return out

    def summarise(self, requests: Sequence[Request], wall_s: float, rate: float, stats: Any = None) -> TestResult:
        done = [r for r in requests if r.status is RequestStatus.COMPLETED]
        toks = sum(len(r.output) for r in done)
        res = TestResult(len(requests), len(done), sum(r.status is RequestStatus.FAILED for r in requests), wall_s,
                         toks, toks / max(wall_s, 1e-9), rate,
                         self.percentiles([r.metrics.ttft for r in done]),
                         self.percentiles([r.metrics.tpot for r in done]),
                         self.percentiles([r.metrics.latency for r in done]))
        if stats is not None:
            res.compression = {"compressions": stats.compressions, "rows_in": stats.compressed_rows_in,
                               "rows_out": stats.compressed_rows_out, "blocks_freed": stats.blocks_freed,
                               "lazy_triggers": stats.lazy_triggers, "preemptions": stats.preemptions}
        return res


# ---------------------------------------------------------------------------- tester
class ConcurrentTester:
    """Open-loop load test of an engine: arrivals at `req_per_sec` (Poisson by default, fixed
    spacing like the reference with poisson=False), engine steps in the calling thread.

    `batching = [prefill, compress, decode]` sets the per-stage batch caps of the engine's scheduler
    (default [15, 45, 90]; `ccm_intensity_rule(decode)` gives the MiniCPM harness' rule
    compress = decode // 3, prefill = compress // 3).
    """

    def __init__(self, llm: Any, batching: Sequence[int] = (15, 45, 90), req_per_sec: float = 10.0,
                 poisson: bool = True, seed: int = 0, monitor_gpu: bool = False):
        self.llm = llm
        self.rate, self.poisson = req_per_sec, poisson
        self.rng = random.Random(seed)
        sch = llm.scheduler
        sch.prefill_cap, sch.compress_cap, sch.decode_cap = (int(b) for b in batching)
        self.timestamps = TimestampManager()
        self.monitor = GPUMonitor() if monitor_gpu else None
        self.perf = PerformanceMonitor()

    @staticmethod
    def ccm_intensity_rule(decode: int = 135) -> List[int]:
        compress = decode // 3
        return [compress // 3, compress, decode]

    def arrival_times(self, n: int) -> List[float]:
        t, out = 0.0, []
        for _ in range(n):
            out.append(t)
            t += self.rng.expovariate(self.rate) if self.poisson else 1.0 / self.rate
        return out

    def run(self, prompts: Sequence[Any], max_tokens: int = 128, images: Optional[Sequence[Any]] = None,
            temperature: float = 0.0, time_scale: float = 1.0,
            on_step: Optional[Callable[[int], None]] = None,
            agree: Optional[Callable[[int], int]] = None) -> TestResult:
        """`agree(n)`: under tensor parallelism every rank must admit the same requests before the same
        step; each rank passes the number of arrivals it sees as due and gets back rank 0's number."""
        from ..sampling_params import SamplingParams
        llm = self.llm
        reqs = [Request(i, p, max_tokens, images[i] if images else None) for i, p in enumerate(prompts)]
        arrivals = [a * time_scale for a in self.arrival_times(len(reqs))]
        if self.monitor is not None:
            self.monitor.start()
        seq_of: Dict[int, Request] = {}
        nxt, steps = 0, 0
        t0 = time.perf_counter()
        while nxt < len(reqs) or not llm.is_finished():
            now = time.perf_counter() - t0
            due = nxt
            while due < len(reqs) and arrivals[due] <= now:
                due += 1
            if agree is not None:
                due = max(nxt, min(len(reqs), int(agree(due))))
            while nxt < due:
                r = reqs[nxt]
                r.metrics.arrival = t0 + arrivals[nxt]
                self.timestamps.record(r.request_id, "arrival", r.metrics.arrival)
                try:
                    seq = llm.add_request(r.prompt, SamplingParams(temperature=temperature, max_tokens=r.max_tokens,
                                                                   ignore_eos=True), r.image)
                    seq.arrival_time = r.metrics.arrival
                    seq_of[seq.seq_id] = r
                    r.status = RequestStatus.PREFILLING
                    r._seq = seq
                except Exception as exc:
                    r.fail(str(exc))
                nxt += 1
            if llm.is_finished():
                if nxt < len(reqs):
                    time.sleep(max(0.0, min(0.01, arrivals[nxt] - now)))
                continue
            if self.monitor is not None:
                self.monitor.stage = f"step{steps}"
            outputs, _ = llm.step()
            steps += 1
            t = time.perf_counter()
            for sid, toks in outputs:
                r = seq_of.pop(sid, None)
                if r is None:
                    continue
                s = r._seq
                r.output = list(toks)
                r.metrics.prefill_end = s.first_token_time or t
                r.metrics.decode_start = r.metrics.prefill_end
                r.metrics.decode_end = t
                r.metrics.generated = len(toks)
                r.status = RequestStatus.COMPLETED
                self.timestamps.record(r.request_id, "prefill_finish", r.metrics.prefill_end)
                self.timestamps.record(r.request_id, "generated_lens", len(toks))
                self.timestamps.record(r.request_id, "decoding_finish", t)
            if on_step is not None:
                on_step(steps)
        wall = time.perf_counter() - t0
        if self.monitor is not None:
            self.monitor.stop()
        return self.perf.summarise(reqs, wall, self.rate, getattr(llm, "stats", None))


# names used by the reference's scripts
ImprovedConcurrentTester = ConcurrentTester


class ServiceMiddleware:
    """Thin front for the tester: keeps the engine, the tester settings and the last result."""

    def __init__(self, llm: Any, **tester_kwargs: Any):
        self.llm, self.kw = llm, tester_kwargs
        self.last: Optional[TestResult] = None

    def run_concurrent_test(self, prompts: Sequence[Any], **run_kwargs: Any) -> TestResult:
        self.last = ConcurrentTester(self.llm, **self.kw).run(prompts, **run_kwargs)
        return self.last


# ----------------------------------------------------------------------- reporting
def format_metrics(metrics: Dict[str, Dict[str, float]], output_type: str = "print") -> Optional[str]:
    """The `calculate_metrics` table as text (printed, returns None) or as a JSON string."""
    import json
    if output_type == "json":
        return json.dumps(metrics, indent=2)
    lines = ["=== Performance Test Results ==="]
    for method in ("orig", "comp"):
        lines.append(f"--- {method.upper()} ---")
        row = metrics.get(method)
        if not row:
            lines.append("no data")
            continue
        lines.append(f"requests {row['total_requests']}  success {row['success_rate']:.1f} %  "
                     f"{row['requests_per_second']:.2f} req/s  {row['avg_throughput']:.1f} tok/s")
        for name in ("ttft", "tpot"):
            lines.append(f"{name.upper()} (s): avg {row[f'avg_{name}']:.4f}  p50 {row[f'median_{name}']:.4f}  "
                         f"p90 {row[f'p90_{name}']:.4f}  p99 {row[f'p99_{name}']:.4f}  "
                         f"min {row[f'min_{name}']:.4f}  max {row[f'max_{name}']:.4f}")
        if "avg_compression_ratio" in row:
            lines.append(f"compression: ratio {row['avg_compression_ratio']:.2f}  "
                         f"time {row['avg_compression_time']:.4f} s")
    print("\n".join(lines))
    return None


def print_metrics(metrics: Dict[str, Dict[str, float]]) -> None:
    format_metrics(metrics, "print")


def generate_results_txt(metrics: Dict[str, Dict[str, float]], analyze_times_result: Any,
                         system_completion_time: float, system_total_generated_lens: int, comp_mode: str,
                         file_path: str) -> str:
    """Write the run summary the harness scripts keep per run (scripts/llava_testcon2.6.py:2056-2076)."""
    import json
    os_lines = [f"mode: {comp_mode}", format_metrics(metrics, "json") or "",
                "stage times: " + json.dumps(analyze_times_result, default=str),
                f"service completed in {system_completion_time:.2f} s",
                f"service generated {system_total_generated_lens} tokens",
                f"throughput: {system_total_generated_lens / (system_completion_time + 1e-5):.2f} tokens/s"]
    with open(file_path, "w") as fh:
        fh.write("\n".join(os_lines) + "\n")
    return file_path


def print_gpu_memory(step: str) -> float:
    """MiB allocated by torch on the current device (0 without a GPU); prints it with the label."""
    mb = torch.cuda.memory_allocated() / 2 ** 20 if torch.cuda.is_available() else 0.0
    print(f"=== {step} ===\nGPU memory allocated: {mb:.2f} MB")
    return mb


def load_checkpoint_only_model(model: Any, filename: str, device: Any = None) -> Any:
    """Load a compressor `.pth` (any of the three layouts the loaders accept) into `model` in place."""
    from ..compress.ccm import _extract_state
    if device is None:
        device = next(model.parameters()).device
    blob = torch.load(filename, map_location=device, weights_only=False)
    model.load_state_dict(_extract_state(blob), strict=False)
    return model
