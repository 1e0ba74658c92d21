"""The three-stage serving pipeline over a HuggingFace-style causal LM (the reference's first system).

Parity: scripts/llava_testcon2.6.py:385-1695 (`ImprovedConcurrentTester`): a collector thread feeds
arrivals into the prefill queue of the `DynamicScheduler`, a dispatcher thread picks batches and
runs them on one worker; a prefill batch runs the model once over the left-padded prompts and
parks every request's KV in the `KVCachePool`; a decode batch pops its requests' KV from the pool,
compresses it in chunks of the compress batch size, pads the (now shorter, ragged) caches on the
left, builds the attention mask from the valid lengths and generates.

Differences from the reference, by design:
  * every request is compressed with its own image / text split (the reference applies the split
    of the first request of a merged batch to all of them, llava_testcon2.6.py:656-660);
  * decode is an explicit token loop with position ids taken from the valid lengths, so the
    tokens equal those of serving each request alone (no dependence on `generate()` internals);
  * timing brackets device work with a synchronize (the reference reads a tensor's shape instead,
    llava_testcon2.6.py:577-578).

The model is reached through a small backend object, so the pipeline also runs with any callable
pair `prefill` / `decode_step` (tests use a tiny random Llama on the CPU).
"""
from __future__ import annotations

import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .harness import (DynamicScheduler, GPUMonitor, KVCachePool, PerformanceMonitor, Request, RequestStatus,
                      TestResult, TimestampManager)

KV = List[Tuple[torch.Tensor, torch.Tensor]]


# ------------------------------------------------------------------------ backend
def cache_to_pairs(cache: Any) -> KV:
    """HuggingFace cache object (new `.layers[i].keys/.values`, older `.key_cache`, or legacy tuples) -> pairs."""
    if hasattr(cache, "layers"):
        return [(l.keys, l.values) for l in cache.layers]
    if hasattr(cache, "key_cache"):
        return list(zip(cache.key_cache, cache.value_cache))
    return [(k, v) for k, v in cache]


def pairs_to_cache(pairs: KV) -> Any:
    from transformers import DynamicCache
    cache = DynamicCache()
    for i, (k, v) in enumerate(pairs):
        cache.update(k, v, i)
    return cache


class TransformersBackend:
    """`prefill` and `decode_step` of a HuggingFace causal LM (text path; a multimodal model is used
    through its language model, with `inputs_embeds` prepared by the caller's `embed` hook)."""

    def __init__(self, model: Any, embed: Optional[Callable[[Dict[str, Any]], torch.Tensor]] = None):
        self.model, self.embed = model, embed
        self.device = next(model.parameters()).device

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, attention_mask: torch.Tensor, extra: Optional[Dict[str, Any]] = None
                ) -> Tuple[torch.Tensor, KV]:
        pos = (attention_mask.cumsum(-1) - 1).clamp_min(0)
        kw: Dict[str, Any] = {"attention_mask": attention_mask, "position_ids": pos, "use_cache": True}
        if self.embed is not None and extra:
            kw["inputs_embeds"] = self.embed({"input_ids": input_ids, **extra})
        else:
            kw["input_ids"] = input_ids
        out = self.model(**kw)
        return out.logits[:, -1].float(), [(k, v) for k, v in cache_to_pairs(out.past_key_values)]

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, cache: Any, attention_mask: torch.Tensor,
                    position_ids: torch.Tensor) -> torch.Tensor:
        out = self.model(input_ids=tokens, attention_mask=attention_mask, position_ids=position_ids,
                         past_key_values=cache, use_cache=True)
        return out.logits[:, -1].float()

    def make_cache(self, pairs: KV) -> Any:
        return pairs_to_cache(pairs)


# ------------------------------------------------------------------------ helpers
def left_pad(rows: Sequence[Sequence[int]], pad_id: int, device: Any) -> Tuple[torch.Tensor, torch.Tensor]:
    n = max(len(r) for r in rows)
    ids = torch.full((len(rows), n), pad_id, dtype=torch.long)
    mask = torch.zeros(len(rows), n, dtype=torch.long)
    for i, r in enumerate(rows):
        ids[i, n - len(r):] = torch.as_tensor(list(r), dtype=torch.long)
        mask[i, n - len(r):] = 1
    return ids.to(device), mask.to(device)


def create_attention_mask_from_padding(valid_lens: Sequence[int], total: int, device: Any) -> torch.Tensor:
    """[B, total] mask for left-padded caches: the last `valid_lens[b]` positions of row b are real."""
    ar = torch.arange(total, device=device)[None, :]
    return (ar >= (total - torch.as_tensor(list(valid_lens), device=device)[:, None])).long()


def merge_kv_cache(entries: Sequence[KV]) -> Tuple[KV, List[int]]:
    """Per-request caches [1, H, S_i, D] -> one left-padded batch [B, H, max S, D] and the S_i."""
    lens = [e[0][0].shape[2] for e in entries]
    S = max(lens)
    merged: KV = []
    for layer in range(len(entries[0])):
        ks, vs = [], []
        for e, n in zip(entries, lens):
            k, v = e[layer]
            if n < S:
                k = torch.nn.functional.pad(k, (0, 0, S - n, 0))
                v = torch.nn.functional.pad(v, (0, 0, S - n, 0))
            ks.append(k)
            vs.append(v)
        merged.append((torch.cat(ks, 0), torch.cat(vs, 0)))
    return merged, lens


@dataclass
class _Group:
    """Requests that were prefetched together and wait for decode (`batch` is what the scheduler sizes)."""
    requests: List[Request]
    first_tokens: List[int]
    batch: Dict[str, Any] = field(default_factory=dict)


@dataclass
class _Arrival:
    request: Request
    batch: Dict[str, Any]


# ------------------------------------------------------------------------ pipeline
class HFPipelineTester:
    """batching = [prefill, compress, decode] batch sizes; `compressor(kv, it_len) -> kv` (a CCM module,
    a `KVPressCompressor`, a quantiser, or None)."""

    def __init__(self, backend: Any, compressor: Optional[Callable] = None, batching: Sequence[int] = (15, 45, 90),
                 req_per_sec: float = 10.0, max_wait_time: float = 0.5, worker_check_time: float = 0.002,
                 pad_token_id: int = 0, eos_token_id: Optional[int] = None, temperature: float = 0.0,
                 seed: int = 0, monitor_gpu: bool = False):
        self.backend, self.compressor = backend, compressor
        self.prefill_batch, self.compress_batch, self.decode_batch = (int(b) for b in batching)
        self.rate, self.check = req_per_sec, worker_check_time
        self.pad, self.eos, self.temperature = pad_token_id, eos_token_id, temperature
        self.pool = KVCachePool()
        self.scheduler = DynamicScheduler(self.prefill_batch, self.decode_batch, max_wait_time, self.compress_batch)
        self.timestamps = TimestampManager()
        self.monitor = GPUMonitor() if monitor_gpu else None
        self.perf = PerformanceMonitor()
        self.gen = torch.Generator().manual_seed(seed)
        self.compress_stats = {"calls": 0, "rows_in": 0, "rows_out": 0, "seconds": 0.0}
        self._done = threading.Event()
        self._errors: List[str] = []
        self._lock = threading.Lock()
        self._outstanding = 0

    # ------------------------------------------------------------ compression
    def get_comp_len(self, request: Request) -> Tuple[int, int]:
        """(image rows, text rows) of a request's prompt KV."""
        img = int(getattr(request, "image_rows", 0) or 0)
        return img, max(0, request.kv_rows - img)

    def run_compressor(self, entries: List[KV], requests: List[Request]) -> List[KV]:
        """Compress in chunks of the compress batch size (each request with its own split)."""
        if self.compressor is None:
            return entries
        out: List[KV] = []
        for i in range(0, len(entries), self.compress_batch):
            for kv, r in zip(entries[i:i + self.compress_batch], requests[i:i + self.compress_batch]):
                self.timestamps.record(r.request_id, "compress_start")
                t0 = self._now(sync=True)
                ckv = self._apply(kv, list(self.get_comp_len(r)))
                dt = self._now(sync=True) - t0
                self.timestamps.record(r.request_id, "compress_finish")
                self.compress_stats["calls"] += 1
                self.compress_stats["rows_in"] += kv[0][0].shape[2]
                self.compress_stats["rows_out"] += ckv[0][0].shape[2]
                self.compress_stats["seconds"] += dt
                out.append([(k.contiguous(), v.contiguous()) for k, v in ckv])
        return out

    def _apply(self, kv: KV, it_len: List[int]) -> KV:
        """Compressors take (kv, it_len); quantisers and other one-argument callables take the cache only."""
        if getattr(self, "_one_arg", None) is None:
            import inspect
            try:
                params = [p for p in inspect.signature(self.compressor).parameters.values()
                          if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD, p.VAR_POSITIONAL)]
                self._one_arg = len(params) == 1 and params[0].kind is not params[0].VAR_POSITIONAL
            except (TypeError, ValueError):
                self._one_arg = False
        return self.compressor(kv) if self._one_arg else self.compressor(kv, it_len)

    def _now(self, sync: bool = False) -> float:
        if sync and torch.cuda.is_available() and str(getattr(self.backend, "device", "cpu")).startswith("cuda"):
            torch.cuda.synchronize()
        return time.perf_counter()

    # ---------------------------------------------------------------- stages
    def _process_prefill(self, batch: List[_Arrival]) -> None:
        reqs = [a.request for a in batch]
        ids, mask = left_pad([r.prompt for r in reqs], self.pad, getattr(self.backend, "device", "cpu"))
        for r in reqs:
            r.status = RequestStatus.PREFILLING
            self.timestamps.record(r.request_id, "prefill_start")
        extra = batch[0].batch.get("extra")
        logits, kv = self.backend.prefill(ids, mask, extra)
        first = self._sample(logits)
        t = self._now(sync=True)
        lens = [len(r.prompt) + int(getattr(r, "extra_rows", 0) or 0) for r in reqs]
        self.pool.store_kvcache([r.request_id for r in reqs], kv, lens)
        for r, n, tok in zip(reqs, lens, first):
            r.kv_rows = n
            r.output = [int(tok)]
            r.metrics.prefill_end = t
            self.timestamps.record(r.request_id, "prefill_finish", t)
            self.timestamps.record(r.request_id, "decoding_queueing_start", t)
        group = _Group(reqs, [int(x) for x in first], {"request_size": len(reqs)})
        self.scheduler.add_request(group, "decoding")

    def _merge_prefill_results(self, groups: List[_Group]) -> Tuple[List[Request], KV, List[int], List[int]]:
        reqs = [r for g in groups for r in g.requests]
        first = [t for g in groups for t in g.first_tokens]
        entries = [self.pool.pop_kvcache(r.request_id) for r in reqs]
        for r in reqs:
            r.status = RequestStatus.COMPRESSING
        entries = self.run_compressor(entries, reqs)
        merged, lens = merge_kv_cache(entries)
        return reqs, merged, lens, first

    def _process_decoding(self, groups: List[_Group]) -> None:
        reqs, kv, lens, first = self._merge_prefill_results(groups)
        dev = kv[0][0].device
        B, S = len(reqs), kv[0][0].shape[2]
        mask = create_attention_mask_from_padding(lens, S, dev)
        cache = self.backend.make_cache(kv)
        tokens = torch.as_tensor(first, dtype=torch.long, device=dev)[:, None]
        valid = torch.as_tensor(lens, dtype=torch.long, device=dev)
        # position of a new token: the true prompt length when the cache was evicted or merged keeps
        # HuggingFace semantics only through the mask, so the valid (compressed) length is used, as
        # `generate()` would derive it from the mask
        alive = torch.ones(B, dtype=torch.bool, device=dev)
        budget = torch.as_tensor([r.max_tokens for r in reqs], device=dev)
        t0 = self._now(sync=True)
        for r in reqs:
            r.status = RequestStatus.DECODING
            r.metrics.decode_start = t0
            self.timestamps.record(r.request_id, "decoding_start", t0)
        steps = int(budget.max()) - 1
        for step in range(max(0, steps)):
            mask = torch.cat([mask, torch.ones(B, 1, dtype=mask.dtype, device=dev)], 1)
            logits = self.backend.decode_step(tokens, cache, mask, (valid + step)[:, None])
            nxt = torch.as_tensor(self._sample(logits), device=dev)
            for b, r in enumerate(reqs):
                if not alive[b]:
                    continue
                r.output.append(int(nxt[b]))
                if len(r.output) >= r.max_tokens or (self.eos is not None and int(nxt[b]) == self.eos):
                    alive[b] = False
            tokens = nxt[:, None]
            if not bool(alive.any()):
                break
        t1 = self._now(sync=True)
        for r in reqs:
            r.metrics.decode_end, r.metrics.generated = t1, len(r.output)
            r.status = RequestStatus.COMPLETED
            self.timestamps.record(r.request_id, "decoding_finish", t1)
            self.timestamps.record(r.request_id, "generated_lens", len(r.output))
        with self._lock:
            self._outstanding -= len(reqs)

    def _sample(self, logits: torch.Tensor) -> List[int]:
        if self.temperature <= 0:
            return logits.argmax(-1).tolist()
        p = torch.softmax(logits.float().cpu() / self.temperature, -1)
        return torch.multinomial(p, 1, generator=self.gen)[:, 0].tolist()

    # --------------------------------------------------------------- threads
    def _collect_requests(self, reqs: List[Request], arrivals: List[float], t0: float) -> None:
        for r, at in zip(reqs, arrivals):
            delay = t0 + at - time.perf_counter()
            if delay > 0:
                time.sleep(delay)
            now = time.perf_counter()
            r.metrics.arrival = now
            r.enter_queue()
            self.timestamps.create_request([r.request_id])
            self.timestamps.record(r.request_id, "arrival", now)
            self.timestamps.record(r.request_id, "prefill_queueing_start", now)
            batch = {"input_ids": torch.empty(1, len(r.prompt), dtype=torch.uint8), "extra": getattr(r, "extra", None)}
            arrival = _Arrival(r, batch)
            self.scheduler.add_request(arrival, "prefill")
        self._done.set()

    def _dispatch_requests(self, pool: ThreadPoolExecutor) -> None:
        while True:
            with self._lock:
                finished = self._done.is_set() and self._outstanding == 0
            if finished:
                return
            kind, batch = self.scheduler.select_batch()
            if kind is None:
                time.sleep(self.check)
                continue
            if self.monitor is not None:
                self.monitor.accum_state_round(kind)
            fn = self._process_prefill if kind == "prefill" else self._process_decoding
            try:
                pool.submit(fn, batch).result()
            except Exception as exc:              # the failing batch is marked; the others keep going
                self._errors.append(f"{kind}: {type(exc).__name__}: {exc}")
                members = [a.request for a in batch] if kind == "prefill" else [r for g in batch for r in g.requests]
                for r in members:
                    r.fail(exc)
                with self._lock:
                    self._outstanding -= len(members)

    # -------------------------------------------------------------------- run
    def run_concurrent_test(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64,
                            image_rows: Optional[Sequence[int]] = None, extras: Optional[Sequence[Any]] = None,
                            poisson: bool = False) -> TestResult:
        """`prompts`: token ids per request; `image_rows[i]`: how many leading KV rows of request i are
        image rows (for the image / text split of the merge compressor); `extras[i]`: passed to the
        backend's prefill (pixel values and the like)."""
        import random
        rng = random.Random(0)
        reqs = []
        for i, p in enumerate(prompts):
            r = Request(i, list(p), max_new_tokens)
            r.image_rows = int(image_rows[i]) if image_rows else 0
            r.extra = extras[i] if extras else None
            r.kv_rows = 0
            reqs.append(r)
        t, arrivals = 0.0, []
        for _ in reqs:
            arrivals.append(t)
            t += rng.expovariate(self.rate) if poisson else 1.0 / self.rate
        self._outstanding = len(reqs)
        self._done.clear()
        if self.monitor is not None:
            self.monitor.start_monitoring()
        t0 = time.perf_counter()
        collector = threading.Thread(target=self._collect_requests, args=(reqs, arrivals, t0), daemon=True)
        with ThreadPoolExecutor(max_workers=1) as pool:
            collector.start()
            self._dispatch_requests(pool)
        collector.join()
        wall = time.perf_counter() - t0
        if self.monitor is not None:
            self.monitor.stop_monitoring()
        res = self.perf.summarise(reqs, wall, self.rate)
        res.compression = dict(self.compress_stats, errors=list(self._errors))
        self.requests = reqs
        return res


ImprovedConcurrentTesterHF = HFPipelineTester
