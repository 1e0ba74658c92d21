"""HTTP serving layer.

Parity: nanovllm_fastapi_server.py — request/response schemas (:158-206), endpoints
POST /generate, POST /generate_batch, GET /status, GET /metrics, POST /switch_mode,
POST /benchmark, POST /comprehensive_test (:474-634), compression modes
none / eager / async / lazy (:214, :260-261), the lazy policy wrapper (:54-153) and the
CLI (:637-677).

Differences by design: one engine thread steps continuously and HTTP handlers only
enqueue requests and await their completion, so concurrent HTTP requests are batched
together (the reference runs every request to completion behind a global lock);
`text` in the response is the decoded completion (the reference returns an empty
string); `prompt_token_ids` is accepted besides `prompt` so the server is usable with
random-init models that have no tokenizer.
"""
from __future__ import annotations

import argparse
import threading
import time
from collections import deque
from concurrent.futures import Future
from typing import Any, Deque, Dict, List, Optional

from ..sampling_params import SamplingParams

try:                                            # the schemas need pydantic; the engine classes do not
    from pydantic import BaseModel
except Exception:                               # pragma: no cover
    BaseModel = object                          # type: ignore


class GenerateRequest(BaseModel):
    prompt: str = ""
    max_tokens: int = 64
    temperature: float = 1.0
    top_p: float = 1.0
    prompt_token_ids: Optional[List[int]] = None


class BatchGenerateRequest(BaseModel):
    prompts: List[str] = []
    max_tokens: int = 64
    temperature: float = 1.0
    top_p: float = 1.0
    prompt_token_ids: Optional[List[List[int]]] = None


class GenerateResponse(BaseModel):
    text: str
    tokens_generated: int
    total_time_ms: float
    tokens_per_second: float
    compression_mode: str
    compression_method: Optional[str] = None
    token_ids: List[int] = []
    ttft_ms: float = 0.0


class BatchGenerateResponse(BaseModel):
    results: List[Dict[str, Any]]
    total_tokens: int
    total_time_ms: float
    avg_throughput: float
    compression_mode: str


class ServerStatus(BaseModel):
    active_requests: int
    completed_requests: int
    total_tokens_generated: int
    avg_throughput: float
    compression_mode: str
    compression_method: str
    compression_stats: Dict[str, Any]
    gpu_memory_used_gb: float
    gpu_memory_peak_gb: float


class CompressionTestResult(BaseModel):
    mode: str
    method: str
    throughput: float
    speedup_vs_none: float
    is_beneficial: bool


class LazyCompressionEngine:
    """The reference wraps its engine to add "compress everything when free blocks run low".
    The engine of this package has that policy built in (`compression_mode="lazy"`); this class
    keeps the wrapper's interface: `step()`, `get_stats()`, the threshold on free blocks."""

    def __init__(self, llm: Any, compression_threshold: float = 0.3):
        self.llm = llm
        self.compression_threshold = compression_threshold
        llm.scheduler.lazy_threshold = 1.0 - compression_threshold
        llm.compression_mode = "lazy" if llm.enable_compression else "none"

    def step(self):
        return self.llm.step()

    def add_request(self, prompt: Any, sampling_params: Any = None, image: Any = None):
        if image is None:
            return self.llm.add_request(prompt, sampling_params)
        return self.llm.add_request(prompt, sampling_params, image=image)

    def is_finished(self) -> bool:
        return self.llm.is_finished()

    def get_stats(self) -> Dict[str, Any]:
        st, bm = self.llm.stats, self.llm.scheduler.block_manager
        return {"compression_count": st.compressions, "lazy_triggers": st.lazy_triggers,
                "blocks_freed": st.blocks_freed, "rows_in": st.compressed_rows_in,
                "rows_out": st.compressed_rows_out, "free_blocks": bm.num_free_blocks,
                "total_blocks": bm.num_blocks, "occupancy": bm.occupancy}


class _Pending:
    def __init__(self, seq, future: Future):
        self.seq, self.future, self.t0 = seq, future, time.perf_counter()


class FastCacheServer:
    """Owns the engine and its stepping thread."""

    MODES = ("none", "eager", "async", "lazy")

    def __init__(self, model: Any, compressor_path: Optional[str] = None, compression_mode: str = "lazy",
                 compression_backend: str = "kvpress", kvpress_method: str = "streaming_llm",
                 compression_factor: int = 5, compression_threshold: float = 0.3, max_model_len: int = 8192,
                 start_thread: bool = True, **engine_kwargs: Any):
        if compression_mode not in self.MODES:
            raise ValueError(f"compression mode must be one of {self.MODES}")
        self.model, self.compressor_path = model, compressor_path
        self.compression_backend, self.kvpress_method = compression_backend, kvpress_method
        self.compression_factor, self.compression_threshold = compression_factor, compression_threshold
        self.max_model_len = max_model_len
        self.engine_kwargs = engine_kwargs
        self.compression_mode = compression_mode
        self.metrics_history: Deque[Dict[str, Any]] = deque(maxlen=1000)
        self.completed_requests = 0
        self.total_tokens = 0
        self._lock = threading.Lock()
        self._inbox: Deque = deque()
        self._pending: Dict[int, _Pending] = {}
        self._stop = threading.Event()
        self._wake = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.llm = None
        self.lazy_engine: Optional[LazyCompressionEngine] = None
        self._build_engine()
        if start_thread:
            self.start()

    # ------------------------------------------------------------------ engine
    def _build_engine(self) -> None:
        from ..engine.llm_engine import LLMEngine
        mode = self.compression_mode
        self.llm = LLMEngine(self.model, compressor_path=self.compressor_path,
                             compression_factor=self.compression_factor, enable_compression=mode != "none",
                             async_compression=mode == "async", compression_backend=self.compression_backend,
                             kvpress_method=self.kvpress_method, max_model_len=self.max_model_len,
                             compression_mode=mode, lazy_occupancy_threshold=1.0 - self.compression_threshold,
                             **self.engine_kwargs)
        self.lazy_engine = LazyCompressionEngine(self.llm, self.compression_threshold) if mode == "lazy" else None

    def start(self) -> None:
        if self._thread is None or not self._thread.is_alive():
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, name="engine-loop", daemon=True)
            self._thread.start()

    def shutdown(self) -> None:
        self._stop.set()
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
        if self.llm is not None:
            self.llm.exit()

    def _admit(self) -> None:
        while self._inbox:
            prompt, sp, image, fut = self._inbox.popleft()
            try:
                seq = self.llm.add_request(prompt, sp, image)
                self._pending[seq.seq_id] = _Pending(seq, fut)
            except Exception as exc:                       # bad request: fail it, keep serving
                fut.set_exception(exc)

    def _loop(self) -> None:
        while not self._stop.is_set():
            with self._lock:
                self._admit()
                busy = not self.llm.is_finished()
                if busy:
                    try:
                        self.llm.step()
                    except Exception as exc:               # engine failure: fail what is in flight
                        for p in self._pending.values():
                            if not p.future.done():
                                p.future.set_exception(exc)
                        self._pending.clear()
                        continue
                    self._harvest()
            if not busy:
                self._wake.wait(timeout=0.05)
                self._wake.clear()

    def _harvest(self) -> None:
        for seq in getattr(self.llm, "_last_finished", []):
            p = self._pending.pop(seq.seq_id, None)
            if p is None:
                continue
            now = time.perf_counter()
            toks = seq.completion_token_ids
            text = self.llm.tokenizer.decode(toks) if self.llm.tokenizer is not None else ""
            dt = now - p.t0
            ttft = (seq.first_token_time - seq.arrival_time) if seq.first_token_time else 0.0
            res = {"text": text, "token_ids": toks, "tokens_generated": len(toks), "total_time_ms": dt * 1e3,
                   "tokens_per_second": len(toks) / max(dt, 1e-9), "ttft_ms": ttft * 1e3,
                   "compression_mode": self.compression_mode,
                   "compression_method": self._method_name()}
            self.completed_requests += 1
            self.total_tokens += len(toks)
            self.metrics_history.append({"time": time.time(), "tokens": len(toks), "latency_ms": dt * 1e3,
                                         "ttft_ms": ttft * 1e3, "throughput": res["tokens_per_second"],
                                         "mode": self.compression_mode})
            p.future.set_result(res)

    def _method_name(self) -> str:
        if self.compression_mode == "none":
            return "none"
        return self.kvpress_method if self.compression_backend == "kvpress" else "mlp"

    # ------------------------------------------------------------------- calls
    def submit(self, prompt: Any, max_tokens: int = 64, temperature: float = 1.0, image: Any = None) -> Future:
        fut: Future = Future()
        sp = SamplingParams(temperature=temperature, max_tokens=max_tokens)
        self._inbox.append((prompt, sp, image, fut))
        self._wake.set()
        return fut

    def generate(self, prompt: Any, max_tokens: int = 64, temperature: float = 1.0, image: Any = None,
                 timeout: Optional[float] = None) -> Dict[str, Any]:
        return self.submit(prompt, max_tokens, temperature, image).result(timeout)

    def generate_batch(self, prompts: List[Any], max_tokens: int = 64, temperature: float = 1.0,
                       timeout: Optional[float] = None) -> Dict[str, Any]:
        t0 = time.perf_counter()
        futs = [self.submit(p, max_tokens, temperature) for p in prompts]
        results = [f.result(timeout) for f in futs]
        dt = time.perf_counter() - t0
        total = sum(r["tokens_generated"] for r in results)
        return {"results": results, "total_tokens": total, "total_time_ms": dt * 1e3,
                "avg_throughput": total / max(dt, 1e-9), "compression_mode": self.compression_mode}

    def get_status(self) -> Dict[str, Any]:
        used = peak = 0.0
        try:
            import torch
            if torch.cuda.is_available():
                used = torch.cuda.memory_allocated() / 2 ** 30
                peak = torch.cuda.max_memory_allocated() / 2 ** 30
        except Exception:
            pass
        hist = list(self.metrics_history)
        avg = sum(m["throughput"] for m in hist) / len(hist) if hist else 0.0
        stats = LazyCompressionEngine.get_stats(self.lazy_engine) if self.lazy_engine else \
            {"compression_count": self.llm.stats.compressions, "blocks_freed": self.llm.stats.blocks_freed}
        return {"active_requests": len(self._pending) + len(self._inbox),
                "completed_requests": self.completed_requests, "total_tokens_generated": self.total_tokens,
                "avg_throughput": avg, "compression_mode": self.compression_mode,
                "compression_method": self._method_name(), "compression_stats": stats,
                "gpu_memory_used_gb": used, "gpu_memory_peak_gb": peak}

    def get_metrics(self, last_n: int = 100) -> List[Dict[str, Any]]:
        return list(self.metrics_history)[-last_n:]

    def switch_compression_mode(self, mode: str, method: Optional[str] = None) -> None:
        """Rebuild the engine with another policy (waits for in-flight requests)."""
        if mode not in self.MODES:
            raise ValueError(f"compression mode must be one of {self.MODES}")
        deadline = time.time() + 120
        while (self._pending or self._inbox) and time.time() < deadline:
            time.sleep(0.01)
        with self._lock:
            self.llm.exit()
            self.compression_mode = mode
            if method:
                self.kvpress_method = method
            self._build_engine()

    def benchmark(self, prompts: List[Any], max_tokens: int = 64) -> Dict[str, Any]:
        return self.generate_batch(prompts, max_tokens, temperature=0.0)

    def comprehensive_test(self, prompts: List[Any], max_tokens: int = 64,
                           modes: Optional[List[str]] = None) -> List[Dict[str, Any]]:
        """Throughput of each compression mode on the same prompts, relative to `none`."""
        out, base = [], None
        keep = self.compression_mode
        for mode in modes or list(self.MODES):
            self.switch_compression_mode(mode)
            r = self.benchmark(prompts, max_tokens)
            if mode == "none":
                base = r["avg_throughput"]
            sp = r["avg_throughput"] / base if base else 1.0
            out.append({"mode": mode, "method": self._method_name(), "throughput": r["avg_throughput"],
                        "speedup_vs_none": sp, "is_beneficial": sp > 1.0})
        self.switch_compression_mode(keep)
        return out


# names used by scripts written against the reference
NanoVLLMServer = FastCacheServer


def create_app(server: FastCacheServer):
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="fastcache_b200 server",
                  description="KV-cache compression serving: none, eager, async, lazy")

    def _prompt(text, ids):
        return list(ids) if ids is not None else text

    @app.post("/generate", response_model=GenerateResponse)
    async def generate(req: GenerateRequest):
        import asyncio
        try:
            fut = server.submit(_prompt(req.prompt, req.prompt_token_ids), req.max_tokens, req.temperature)
            return await asyncio.wrap_future(fut)
        except Exception as exc:
            raise HTTPException(status_code=400, detail=str(exc))

    @app.post("/generate_batch", response_model=BatchGenerateResponse)
    async def generate_batch(req: BatchGenerateRequest):
        import asyncio
        prompts = req.prompt_token_ids if req.prompt_token_ids is not None else req.prompts
        t0 = time.perf_counter()
        futs = [asyncio.wrap_future(server.submit(p, req.max_tokens, req.temperature)) for p in prompts]
        try:
            results = await asyncio.gather(*futs)
        except Exception as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        dt = time.perf_counter() - t0
        total = sum(r["tokens_generated"] for r in results)
        return {"results": results, "total_tokens": total, "total_time_ms": dt * 1e3,
                "avg_throughput": total / max(dt, 1e-9), "compression_mode": server.compression_mode}

    @app.get("/status", response_model=ServerStatus)
    async def status():
        return server.get_status()

    @app.get("/metrics")
    async def metrics(last_n: int = 100):
        return server.get_metrics(last_n)

    @app.post("/switch_mode")
    async def switch_mode(mode: str, method: Optional[str] = None):
        import asyncio
        try:
            await asyncio.get_event_loop().run_in_executor(None, server.switch_compression_mode, mode, method)
        except ValueError as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        return {"status": "ok", "mode": server.compression_mode, "method": server._method_name()}

    @app.post("/benchmark")
    async def benchmark(num_prompts: int = 8, prompt_len: int = 256, max_tokens: int = 64):
        import asyncio
        prompts = _synthetic_prompts(server, num_prompts, prompt_len)
        return await asyncio.get_event_loop().run_in_executor(None, server.benchmark, prompts, max_tokens)

    @app.post("/comprehensive_test")
    async def comprehensive_test(num_prompts: int = 8, prompt_len: int = 256, max_tokens: int = 64):
        import asyncio
        prompts = _synthetic_prompts(server, num_prompts, prompt_len)
        return await asyncio.get_event_loop().run_in_executor(None, server.comprehensive_test, prompts, max_tokens)

    return app


def _synthetic_prompts(server: FastCacheServer, n: int, length: int) -> List[List[int]]:
    import random
    from ..config import text_config_of
    vocab = text_config_of(server.llm.config.hf_config).vocab_size
    rng = random.Random(0)
    return [[rng.randrange(3, vocab) for _ in range(length)] for _ in range(n)]


def main(argv: Optional[List[str]] = None) -> None:
    from .paths import CKPT_DIR
    ap = argparse.ArgumentParser(description="fastcache_b200 HTTP server")
    ap.add_argument("--model", required=True)
    ap.add_argument("--compressor", default=str(CKPT_DIR / "llava_mlp.pth"))
    ap.add_argument("--compression-mode", default="lazy", choices=list(FastCacheServer.MODES))
    ap.add_argument("--compression-backend", default="kvpress", choices=["kvpress", "mlp"])
    ap.add_argument("--kvpress-method", default="streaming_llm")
    ap.add_argument("--compression-factor", type=int, default=5)
    ap.add_argument("--compression-threshold", type=float, default=0.3,
                    help="lazy mode compresses when the share of free blocks falls below this")
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    # engine settings beyond the reference's command line
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--chunked-prefill-tokens", type=int, default=0,
                    help="> 0: prompts that do not fit a prefill step's token budget run in pieces of at least this size")
    ap.add_argument("--greenctx-compress-ratio", type=float, default=0.0,
                    help="> 0: compression streams get this share of the SMs (green context)")
    a = ap.parse_args(argv)
    import uvicorn
    extra = {}
    if a.tensor_parallel_size > 1:
        extra["tensor_parallel_size"] = a.tensor_parallel_size
    if a.chunked_prefill_tokens > 0:
        extra["chunked_prefill_tokens"] = a.chunked_prefill_tokens
    if a.greenctx_compress_ratio > 0:
        extra.update(greenctx_enabled=True, greenctx_compress_ratio=a.greenctx_compress_ratio,
                     greenctx_main_ratio=1.0 - a.greenctx_compress_ratio)
    server = FastCacheServer(a.model, a.compressor if a.compression_backend == "mlp" else None,
                             a.compression_mode, a.compression_backend, a.kvpress_method, a.compression_factor,
                             a.compression_threshold, a.max_model_len, **extra)
    uvicorn.run(create_app(server), host=a.host, port=a.port)


if __name__ == "__main__":
    main()
