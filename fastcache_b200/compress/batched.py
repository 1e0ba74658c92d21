"""HF-tensor front ends of the merge compressor: batched, stream-pipelined and layer-chunked.

Parity (interfaces; the execution underneath is this package's GEMM op):
  * BatchedGEMMCompressor   "kv-cache pipeline"/nanovllm/kernels/batched_compress.py:181-654 — stacked
    weights of all layers, `load_from_original_compressor`, `forward(kv_cache, it_len)`,
    `compress_layers(layer_start, layer_end, stream)` for chunked overlap
  * PipelineAsyncCompressor  :669-820 — N round-robin side streams, submit / ready / wait / cleanup
  * FusedCompressor + fused_linear_relu_dropout   kernels/fused_compress.py:22-378 (dropout is the
    identity at inference, so the fused op is linear + ReLU in the GEMM epilogue)
  * StreamPriorityManager, LayerwiseCompressor, ZeroOverheadScheduler, ZeroOverheadCompressEngine,
    create_zero_overhead_compressor   kernels/zero_overhead_compress.py:46-591 — decode-overlap engine
    that compresses `layers_per_decode_step` layers per call on a low-priority stream
The serving engine itself does not go through these classes: it compresses inside the paged pool
(`fastcache_b200.compress.inpool`).  They exist for code that holds HuggingFace-format KV tensors.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import ops
from .ccm import PackedCCMWeights, _CCMBase

KV = List[Tuple[torch.Tensor, torch.Tensor]]


def batched_linear_relu(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], relu: bool = True
                        ) -> torch.Tensor:
    """Y[l] = act(X[l] @ W[l].T + B[l]) for stacked layers: x [L, M, K], w [L, N, K], b [L, N].

    One batched matrix product for all layers (the reference's own fallback form of this op,
    "kv-cache pipeline"/nanovllm/kernels/batched_compress.py:347-358: `torch.bmm` over the stacked layers, one
    launch instead of L).  The engine does not come through here: its merge compression is the fused in-pool kernel
    (csrc/ccm.cu), which also does the gather and the scatter; this front end serves callers that hold
    HuggingFace-format tensors."""
    y = torch.bmm(x, w.transpose(1, 2))
    if b is not None:
        y = y + b[:, None, :].to(y.dtype)
    return torch.relu(y) if relu else y


def fused_linear_relu_dropout(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], p: float = 0.0,
                              training: bool = False) -> torch.Tensor:
    y = ops.linear(x, w, b, "relu")
    return torch.nn.functional.dropout(y, p, True) if (training and p > 0) else y


class BatchedGEMMCompressor(nn.Module):
    def __init__(self, n_layer: int = 0, head_dim: int = 0, compression_factor: int = 0, min_seq_len: int = 1):
        super().__init__()
        self.n_layer, self.head_dim, self.compression_factor = n_layer, head_dim, compression_factor
        self.min_seq_len = min_seq_len
        self.w: Optional[PackedCCMWeights] = None

    def load_from_original_compressor(self, original: _CCMBase, dtype: Optional[torch.dtype] = None,
                                      device: Any = None) -> "BatchedGEMMCompressor":
        p0 = next(original.parameters())
        self.w = original.pack(dtype or p0.dtype, device or p0.device)
        self.n_layer, self.head_dim = original.n_layer, original.head_dim
        self.compression_factor, self.min_seq_len = original.compression_factor, original.min_seq_len
        return self

    def _segment(self, x: torch.Tensor, layer: int, bank: int) -> torch.Tensor:
        B, H, S, D = x.shape
        f = self.compression_factor
        s = S // f
        if S == 0 or s < self.min_seq_len:
            return x
        z = x[:, :, : s * f].reshape(B * H * s, D * f)
        w = self.w
        h = ops.linear(z, w.w1[layer, bank], w.b1[layer, bank], "relu")
        h = ops.linear(h, w.w2[layer, bank], w.b2[layer, bank], "relu")
        y = ops.linear(h, w.w3[layer, bank], w.b3[layer, bank]).view(B, H, s, D).to(x.dtype)
        return torch.cat([y, x[:, :, s * f:]], dim=2) if S > s * f else y

    def compress_layers(self, kv_cache: KV, it_len: Sequence[int], layer_start: int, layer_end: int,
                        stream: Any = None) -> KV:
        if self.w is None:
            raise RuntimeError("call load_from_original_compressor first")
        img = 0 if self.w.single_segment else int(it_len[0])
        ctx = torch.cuda.stream(stream) if stream is not None else _null()
        out: KV = []
        with ctx:
            for layer in range(layer_start, layer_end):
                k, v = kv_cache[layer - layer_start] if len(kv_cache) == layer_end - layer_start else kv_cache[layer]
                res = []
                for kvi, x in ((0, k), (1, v)):
                    a = self._segment(x[:, :, :img], layer, 2 + kvi)
                    b = self._segment(x[:, :, img:], layer, kvi)
                    res.append(torch.cat([a, b], dim=2).contiguous())
                out.append((res[0], res[1]))
        return out

    @torch.no_grad()
    def forward(self, kv_cache: KV, it_len: Sequence[int] = (0, 0)) -> KV:
        return self.compress_layers(kv_cache, it_len, 0, len(kv_cache))


class FusedCompressor(BatchedGEMMCompressor):
    def load_from_pytorch_module(self, module: _CCMBase) -> "FusedCompressor":
        self.load_from_original_compressor(module)
        return self

    def compress_layer_fused(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int, it_len: Sequence[int] = (0, 0)):
        return self.compress_layers([(k, v)], it_len, layer_idx, layer_idx + 1)[0]


class CompressionState(Enum):
    NONE = auto()
    PENDING = auto()
    IN_PROGRESS = auto()
    COMPLETED = auto()


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class PipelineAsyncCompressor:
    """Round-robin side streams; each submission records an event that `wait_compression` joins."""

    def __init__(self, compressor: Any, num_streams: int = 2, device: Any = None):
        self.compressor = compressor
        self.streams = [torch.cuda.Stream(device=device) for _ in range(num_streams)] \
            if torch.cuda.is_available() else []
        self._rr = 0
        self._lock = threading.Lock()
        self._state: Dict[int, CompressionState] = {}
        self._events: Dict[int, Any] = {}
        self._results: Dict[int, KV] = {}
        self._lens: Dict[int, int] = {}

    def submit_compression(self, seq_id: int, kv_cache: KV, it_len: Sequence[int]) -> None:
        with self._lock:
            self._state[seq_id] = CompressionState.IN_PROGRESS
            stream = self.streams[self._rr % len(self.streams)] if self.streams else None
            self._rr += 1
        if stream is None:
            out = self.compressor(kv_cache, it_len)
        else:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                out = self.compressor(kv_cache, it_len)
                ev = torch.cuda.Event()
                ev.record(stream)
            with self._lock:
                self._events[seq_id] = ev
        with self._lock:
            self._results[seq_id] = out
            self._lens[seq_id] = out[0][0].shape[2]
            if stream is None:
                self._state[seq_id] = CompressionState.COMPLETED

    def is_compression_ready(self, seq_id: int) -> bool:
        with self._lock:
            ev = self._events.get(seq_id)
            done = self._state.get(seq_id) is CompressionState.COMPLETED or (ev is not None and ev.query())
            if done:
                self._state[seq_id] = CompressionState.COMPLETED
            return done

    def wait_compression(self, seq_id: int) -> Optional[KV]:
        with self._lock:
            ev = self._events.get(seq_id)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        with self._lock:
            self._state[seq_id] = CompressionState.COMPLETED
            return self._results.get(seq_id)

    def get_compressed_len(self, seq_id: int) -> Optional[int]:
        return self._lens.get(seq_id)

    def cleanup(self, seq_id: int) -> None:
        with self._lock:
            for d in (self._state, self._events, self._results, self._lens):
                d.pop(seq_id, None)


# ------------------------------------------------------------------ decode-overlap engine
class StreamPriorityManager:
    def __init__(self, device: Any = None, greenctx_streams: Optional[Tuple[Any, Any]] = None):
        self._events: Dict[int, Any] = {}
        if greenctx_streams is not None:
            self.decode_stream, self.compress_stream = greenctx_streams
        elif torch.cuda.is_available():
            lo, hi = torch.cuda.Stream.priority_range()
            self.decode_stream = torch.cuda.Stream(device=device, priority=hi)
            self.compress_stream = torch.cuda.Stream(device=device, priority=lo)
        else:
            self.decode_stream = self.compress_stream = None

    def get_decode_stream(self):
        return self.decode_stream

    def get_compress_stream(self):
        return self.compress_stream

    def record_compress_event(self, seq_id: int):
        if self.compress_stream is None:
            return None
        ev = torch.cuda.Event()
        ev.record(self.compress_stream)
        self._events[seq_id] = ev
        return ev

    def wait_compress_complete(self, seq_id: int, stream: Any = None) -> None:
        ev = self._events.pop(seq_id, None)
        if ev is not None:
            (stream or torch.cuda.current_stream()).wait_event(ev)


class LayerwiseCompressor(nn.Module):
    def __init__(self, compressor: BatchedGEMMCompressor, layers_per_chunk: int = 4):
        super().__init__()
        self.compressor, self.layers_per_chunk = compressor, max(1, layers_per_chunk)

    @property
    def num_chunks(self) -> int:
        return -(-self.compressor.n_layer // self.layers_per_chunk)

    def get_chunk_layers(self, chunk_idx: int) -> Tuple[int, int]:
        a = chunk_idx * self.layers_per_chunk
        return a, min(self.compressor.n_layer, a + self.layers_per_chunk)

    def compress_chunk(self, kv_cache: KV, it_len: Sequence[int], chunk_idx: int, stream: Any = None) -> KV:
        a, b = self.get_chunk_layers(chunk_idx)
        return self.compressor.compress_layers(kv_cache, it_len, a, b, stream)

    def compress_all(self, kv_cache: KV, it_len: Sequence[int]) -> KV:
        out: KV = []
        for c in range(self.num_chunks):
            out.extend(self.compress_chunk(kv_cache, it_len, c))
        return out


@dataclass
class CompressionTask:
    seq_id: int
    kv_cache: KV
    it_len: Sequence[int]
    next_chunk: int = 0
    result: KV = field(default_factory=list)
    state: CompressionState = CompressionState.PENDING


class ZeroOverheadScheduler:
    """Decides whether a chunk of compression fits beside the current decode step."""

    def __init__(self, layerwise: LayerwiseCompressor, streams: StreamPriorityManager, hardware: Any = None):
        from ..autocompress.context import detect_hardware
        self.layerwise, self.streams = layerwise, streams
        self.hw = hardware or detect_hardware()
        self.tasks: Dict[int, CompressionTask] = {}

    def estimate_decode_load(self, batch_size: int, seq_len: int, num_layers: int = 32, num_kv_heads: int = 8,
                             head_dim: int = 128, hidden_size: int = 4096) -> Dict[str, float]:
        ms = self.hw.estimate_decode_latency_ms(batch_size, seq_len, num_layers, num_kv_heads, head_dim, hidden_size)
        bound = self.hw.is_decode_memory_bound(batch_size, seq_len, num_layers, num_kv_heads, head_dim, hidden_size)
        return {"decode_ms": ms, "memory_bound": float(bound), "tensor_idle_share": 0.8 if bound else 0.2}

    def should_compress_now(self, batch_size: int, seq_len: int) -> bool:
        return self.estimate_decode_load(batch_size, seq_len)["memory_bound"] > 0.5 or batch_size >= 8

    def schedule_compression(self, seq_id: int, kv_cache: KV, it_len: Sequence[int]) -> None:
        self.tasks[seq_id] = CompressionTask(seq_id, kv_cache, it_len)

    def execute_compression_chunk(self, seq_id: int) -> bool:
        t = self.tasks[seq_id]
        if t.state is CompressionState.COMPLETED:
            return True
        t.state = CompressionState.IN_PROGRESS
        stream = self.streams.get_compress_stream()
        if stream is not None and t.next_chunk == 0:
            stream.wait_stream(torch.cuda.current_stream())
        t.result.extend(self.layerwise.compress_chunk(t.kv_cache, t.it_len, t.next_chunk, stream))
        t.next_chunk += 1
        if t.next_chunk >= self.layerwise.num_chunks:
            t.state = CompressionState.COMPLETED
            self.streams.record_compress_event(seq_id)
        return t.state is CompressionState.COMPLETED

    def is_compression_complete(self, seq_id: int) -> bool:
        t = self.tasks.get(seq_id)
        return t is not None and t.state is CompressionState.COMPLETED

    def get_compressed_result(self, seq_id: int) -> Optional[KV]:
        t = self.tasks.get(seq_id)
        if t is None or t.state is not CompressionState.COMPLETED:
            return None
        self.streams.wait_compress_complete(seq_id)
        return t.result


class ZeroOverheadCompressEngine:
    def __init__(self, compressor: BatchedGEMMCompressor, layers_per_decode_step: int = 4, device: Any = None,
                 greenctx_streams: Optional[Tuple[Any, Any]] = None):
        self.streams = StreamPriorityManager(device, greenctx_streams)
        self.layerwise = LayerwiseCompressor(compressor, layers_per_decode_step)
        self.scheduler = ZeroOverheadScheduler(self.layerwise, self.streams)
        self.stats = {"started": 0, "chunks": 0, "completed": 0}

    def start_compression(self, seq_id: int, kv_cache: KV, it_len: Sequence[int]) -> None:
        self.scheduler.schedule_compression(seq_id, kv_cache, it_len)
        self.stats["started"] += 1

    def step_compression(self, seq_id: int) -> bool:
        done = self.scheduler.execute_compression_chunk(seq_id)
        self.stats["chunks"] += 1
        if done:
            self.stats["completed"] += 1
        return done

    def wait_compression(self, seq_id: int) -> None:
        while not self.scheduler.is_compression_complete(seq_id):
            self.step_compression(seq_id)
        self.streams.wait_compress_complete(seq_id)

    def get_compressed_cache(self, seq_id: int) -> Optional[KV]:
        return self.scheduler.get_compressed_result(seq_id)

    def get_stats(self) -> dict:
        return dict(self.stats)


def create_zero_overhead_compressor(original: _CCMBase, layers_per_decode_step: int = 4, device: Any = None,
                                    greenctx_streams: Optional[Tuple[Any, Any]] = None) -> ZeroOverheadCompressEngine:
    batched = BatchedGEMMCompressor().load_from_original_compressor(original)
    return ZeroOverheadCompressEngine(batched, layers_per_decode_step, device, greenctx_streams)


# ----------------------------------------------------------------- self-benchmarks
def _time_ms(fn, like: torch.Tensor, iters: int, warmup: int) -> float:
    """Mean time of `fn()` in ms: CUDA events on the current stream (CUDA) or the host clock (CPU)."""
    for _ in range(warmup):
        fn()
    if like.is_cuda:
        torch.cuda.synchronize(like.device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        b.synchronize()
        return float(a.elapsed_time(b)) / iters
    import time
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) * 1e3 / iters


def benchmark_batched_vs_original(num_layers: int = 32, batch_size: int = 1, num_heads: int = 8, seq_len: int = 600,
                                  head_dim: int = 128, compression_factor: int = 5, image_len: int = 576,
                                  device: Any = None, dtype: Optional[torch.dtype] = None, iters: int = 10,
                                  warmup: int = 3, verbose: bool = True) -> Dict[str, float]:
    """Per-layer module compressor against the stacked-weight compressor on one synthetic cache
    (the reference's self-check, "kv-cache pipeline"/nanovllm/kernels/batched_compress.py:827-942, with
    its shapes as defaults).  Returns the two times, their ratio and the largest output difference."""
    from .ccm import KVCacheLinearDecoupleCompressor
    device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    torch.manual_seed(0)
    orig = KVCacheLinearDecoupleCompressor(None, compression_factor, 2, n_layer=num_layers, nhead=num_heads,
                                           head_dim=head_dim)
    for p in orig.parameters():
        nn.init.normal_(p, std=0.05)
    orig = orig.to(device=device, dtype=dtype).eval()
    batched = BatchedGEMMCompressor().load_from_original_compressor(orig)
    kv = [(torch.randn(batch_size, num_heads, seq_len, head_dim, device=device, dtype=dtype),
           torch.randn(batch_size, num_heads, seq_len, head_dim, device=device, dtype=dtype))
          for _ in range(num_layers)]
    it_len = [min(image_len, seq_len), max(0, seq_len - image_len)]
    a, b = orig(kv, it_len), batched(kv, it_len)
    err = max(float((x[0].float() - y[0].float()).abs().max()) for x, y in zip(a, b))
    t_orig = _time_ms(lambda: orig(kv, it_len), kv[0][0], iters, warmup)
    t_batched = _time_ms(lambda: batched(kv, it_len), kv[0][0], iters, warmup)
    out = {"original_ms": t_orig, "batched_ms": t_batched, "speedup": t_orig / max(t_batched, 1e-9),
           "max_abs_diff": err, "compressed_len": int(b[0][0].shape[2])}
    if verbose:
        print(f"[{device.type}] layers {num_layers} batch {batch_size} heads {num_heads} seq {seq_len} "
              f"factor {compression_factor}: module {t_orig:.3f} ms, stacked {t_batched:.3f} ms "
              f"({out['speedup']:.2f}x), max |diff| {err:.3g}")
    return out


def benchmark_fused_vs_pytorch(m: int = 4096, k: int = 640, n: int = 128, device: Any = None,
                               dtype: Optional[torch.dtype] = None, iters: int = 20, warmup: int = 3,
                               verbose: bool = True) -> Dict[str, float]:
    """`relu(x W^T + b)` through this package's linear op (bias and ReLU in the GEMM epilogue on a
    GPU) against the three PyTorch calls (reference self-check: fused_compress.py:381-462)."""
    device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=g).to(device=device, dtype=dtype)
    w = (torch.randn(n, k, generator=g) * k ** -0.5).to(device=device, dtype=dtype)
    b = torch.randn(n, generator=g).to(device=device, dtype=dtype)
    plain = lambda: torch.relu(torch.nn.functional.linear(x, w, b))   # noqa: E731
    fused = lambda: fused_linear_relu_dropout(x, w, b)                # noqa: E731
    err = float((plain().float() - fused().float()).abs().max())
    out = {"pytorch_ms": _time_ms(plain, x, iters, warmup), "fused_ms": _time_ms(fused, x, iters, warmup),
           "max_abs_diff": err}
    out["speedup"] = out["pytorch_ms"] / max(out["fused_ms"], 1e-9)
    if verbose:
        print(f"[{device.type}] {m}x{k}x{n}: PyTorch {out['pytorch_ms']:.3f} ms, fused {out['fused_ms']:.3f} ms "
              f"({out['speedup']:.2f}x), max |diff| {err:.3g}")
    return out
