"""Online controller: per-prefill compression decisions and the prefill/decode batch choice.

Parity: "kv-cache pipeline"/nanovllm/engine/auto_compress_controller.py:12-381.
`decide()` (every `decision_interval` prefill steps) returns the pipeline
(prefill / decode / none), whether compression runs asynchronously, the number of
compression streams (1-4), layers per decode step (1-8), whether to use a green
context and the SM share of compression (0.10-0.60; base 0.40 for GEMM methods,
0.20 for memory-bound ones, 0.25 for mixed; moved in 0.05 steps from the EWMA of
compression time against decode or prefill time).  `decide_batch_type()` is the
dual-batch choice between a prefill and a decode batch under a decode-share budget
per interval.  Thresholds: min_seq_len 256, min_output_len 64, min_speedup 1.05.

The meters are fed with device-timed intervals by the engine; decisions only change
at interval boundaries, which keeps tensor-parallel ranks (that all run this
controller on identical inputs) in agreement as long as they are fed the same
numbers — the engine feeds rank-local timings, so under TP the engine all-reduces
(max) them first.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..autocompress.context import WorkloadContext, detect_hardware
from ..autocompress.pipeline import PipelineOrchestrator, PipelineStrategy
from ..autocompress.profiles import ComputeType, get_profile


class EWMAMeter:
    def __init__(self, alpha: float = 0.2):
        self.alpha = alpha
        self.value: Optional[float] = None
        self.samples = 0

    def update(self, x: Optional[float]) -> None:
        if x is None:
            return
        self.value = x if self.value is None else self.alpha * x + (1.0 - self.alpha) * self.value
        self.samples += 1


@dataclass
class AutoCompressionDecision:
    pipeline: str                  # prefill | decode | none
    async_compress: bool
    compression_streams: int
    decode_layers_per_step: int
    greenctx_enabled: bool
    sm_compress_ratio: float
    sm_main_ratio: float


_BASE_SM = {ComputeType.GEMM: 0.40, ComputeType.MEMORY: 0.20, ComputeType.MIXED: 0.25}


class AutoCompressionController:
    def __init__(self, *, compression_backend: str, kvpress_method: Optional[str], compression_factor: int,
                 num_layers: int, num_kv_heads: int, head_dim: int, greenctx_enabled: bool,
                 decision_interval: int = 4, min_seq_len: int = 256, min_output_len: int = 64,
                 min_speedup: float = 1.05, min_sm_ratio: float = 0.10, max_sm_ratio: float = 0.60,
                 greenctx_min_batch: int = 8, greenctx_min_output_len: int = 128, force_compress: bool = False,
                 dual_batch_enabled: bool = True, dual_batch_interval: int = 4,
                 dual_batch_min_decode_share: float = 0.20, dual_batch_max_decode_share: float = 0.80,
                 hidden_size: int = 4096):
        self.backend = compression_backend
        self.factor = max(1, compression_factor)
        self.num_layers, self.num_kv_heads, self.head_dim, self.hidden_size = num_layers, num_kv_heads, head_dim, hidden_size
        self.greenctx_available = greenctx_enabled
        self.interval = max(1, decision_interval)
        self.min_seq_len, self.min_output_len, self.min_speedup = min_seq_len, min_output_len, min_speedup
        self.sm_lo, self.sm_hi = min_sm_ratio, max_sm_ratio
        self.green_min_batch, self.green_min_out = greenctx_min_batch, greenctx_min_output_len
        self.force = force_compress
        self.dual_enabled = dual_batch_enabled
        self.dual_interval = max(1, dual_batch_interval)
        self.dual_lo, self.dual_hi = dual_batch_min_decode_share, dual_batch_max_decode_share

        if compression_backend == "kvpress":
            self.method_name = kvpress_method or "streaming_llm"
            self.method_kwargs = {"compression_ratio": 1.0 - 1.0 / self.factor}
        else:
            self.method_name = "mlp"
            self.method_kwargs = {"compression_ratio": float(self.factor)}
        self.compute_type = get_profile(self.method_name).compute_type
        self.orchestrator = PipelineOrchestrator(detect_hardware(), min_speedup=min_speedup)

        self.sm_ratio = _BASE_SM[self.compute_type]
        self.streams = 2
        self.layers_per_step = 4
        self.pipeline = "prefill"
        self._last_decision: Optional[AutoCompressionDecision] = None
        self._decisions = 0
        self._dual_step = 0
        self._dual_budget = 0
        self._dual_share = 0.5
        self.prefill_ms_per_token = EWMAMeter()
        self.prefill_step_ms = EWMAMeter()
        self.decode_step_ms = EWMAMeter()
        self.compress_ms = EWMAMeter()
        self.compress_ms_per_layer = EWMAMeter()

    # ---------------------------------------------------------------- meters
    def update_prefill(self, elapsed_ms: float, tokens: int) -> None:
        if tokens > 0:
            self.prefill_ms_per_token.update(elapsed_ms / tokens)
        self.prefill_step_ms.update(elapsed_ms)

    def update_decode(self, elapsed_ms: float, batch_size: int = 0) -> None:
        self.decode_step_ms.update(elapsed_ms)

    def update_compress(self, elapsed_ms: float, tokens: int = 0) -> None:
        self.compress_ms.update(elapsed_ms)
        if self.num_layers > 0:
            self.compress_ms_per_layer.update(elapsed_ms / self.num_layers)

    # ------------------------------------------------------------ dual batch
    def decide_batch_type(self, *, waiting: int, running: int, pending_compressions: int = 0) -> str:
        if waiting <= 0:
            return "decode"
        if running <= 0 or not self.dual_enabled or self.pipeline in ("none", "prefill"):
            return "prefill"
        self._dual_step += 1
        total = max(1, waiting + running)
        run_share, wait_share = running / total, waiting / total
        if wait_share >= 0.65:
            return "prefill"
        if run_share >= 0.85 and wait_share <= 0.15:
            return "decode"
        p_ms, d_ms = self.prefill_step_ms.value, self.decode_step_ms.value
        if p_ms and d_ms:
            if p_ms > 1.8 * d_ms and self.pipeline != "decode":
                return "prefill"
            if d_ms > 1.8 * p_ms and wait_share <= 0.40:
                return "decode"
        # a new budget only at interval boundaries: once it is spent the rest of the interval prefills
        if self._dual_step % self.dual_interval == 1 or self.dual_interval == 1:
            share = run_share
            if p_ms and d_ms:
                r = d_ms / max(p_ms, 1e-6)
                share += 0.15 if r > 1.25 else (-0.15 if r < 0.80 else 0.0)
            lo, hi = self.dual_lo, self.dual_hi
            if self.pipeline == "decode":
                share += 0.15
                lo, hi = max(lo, 0.25), max(hi, 0.85)
            share = min(hi, max(lo, share))
            self._dual_share = share
            budget = 0 if share < 0.15 else int(round(share * self.dual_interval))
            self._dual_budget = max(0, min(self.dual_interval - 1, budget))
        if self._dual_budget > 0:
            self._dual_budget -= 1
            return "decode"
        return "prefill"

    # ----------------------------------------------------------------- tuning
    def _tune_sm_ratio(self, pending: int) -> float:
        r = self.sm_ratio
        c = self.compress_ms.value
        if self.compute_type is ComputeType.GEMM:
            d = self.decode_step_ms.value
            if c and d:
                r += 0.05 if c > 1.10 * d else (-0.05 if c < 0.60 * d else 0.0)
        else:
            p = self.prefill_step_ms.value
            if c and p:
                r += 0.05 if c > 0.80 * p else (-0.05 if c < 0.40 * p else 0.0)
        if pending > self.streams:
            r += 0.05
        return min(self.sm_hi, max(self.sm_lo, r))

    def _tune_streams(self, pending: int) -> int:
        s = self.streams
        c, p = self.compress_ms.value, self.prefill_step_ms.value
        if c and p:
            ratio = c / max(p, 1e-6)
            s += 1 if ratio > 0.80 else (-1 if ratio < 0.40 else 0)
        if pending > s:
            s += 1
        if pending == 0 and s > 1:
            s -= 1
        return max(1, min(4, s))

    def _tune_layers_per_step(self) -> int:
        cur = self.layers_per_step
        cl, d = self.compress_ms_per_layer.value, self.decode_step_ms.value
        if cl and d:
            want = max(1, min(8, int(round(d / max(cl, 1e-6)))))
            if abs(want - cur) >= 2:
                cur += 1 if want > cur else -1
            else:
                cur = want
        return cur

    # ----------------------------------------------------------------- decide
    def decide(self, *, batch_size: int, seq_len: int, expected_output_len: int, pending_compressions: int = 0
               ) -> AutoCompressionDecision:
        self._decisions += 1
        # the size gate is cheap and is looked at every time: a decision cached for the interval is kept
        # only while the batch stays on the same side of it (a short warm-up batch must not switch
        # compression off for the long batches that follow, nor the other way round)
        too_small = (seq_len < self.min_seq_len or expected_output_len < self.min_output_len) and not self.force
        if (self._last_decision is not None and self._decisions % self.interval != 0
                and too_small == getattr(self, "_last_too_small", too_small)):
            return self._last_decision
        self._last_too_small = too_small
        if too_small:
            d = AutoCompressionDecision("none", False, self.streams, self.layers_per_step, False, 0.0, 1.0)
            self.pipeline = "none"
            self._last_decision = d
            return d
        w = WorkloadContext(batch_size=batch_size, seq_len=seq_len, expected_output_len=expected_output_len,
                            num_layers=self.num_layers, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                            hidden_size=self.hidden_size)
        plan = self.orchestrator.create_pipeline(self.method_name, w, **self.method_kwargs)
        if plan.estimated_speedup < self.min_speedup and not self.force:
            pipeline = "none"
        else:
            pipeline = "decode" if plan.strategy is PipelineStrategy.ASYNC_WITH_DECODE else "prefill"
        sm = self._tune_sm_ratio(pending_compressions)
        green = self.greenctx_available and pipeline != "none"
        if green and self.compute_type is ComputeType.GEMM and (
                batch_size < self.green_min_batch or expected_output_len < self.green_min_out):
            green = False
        if green and self.compress_ms.samples >= 3:
            ref = self.prefill_step_ms.value if pipeline == "prefill" else self.decode_step_ms.value
            if ref and self.compress_ms.value / max(ref, 1e-6) < 0.35:
                green = False                      # compression is too small to deserve its own SMs
        streams, layers = self.streams, self.layers_per_step
        if pipeline == "prefill":
            streams = self._tune_streams(pending_compressions)
        elif pipeline == "decode":
            layers = self._tune_layers_per_step()
            if plan.chunk_size > 0:
                layers = max(1, min(8, plan.chunk_size))
        async_c = False
        if pipeline == "prefill":
            c, p = self.compress_ms.value, self.prefill_step_ms.value
            if pending_compressions > 0:
                async_c = True
            elif c and p:
                async_c = c > 0.40 * p
            else:
                async_c = batch_size >= 8
        d = AutoCompressionDecision(pipeline, async_c, streams, layers, green, sm if green else sm,
                                    max(0.05, 1.0 - sm))
        self.sm_ratio, self.streams, self.layers_per_step, self.pipeline = sm, streams, layers, pipeline
        self._last_decision = d
        return d
