"""Serving engine: request intake, the step loop and the compression policies.

Parity
  * text engine and `generate()`       nanovllm/engine/llm_engine.py:12-82
  * multimodal engine with compression "kv-cache pipeline"/nanovllm/engine/
    llava_engine.py:52-620 — constructor kwargs (:61-86), `add_request`,
    `step(apply_compression) -> (outputs, num_tokens)` with num_tokens > 0 for
    prefill tokens and < 0 for minus the decode batch size, dual-batch choice,
    per-prefill controller decision, sync / async / decode-overlap
    compression, `_free_compressed_blocks`
  * lazy policy (compress when the pool is nearly full)
    nanovllm_fastapi_server.py:98-145

One engine class serves text and image requests.  Host decisions never depend
on `event.query()` or timing, only on step counts and queue state, so the
replicated schedulers of tensor-parallel ranks stay in lockstep; the ordering
"compression finished before its tail blocks are reused" is enforced on the
device (`main_stream.wait_event`) before the blocks return to the free list.
"""
from __future__ import annotations

import atexit
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence as Seq, Tuple, Union

import torch

from ..config import Config, ModelConfig, text_config_of
from ..parallel import tp as tpmod
from ..sampling_params import SamplingParams
from ..utils.tracing import StepTrace, nvtx_range
from .model_runner import ModelRunner
from .scheduler import Scheduler
from .async_compression import AsyncCompressionManager
from .sequence import CompressionState, Sequence


@dataclass
class PendingCompression:
    """A compression launched on a side stream (or in layer chunks)."""
    seq: Sequence
    event: Any = None
    start_event: Any = None
    tokens: int = 0
    next_layer: int = 0           # decode pipeline: first layer not yet launched
    rows: int = 0                 # rows that were compressed
    new_len: int = 0
    reported: bool = False
    stream: Any = None            # decode pipeline: the one stream all layer chunks of this request run on
    shadow: bool = False          # the result goes to `seq.shadow_table`; the request keeps decoding meanwhile


@dataclass
class StepStats:
    steps: int = 0
    prefill_steps: int = 0
    decode_steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    compressions: int = 0
    compressed_rows_in: int = 0
    compressed_rows_out: int = 0
    blocks_freed: int = 0
    lazy_triggers: int = 0
    preemptions: int = 0
    compress_failures: int = 0
    aborted: int = 0
    recoveries: int = 0
    history: List[dict] = field(default_factory=list)


class LLMEngine:
    def __init__(self, model: Union[str, Any] = "", compressor_path: Optional[str] = None,
                 compression_factor: int = 5, enable_compression: bool = False,
                 async_compression: bool = False, compression_backend: str = "mlp",
                 kvpress_method: str = "streaming_llm", compression_pipeline: str = "auto",
                 compression_streams: int = 2, greenctx_enabled: bool = False,
                 greenctx_compress_ratio: float = 0.25, greenctx_main_ratio: float = 0.75,
                 greenctx_main_stream: bool = False, decode_layers_per_step: int = 4,
                 auto_tune: bool = False, auto_tune_interval: int = 4, auto_dual_batch: bool = True,
                 auto_dual_interval: int = 4, auto_min_seq_len: int = 256, auto_min_output_len: int = 64,
                 auto_min_speedup: float = 1.05, auto_force_compress: bool = False,
                 compressor: Any = None, tokenizer: Any = None, decode_overlap: str = "shadow",
                 check_streams: Optional[bool] = None, **kwargs):
        hf_config = kwargs.pop("hf_config", None)
        if not isinstance(model, str):          # a config object / dict instead of a path: random init
            hf_config, model = model, ""
        if isinstance(hf_config, dict):
            hf_config = ModelConfig(**hf_config)
        config = Config.from_kwargs(model, **kwargs)
        if hf_config is not None:
            config.hf_config = hf_config
            if not model:
                config.extra["random_init"] = True
        elif model:
            config.hf_config = ModelConfig.from_pretrained(model)
        else:
            raise ValueError("give a model directory or an hf_config")
        tc = text_config_of(config.hf_config)
        config.max_model_len = min(config.max_model_len, getattr(tc, "max_position_embeddings", 1 << 30))
        if config.tensor_parallel_size > 1 and not tpmod.is_tp_initialized():
            tpmod.init_tensor_parallel(config.tensor_parallel_size)
        self.config = config
        Sequence.block_size = config.kvcache_block_size

        self.tokenizer = tokenizer
        self.processor = None
        if tokenizer is None and model:
            self._load_tokenizer(model)
        if config.eos < 0:
            eos = getattr(self.tokenizer, "eos_token_id", None)
            if eos is None:
                eos = getattr(tc, "eos_token_id", -1)
                if isinstance(eos, (list, tuple)):
                    eos = eos[0]
            config.eos = -1 if eos is None else int(eos)

        # a compression mode given through Config wins over the bool pair
        if config.compression_mode != "none":
            enable_compression = True
            async_compression = config.compression_mode == "async"
        elif enable_compression:
            config.compression_mode = "async" if async_compression else "eager"
        self.model_runner = ModelRunner(
            config, compressor_path=compressor_path, compression_factor=compression_factor,
            enable_compression=enable_compression, async_compression=async_compression,
            compression_backend=compression_backend, kvpress_method=kvpress_method,
            compression_pipeline=compression_pipeline, compression_streams=compression_streams,
            greenctx_enabled=greenctx_enabled, greenctx_compress_ratio=greenctx_compress_ratio,
            greenctx_main_ratio=greenctx_main_ratio, greenctx_main_stream=greenctx_main_stream,
            decode_layers_per_step=decode_layers_per_step, compressor=compressor,
            min_seq_len=int(config.extra.get("min_seq_len", 2)),
            kvpress_params=config.extra.get("kvpress_params"))
        self.scheduler = Scheduler(config)
        self.scheduler.on_release = self._on_release

        r = self.model_runner
        self.enable_compression = enable_compression and r.compression_pipeline != "none"
        self.async_compression = async_compression
        self.compression_factor = r.compression_factor
        self.compression_backend = compression_backend
        self.kvpress_method = kvpress_method
        self.compression_pipeline = r.compression_pipeline
        self.compression_mode = config.compression_mode if self.enable_compression else "none"
        self.image_token_len = r.image_token_len
        self.image_token_id = r.image_token_id
        self.auto_tune = auto_tune
        self.auto_tune_interval = max(1, auto_tune_interval)
        self.auto_dual_batch = auto_dual_batch
        self.auto_dual_interval = max(1, auto_dual_interval)
        self._auto_controller = None
        if auto_tune and self.enable_compression:
            from .auto_compress_controller import AutoCompressionController
            self._auto_controller = AutoCompressionController(
                compression_backend=compression_backend, kvpress_method=kvpress_method,
                compression_factor=self.compression_factor, num_layers=r.num_hidden_layers,
                num_kv_heads=r.num_key_value_heads, head_dim=r.head_dim,
                greenctx_enabled=r.greenctx_enabled, decision_interval=self.auto_tune_interval,
                min_seq_len=auto_min_seq_len, min_output_len=auto_min_output_len,
                min_speedup=auto_min_speedup, force_compress=auto_force_compress,
                dual_batch_enabled=auto_dual_batch, dual_batch_interval=self.auto_dual_interval)
        # decode pipeline: "shadow" = the layers are compressed into a second set of blocks while the request keeps
        # decoding over its original rows (the reference's decode-overlap engine, "kv-cache pipeline"/nanovllm/
        # engine/llava_model_runner.py:1271-1338: snapshot, a few layers per decode step, the tokens decoded
        # meanwhile appended at the end); "hold" = in place, the request sits out of the decode batches until
        # its last layer is done (no extra blocks).  Shadow needs merge compression and free blocks for the
        # compressed copy, and falls back to hold per request when it has neither.
        # several decode steps per engine step, launched back to back with one host synchronisation (only while no
        # request is waiting, compressing or about to finish; see `step`)
        self.decode_steps_per_call = max(1, int(config.extra.get("decode_steps_per_call", 1)))
        if decode_overlap not in ("shadow", "hold"):
            raise ValueError("decode_overlap must be 'shadow' or 'hold'")
        self.decode_overlap = decode_overlap
        self._pending: Dict[int, PendingCompression] = {}
        self._pending_compression_events = self._pending     # name used by the reference's benches
        self.async_manager = AsyncCompressionManager(self)
        self.model_runner._async_manager = self.async_manager   # where the reference keeps it
        self.stats = StepStats()
        self.trace: Optional[StepTrace] = None
        self._timing: Optional[dict] = None
        # host-side race detector for the pool (utils/stream_check.py): every launch that touches blocks is checked
        # against the stream order that the events below establish
        if check_streams is None:
            check_streams = os.environ.get("FC_CHECK_STREAMS", "0") == "1"
        self.stream_check = None
        if check_streams:
            from ..utils.stream_check import StreamOrderChecker
            self.stream_check = StreamOrderChecker()
            self.stream_check.name_stream(r.main_stream, "main")
        atexit.register(self.exit)

    # ------------------------------------------------------------------ set-up
    def _load_tokenizer(self, model: str) -> None:
        try:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(model, use_fast=True, trust_remote_code=False)
        except Exception:
            self.tokenizer = None
        try:
            from transformers import AutoProcessor
            self.processor = AutoProcessor.from_pretrained(model, trust_remote_code=False)
        except Exception:
            self.processor = None

    def exit(self) -> None:
        """Release the device memory of this engine (CUDA graphs, KV pool, weights).  The engine cannot
        step afterwards.  Also drops the interpreter-exit hook, which would otherwise keep the engine
        (and its pool) alive for the rest of the process."""
        atexit.unregister(self.exit)
        r = getattr(self, "model_runner", None)
        if r is not None:
            r.exit()

    # ---------------------------------------------------------------- requests
    def preprocess_image(self, image: Any) -> Tuple[torch.Tensor, Any]:
        """PIL image / array / tensor -> (pixel tensor on the model device, metadata)."""
        return self.model_runner.model.preprocess_image(image, self.model_runner.device,
                                                        self.model_runner.dtype, self.processor)

    def add_request(self, prompt: Union[str, List[int]], sampling_params: Optional[SamplingParams] = None,
                    image: Any = None) -> Sequence:
        sp = sampling_params or SamplingParams()
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("no tokenizer is loaded: pass token ids")
            prompt = self.tokenizer.encode(prompt)
        prompt = list(prompt)
        n_img, img_pos, pixels, meta = 0, -1, None, None
        if image is not None:
            if not self.model_runner.is_multimodal:
                raise ValueError("this model takes no images")
            pixels, meta = self.preprocess_image(image)
            n_img = self.model_runner.model.num_image_rows(meta)
            tok = self.image_token_id
            if tok in prompt:
                img_pos = prompt.index(tok)
            else:                                   # no placeholder given: put the image first
                prompt = [tok] + prompt
                img_pos = 0
        seq = Sequence(prompt, sp, num_image_tokens=n_img, image_token_pos=img_pos)
        seq.pixel_values, seq.image_meta = pixels, meta
        if seq.prompt_rows + 1 > self.config.max_model_len:
            raise ValueError(f"prompt of {seq.prompt_rows} rows exceeds max_model_len {self.config.max_model_len}")
        self.scheduler.add(seq)
        return seq

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    # ------------------------------------------------------- failures and recovery
    compression_error_policy = "skip"        # or "raise"
    last_compress_error: Optional[BaseException] = None

    def abort_request(self, seq_id: int) -> bool:
        """Cancel one request (waiting, running or mid-compression).  True if it was live."""
        sch = self.scheduler
        for seq in list(sch.waiting) + list(sch.running):
            if seq.seq_id == seq_id:
                ok = sch.abort(seq)       # running: `finish` orders any compression in flight first
                self._pending.pop(seq_id, None)
                self.stats.aborted += int(ok)
                return ok
        return False

    def recover(self) -> int:
        """Abort the step in flight after a failure (a device wait that ran out, a dead peer, a
        watchdog deadline): drop outstanding compressions, take every running request's blocks back
        and queue it for prefill again.  Finished requests and their outputs are untouched.  Returns
        the number of requests that will be recomputed."""
        r = self.model_runner
        if r.main_stream is not None:
            for p in self._pending.values():
                if p.event is not None:
                    self._wait(r.main_stream, p.event)
        self._pending.clear()
        r.reset_sync_state()                 # arrival counters a kernel that gave up may have left mid-count
        n = self.scheduler.requeue_running()
        self.stats.recoveries += 1
        self.scheduler.block_manager.check_invariants()
        return n

    def enable_trace(self, capacity: int = 4096, device_timing: bool = True) -> StepTrace:
        """Starts a per-step trace (kind, batch, tokens, pool state, host and device time per step); returns it.
        `llm.trace.dump(path)` writes a chrome://tracing file, `llm.trace.summary()` the totals per phase."""
        self.trace = StepTrace(capacity, device_timing)
        return self.trace

    def check_device_status(self) -> None:
        """Raise if a kernel of this package reported a wait that ran out or a bad index since the
        last call (the kernels return instead of hanging and leave a code in a status word)."""
        r = self.model_runner
        code = r.read_device_status() if hasattr(r, "read_device_status") else 0
        if code:
            from ..utils.watchdog import DeviceWaitTimeout
            raise DeviceWaitTimeout(code)


    # ------------------------------------------------------ stream order (checked when `stream_check` is set)
    def _record(self, event, stream) -> None:
        event.record(stream)
        if self.stream_check is not None:
            self.stream_check.record(event, stream)

    def _wait(self, stream, event) -> None:
        stream.wait_event(event)
        if self.stream_check is not None:
            self.stream_check.wait(stream, event)

    def _rows(self, table: Seq[int], lo: int, hi: int):
        """(block, first row, end row) of rows [lo, hi) of a request with block table `table`."""
        bs = self.scheduler.block_manager.block_size
        return [(table[i], max(lo - i * bs, 0), min(hi - i * bs, bs))
                for i in range(max(lo, 0) // bs, min(-(-hi // bs), len(table)))] if hi > lo else []

    def _note_step(self, seqs: Seq[Sequence], is_prefill: bool, decode_steps: int = 1) -> None:
        reads, writes = [], []
        for s in seqs:
            if is_prefill:
                end = s.logical_len if s.prefill_end is None else int(s.prefill_end)
                first = s.prefill_start
            else:
                first = s.kv_cache_len - 1
                end = s.kv_cache_len + decode_steps - 1
            reads += self._rows(s.block_table, 0, first)
            writes += self._rows(s.block_table, first, end)
        self.stream_check.launch(self.model_runner.main_stream, reads, writes,
                                 "prefill step" if is_prefill else "decode step")

    def _note_compress(self, stream, seqs: Seq[Sequence], rows: Seq[int], shadow: bool, what: str) -> None:
        reads, writes = [], []
        bs = self.scheduler.block_manager.block_size
        for s, n in zip(seqs, rows):
            src = self._rows(s.block_table, 0, n)
            if shadow:
                reads += src
                writes += self._rows(s.shadow_table, 0, len(s.shadow_table) * bs)
            else:
                writes += src                        # compaction in place reads and rewrites the rows
        self.stream_check.launch(stream, reads, writes, what)

    # -------------------------------------------------------------- compression
    def _on_release(self, seq: Sequence) -> None:
        """A request is about to lose its blocks: order any running compression first."""
        p = self._pending.pop(seq.seq_id, None)
        if p is not None and p.event is not None and self.model_runner.main_stream is not None:
            self._wait(self.model_runner.main_stream, p.event)
        if seq.shadow_table:                     # the half-written compressed copy goes back to the pool
            self.scheduler.block_manager.release_blocks(seq.shadow_table)
            seq.shadow_table = []
        self.model_runner.release(seq)

    def _privatize(self, seq: Sequence) -> None:
        bm = self.scheduler.block_manager
        for i in bm.private_copy_needed(seq):
            if i >= seq.kv_num_blocks:
                continue
            old, new = bm.make_private(seq, i)
            if self.stream_check is not None:
                self.stream_check.launch(self.model_runner.main_stream, [old], [new], "private copy of a shared block")
            self.model_runner.copy_block(old, new)

    def _free_compressed_blocks(self, seq: Sequence, new_len: Optional[int] = None) -> int:
        """Set the compressed length and give the tail blocks back to the pool."""
        if new_len is not None:
            seq.kv_cache_len = new_len + int(seq._pending_row)
        freed = self.scheduler.block_manager.free_blocks_after_compression(seq, seq.kv_num_blocks)
        self.stats.blocks_freed += freed
        return freed

    def _eligible(self, seq: Sequence) -> bool:
        # NONE: never considered; PENDING: waiting in the scheduler's compress queue for its turn
        return (seq.compression_state in (CompressionState.NONE, CompressionState.PENDING) and not seq.is_finished
                and seq.rows_in_pool >= max(2 * self.compression_factor, 4))

    def _compress_now(self, seqs: List[Sequence]) -> None:
        """Synchronous (main-stream) compression of `seqs`, in chunks of the compress cap."""
        r = self.model_runner
        cap = self.scheduler.compress_cap
        seqs = [s for s in seqs if self._eligible(s)]
        for i in range(0, len(seqs), cap):
            chunk = seqs[i:i + cap]
            for s in chunk:
                self._privatize(s)
            rows = [s.rows_in_pool for s in chunk]
            saved = [s._kv_cache_len for s in chunk]
            for s, n in zip(chunk, rows):
                s._kv_cache_len = n
            if self.stream_check is not None:
                self._note_compress(r.main_stream, chunk, rows, False, "compression (main stream)")
            try:
                with nvtx_range("compress"):
                    new = r.compress_kv_cache_batch(chunk, stream=r.main_stream)
            except Exception as exc:
                for s, v in zip(chunk, saved):
                    s._kv_cache_len = v
                if self.compression_error_policy == "raise":
                    raise
                # the reference's rule (nanovllm/engine/llava_model_runner.py:150-153): a failed
                # compression leaves the request uncompressed and serving continues
                self.stats.compress_failures += 1
                self.last_compress_error = exc
                for s in chunk:
                    s.compression_state = CompressionState.FAILED
                continue
            for s, n_in, n_out in zip(chunk, rows, new):
                s.compression_state = CompressionState.COMPLETED
                self._free_compressed_blocks(s, n_out)
                self.stats.compressions += 1
                self.stats.compressed_rows_in += n_in
                self.stats.compressed_rows_out += n_out

    def _launch_async(self, seqs: List[Sequence]) -> None:
        """Whole-request compression on a side stream; finalised before the request decodes."""
        r = self.model_runner
        seqs = [s for s in seqs if self._eligible(s)]
        if not seqs:
            return
        if r.main_stream is None:                 # no streams on this device: degrade to sync
            self._compress_now(seqs)
            return
        for s in seqs:
            self._privatize(s)
        stream = r.next_compress_stream()
        ready = torch.cuda.Event()
        self._record(ready, r.main_stream)
        self._wait(stream, ready)
        rows = [s.rows_in_pool for s in seqs]
        for s, n in zip(seqs, rows):
            s._kv_cache_len = n
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record(stream)
        if self.stream_check is not None:
            self._note_compress(stream, seqs, rows, False, "asynchronous compression")
        with nvtx_range("compress"):
            new = r.compress_kv_cache_batch(seqs, stream=stream)
        self._record(end, stream)
        for s, n_in, n_out in zip(seqs, rows, new):
            s.compression_state = CompressionState.IN_PROGRESS
            s.kv_cache_len = n_out + int(s._pending_row)
            self._pending[s.seq_id] = PendingCompression(s, end, start, n_in, rows=n_in, new_len=n_out)
            self.stats.compressions += 1
            self.stats.compressed_rows_in += n_in
            self.stats.compressed_rows_out += n_out

    def _shadow_blocks_for(self, seq: Sequence, rows: int) -> Optional[List[int]]:
        """Destination blocks for an out-of-place compression of `rows` rows, or None when this request has to be
        compressed in place: eviction backend, or not enough free blocks (every running request keeps one block
        in reserve for its next rows)."""
        r, bm = self.model_runner, self.scheduler.block_manager
        if self.decode_overlap != "shadow" or self.compression_backend != "mlp" or r.packed_compressor is None:
            return None
        from ..compress.ccm import ccm_output_len
        img = 0 if r.packed_compressor.single_segment else r._image_rows_of(seq)
        n_out = ccm_output_len(rows, img, self.compression_factor, r.min_seq_len)
        steps = -(-r.num_hidden_layers // max(1, r.decode_layers_per_step))
        need = -(-(n_out + steps + 2) // bm.block_size)            # the rows decoded meanwhile follow the copy
        if bm.num_free_blocks - need < len(self.scheduler.running) + 1:
            return None
        return bm.take_blocks(need)

    def _start_chunked(self, seqs: List[Sequence]) -> None:
        """Decode pipeline: compress a few layers per engine step beside decode."""
        for s in seqs:
            if not self._eligible(s):
                continue
            rows = s.rows_in_pool
            shadow = self._shadow_blocks_for(s, rows)
            s.compression_state = CompressionState.IN_PROGRESS
            if shadow is None:
                self._privatize(s)
                s.hold = True
            else:
                s.shadow_table = shadow              # the source rows are only read: shared prefix blocks stay shared
            # every chunk of one request runs on the same stream, so chunk k + 1 is ordered after chunk k
            self._pending[s.seq_id] = PendingCompression(s, None, None, rows, 0, rows, 0,
                                                         stream=self.model_runner.next_compress_stream(),
                                                         shadow=shadow is not None)

    def _advance_chunked(self) -> None:
        r = self.model_runner
        L = r.num_hidden_layers
        todo = [p for p in self._pending.values() if p.seq.hold or (p.shadow and p.next_layer < L)]
        if not todo:
            return
        step = max(1, r.decode_layers_per_step)
        groups: Dict[Tuple[int, int], List[PendingCompression]] = {}
        for p in todo:
            if p.stream is not None and not any(p.stream is c for c in r.compress_streams):
                # the streams were rebuilt for a new SM split (which synchronises the device first)
                p.stream = r.next_compress_stream()
            groups.setdefault((id(p.stream), p.next_layer, p.shadow), []).append(p)
        ready = None
        waited = set()
        for (_, first, shadow), ps in groups.items():
            stream = ps[0].stream
            if stream is not None and id(stream) not in waited:
                if ready is None:
                    ready = torch.cuda.Event()
                    self._record(ready, r.main_stream)
                self._wait(stream, ready)
                waited.add(id(stream))
            last = min(L, first + step)
            seqs = [p.seq for p in ps]
            saved = [s._kv_cache_len for s in seqs]
            for p in ps:
                p.seq._kv_cache_len = p.rows
            if self.stream_check is not None:
                self._note_compress(stream if stream is not None else r.main_stream, seqs, [p.rows for p in ps],
                                    shadow, f"compression of layers {first}-{last - 1}")
            with nvtx_range("compress_chunk"):
                new = r.compress_kv_cache_batch(seqs, first, last, stream=stream,
                                                dst_tables=[q.shadow_table for q in seqs] if shadow else None)
            # an event after every chunk: whoever takes the request's blocks away (preemption, abort, finish)
            # or reads its rows (decode) orders the main stream after the newest chunk launched so far
            ev = None
            if stream is not None:
                ev = torch.cuda.Event()
                self._record(ev, stream)
            for p, s, v, n in zip(ps, seqs, saved, new):
                s._kv_cache_len = v
                p.next_layer = last
                p.new_len = n
                p.event = ev
                if last >= L and shadow:
                    pass                         # switched in by `_finalize_pending` before the request's next decode
                elif last >= L:
                    s.hold = False
                    s.kv_cache_len = n + int(s._pending_row)
                    self.stats.compressions += 1
                    self.stats.compressed_rows_in += p.rows
                    self.stats.compressed_rows_out += n

    def _finalize_pending(self, seqs: Seq[Sequence]) -> None:
        """Before `seqs` read their KV: wait (on the device) for their compression, free tails."""
        r = self.model_runner
        for s in seqs:
            p = self._pending.get(s.seq_id)
            if p is None or s.hold:
                continue
            if p.shadow:
                if p.next_layer >= r.num_hidden_layers:
                    self._switch_to_shadow(s, p)
                continue                             # chunks still to go: the request decodes over its full rows
            if p.event is not None and r.main_stream is not None:
                self._wait(r.main_stream, p.event)
            del self._pending[s.seq_id]
            s.compression_state = CompressionState.COMPLETED
            self._free_compressed_blocks(s)

    def _switch_to_shadow(self, s: Sequence, p: PendingCompression) -> None:
        """All layers of `s` are compressed into its shadow blocks: move the rows decoded meanwhile behind them,
        make the shadow blocks the request's block table and return the original blocks.  Called right before
        the request's next decode step (whose row the scheduler has already made room for in the old table)."""
        r, bm = self.model_runner, self.scheduler.block_manager
        tail = s.rows_in_pool - p.rows                    # rows decoded while the chunks ran
        total = p.new_len + tail + int(s._pending_row)
        need = -(-total // bm.block_size)
        extra = need - len(s.shadow_table)
        if extra > bm.num_free_blocks:
            return                                   # no room right now: keep decoding over the full rows
        if extra > 0:
            s.shadow_table.extend(bm.take_blocks(extra))
        if p.event is not None and r.main_stream is not None:
            self._wait(r.main_stream, p.event)
        if self.stream_check is not None:
            self.stream_check.launch(r.main_stream, self._rows(s.block_table, p.rows, p.rows + tail),
                                     self._rows(s.shadow_table, p.new_len, p.new_len + tail),
                                     "copy of the rows decoded during compression")
        cm = torch.cuda.stream(r.main_stream) if r.main_stream is not None else None
        if cm is not None:
            with cm:
                r.copy_rows(s.block_table, p.rows, s.shadow_table, p.new_len, tail)
        else:
            r.copy_rows(s.block_table, p.rows, s.shadow_table, p.new_len, tail)
        old, s.block_table, s.shadow_table = s.block_table, s.shadow_table, []
        freed = bm.release_blocks(old) - len(s.block_table)
        s.num_cached_tokens = 0
        s.kv_cache_len = total
        s.compression_state = CompressionState.COMPLETED
        r._compressed_lens[s.seq_id] = p.new_len
        del self._pending[s.seq_id]
        self.stats.blocks_freed += max(0, freed)
        self.stats.compressions += 1
        self.stats.compressed_rows_in += p.rows
        self.stats.compressed_rows_out += p.new_len

    def _lazy_check(self) -> None:
        sch = self.scheduler
        if not sch.lazy_compress_due():
            return
        cands = [s for s in sch.lazy_candidates() if self._eligible(s)]
        if not cands:
            return
        self.stats.lazy_triggers += 1
        self._compress_now(cands)

    # ----------------------------------------------------------------------- step
    def step(self, apply_compression: Optional[bool] = None) -> Tuple[List[Tuple[int, List[int]]], int]:
        sch, r = self.scheduler, self.model_runner
        if r.model is None:
            raise RuntimeError("this engine was shut down with exit(); build a new one")
        compress = self.enable_compression if apply_compression is None else \
            (apply_compression and self.enable_compression)
        mode = self.compression_mode
        ctl = self._auto_controller if compress else None
        if compress and mode == "lazy":
            self._lazy_check()
        if compress:
            self._advance_chunked()
        prefer_decode = False
        if ctl is not None and self.auto_dual_batch:
            prefer_decode = ctl.decide_batch_type(waiting=len(sch.waiting), running=len(sch.running),
                                                  pending_compressions=len(self._pending)) == "decode"
        seqs, is_prefill = sch.schedule(prefer_decode=prefer_decode)
        self.stats.preemptions = sch.num_preemptions
        if not seqs:
            if self._pending:
                return [], 0
            raise RuntimeError("nothing to schedule")
        pipeline, use_async = self.compression_pipeline, self.async_compression
        if is_prefill and ctl is not None:
            d = ctl.decide(batch_size=len(seqs), seq_len=max(s.prompt_rows for s in seqs),
                           expected_output_len=max(1, sum(s.max_tokens for s in seqs) // len(seqs)),
                           pending_compressions=len(self._pending))
            pipeline, use_async = d.pipeline, d.async_compress
            streams_before = r.compress_streams
            r.update_streams(d.greenctx_enabled, d.sm_compress_ratio, d.sm_main_ratio, d.compression_streams)
            if self.stream_check is not None and r.compress_streams is not streams_before:
                self.stream_check.synchronize()      # new streams are built after a device synchronisation
            r.decode_layers_per_step = d.decode_layers_per_step
        if not is_prefill:
            self._finalize_pending(seqs)
        timing = self._begin_timing(ctl)
        rec = None
        if self.trace is not None:
            bm = sch.block_manager
            rec = self.trace.begin(self.stats.steps, "prefill" if is_prefill else "decode", len(seqs),
                                   sum((s.logical_len if s.prefill_end is None else s.prefill_end) - s.prefill_start
                                       for s in seqs) if is_prefill else len(seqs),
                                   len(bm.free_block_ids), len(bm.blocks), self.stats.compressions, r.main_stream)
        multi = None
        k = self._decode_steps_now(seqs, is_prefill, ctl)
        if self.stream_check is not None:
            self._note_step(seqs, is_prefill, k)
        with nvtx_range("prefill" if is_prefill else "decode"):
            if k > 1:
                multi = r.run_decode_steps(seqs, k)
            tokens = multi[0] if multi is not None else r.run(seqs, is_prefill)
        if self.stream_check is not None:
            self.stream_check.synchronize(r.main_stream)     # the sampled tokens were read back on the host
        if r.last_status:
            # a bounded wait in a kernel ran out (or an index was out of range) during this step or a compression
            # before it: the tokens cannot be trusted.  The scheduler state is as before the step's postprocess;
            # `recover()` requeues the running requests.
            code, r.last_status = r.last_status, 0
            r.read_device_status()                   # clears the word on the device
            from ..utils.watchdog import DeviceWaitTimeout
            raise DeviceWaitTimeout(code)
        if rec is not None:
            self.trace.end(rec, r.main_stream)
        self._end_timing(ctl, timing, is_prefill, seqs)
        now = time.perf_counter()
        if is_prefill:
            n_tok = sum((s.logical_len if s.prefill_end is None else s.prefill_end) - s.prefill_start for s in seqs)
            whole = [s for s in seqs if s.prefill_end is None]          # not a piece of a split prompt
            for s in whole:
                if s.first_token_time is None:
                    s.first_token_time = now
            if compress and mode in ("eager", "async") and pipeline != "none":
                # the third queue: requests that finished prefill wait here for a compression batch
                sch.enqueue_compress([s for s in whole if self._eligible(s)])
        else:
            n_tok = -len(seqs)
        if compress and mode in ("eager", "async") and pipeline != "none" and sch.compress_queue:
            # one compression batch per engine step, at most `compress_batch_size` requests (the middle number of
            # the harness' [prefill, compress, decode] caps); the rest keep their place in the queue and may
            # decode uncompressed meanwhile
            batch = [s for s in sch.schedule_compress() if self._eligible(s)]
            try:
                if pipeline == "decode":
                    self._start_chunked(batch)
                elif use_async or mode == "async":
                    self._launch_async(batch)
                else:
                    self._compress_now(batch)
            finally:
                for s in batch:                          # not taken after all, or the compressor raised
                    if s.compression_state is CompressionState.PENDING:
                        s.compression_state = CompressionState.NONE
        finished = sch.postprocess(seqs, tokens)
        extra_tokens = 0
        if multi is not None:
            # the later steps of the same launch: a request that finished in between takes no more tokens
            for toks in multi[1:]:
                live = [(s, t) for s, t in zip(seqs, toks) if not s.is_finished]
                extra_tokens += len(live)
                finished += sch.postprocess([s for s, _ in live], [t for _, t in live])
        for s in finished:
            s.finish_time = now
        st = self.stats
        st.steps += 1
        if is_prefill:
            st.prefill_steps += 1
            st.prefill_tokens += n_tok
        else:
            st.decode_steps += len(multi) if multi is not None else 1
            st.decode_tokens += len(seqs) + extra_tokens
            n_tok -= extra_tokens
        outputs = [(s.seq_id, s.completion_token_ids) for s in finished]
        self._last_finished = finished
        return outputs, n_tok

    def _decode_steps_now(self, seqs: Seq[Sequence], is_prefill: bool, ctl) -> int:
        """How many decode steps this engine step launches back to back.  More than one only when nothing else
        could want the next step: no request waiting for prefill, none compressing or queued for it, no controller,
        every request of the batch with that many tokens still to produce, and blocks for the extra rows."""
        k = self.decode_steps_per_call
        sch = self.scheduler
        if (k < 2 or is_prefill or ctl is not None or sch.waiting or self._pending or sch.compress_queue
                or self.compression_mode == "lazy" or len(seqs) < len(sch.running)):
            return 1
        if sch.block_manager.prefix_caching and not all(s.is_compressed or s.has_image for s in seqs):
            return 1                     # filled blocks of these requests are published for prefix reuse step by step
        k = min(k, min(s.max_tokens - s.num_completion_tokens for s in seqs))
        k = min(k, min(self.config.max_model_len - s.kv_cache_len for s in seqs) + 1)
        if k < 2:
            return 1
        bm = sch.block_manager
        if sum(bm.blocks_short_for(s, k - 1) for s in seqs) > bm.num_free_blocks:
            return 1
        for s in seqs:
            bm.reserve_rows(s, k - 1)
        return k

    # ---------------------------------------------------------- controller timing
    def _begin_timing(self, ctl):
        if ctl is None or self.model_runner.main_stream is None:
            return None
        if self.stats.steps % self.auto_tune_interval:
            return None
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(self.model_runner.main_stream)
        return a, b

    def _end_timing(self, ctl, timing, is_prefill: bool, seqs) -> None:
        if timing is None:
            return
        a, b = timing
        b.record(self.model_runner.main_stream)
        b.synchronize()
        ms = a.elapsed_time(b)
        # compressions whose end event has been reached feed an EWMA.  `event.query()` and the measured times
        # are rank-local; the controller's decisions (batch type, pipeline, SM split) must be the same on every
        # tensor-parallel rank, so the ranks agree on one set of numbers first
        cands = [p for p in self._pending.values()
                 if not p.reported and p.start_event is not None and p.event is not None]
        done = [bool(p.event.query()) for p in cands]
        c_ms = [p.start_event.elapsed_time(p.event) if d else 0.0 for p, d in zip(cands, done)]
        ms, done, c_ms = self._agree_on_timings(ms, done, c_ms)
        if is_prefill:
            ctl.update_prefill(ms, sum(s.prompt_rows for s in seqs))
        else:
            ctl.update_decode(ms, len(seqs))
        for p, d, t in zip(cands, done, c_ms):
            if d:
                ctl.update_compress(t, p.tokens)
                p.reported = True

    def _agree_on_timings(self, ms: float, done: List[bool], c_ms: List[float]):
        """One number per measurement for all tensor-parallel ranks: the slowest rank's step time, a
        compression counts as finished only when it has finished everywhere, and then with its longest time.
        (One small all-reduce every `auto_tune_interval` steps, only with `auto_tune` on.)"""
        if tpmod.get_tp_size() <= 1:
            return ms, done, c_ms
        import torch.distributed as dist
        vals = [ms] + [-float(d) for d in done] + list(c_ms)
        dev = self.model_runner.device if self.model_runner.device.type == "cuda" else "cpu"
        t = torch.tensor(vals, dtype=torch.float32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=tpmod.get_tp_group())
        out = t.tolist()
        n = len(done)
        return out[0], [v <= -1.0 for v in out[1:1 + n]], out[1 + n:]

    # ------------------------------------------------------------------- generate
    def generate(self, prompts: List[Union[str, List[int]]],
                 sampling_params: Union[SamplingParams, List[SamplingParams], None] = None,
                 images: Optional[List[Any]] = None, use_tqdm: bool = False,
                 apply_compression: Optional[bool] = None) -> List[dict]:
        if sampling_params is None:
            sampling_params = SamplingParams()
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        images = images or [None] * len(prompts)
        order = []
        for p, sp, im in zip(prompts, sampling_params, images):
            order.append(self.add_request(p, sp, im).seq_id)
        bar = None
        if use_tqdm:
            try:
                from tqdm.auto import tqdm
                bar = tqdm(total=len(prompts), desc="Generating", dynamic_ncols=True)
            except Exception:
                bar = None
        results: Dict[int, List[int]] = {}
        prefill_tps = decode_tps = 0.0
        while not self.is_finished():
            t = time.perf_counter()
            out, n = self.step(apply_compression)
            dt = max(time.perf_counter() - t, 1e-9)
            if n > 0:
                prefill_tps = n / dt
            elif n < 0:
                decode_tps = -n / dt
            for sid, toks in out:
                results[sid] = toks
                if bar is not None:
                    bar.update(1)
            if bar is not None:
                bar.set_postfix({"Prefill": f"{int(prefill_tps)}tok/s", "Decode": f"{int(decode_tps)}tok/s"})
        if bar is not None:
            bar.close()
        outs = []
        for sid in order:
            toks = results[sid]
            text = self.tokenizer.decode(toks) if self.tokenizer is not None else ""
            outs.append({"text": text, "token_ids": toks})
        return outs


# names of the reference's engine classes
LlavaLLMEngine = LLMEngine
