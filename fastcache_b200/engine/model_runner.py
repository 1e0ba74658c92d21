"""Model runner: owns the model, the paged KV pool, step metadata, CUDA graphs
and the compression entry points.

Parity
  * text runner     nanovllm/engine/model_runner.py:12-199 (pool sizing and
    binding :32-45, prefill/decode metadata :56-112, graph capture :155-199)
  * multimodal / compression runner  "kv-cache pipeline"/nanovllm/engine/
    llava_model_runner.py:208-1415 (model-type detection, compressor loading,
    image-expanded prefill metadata, compress batch, async compression on side
    streams, decode-overlap chunks, stream rebuilds, graph capture)

One class serves every model family here.  Differences by design: block
tables always cover image-expanded rows; compression and eviction run in the
pool (see fastcache_b200.compress.inpool); under tensor parallelism every rank
samples the same token from gathered logits with a shared seed instead of
rank 0 broadcasting it; on a CPU device the "graph" path is the same
static-buffer, padded-batch replay code with eager execution in place of
`CUDAGraph.replay()`, which keeps that path testable without a GPU.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence as Seq, Tuple

import numpy as np
import torch

from ..compress.ccm import PackedCCMWeights, load_compressor
from ..compress.inpool import ccm_compress_in_pool, evict_in_pool
from ..compress.scorers import NEEDS_QUERIES, n_kept_for, ratio_from_factor
from ..config import Config, ModelConfig, text_config_of
from ..layers.sampler import Sampler
from ..models.registry import build_model, detect_model_type
from ..parallel import tp as tpmod
from ..utils.context import reset_context, set_context
from ..utils.loader import init_random_weights, load_model
from ..utils.memory import get_gpu_memory
from .async_compression import AsyncCompressionManager  # noqa: F401  (the reference exports it from here)
from .sequence import CompressionState, Sequence  # noqa: F401  (CompressionState: the reference defines it in llava_model_runner.py:43)


def _resolve_device(config: Config) -> torch.device:
    if config.device != "auto":
        return torch.device(config.device)
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _resolve_dtype(config: Config, device: torch.device) -> torch.dtype:
    if config.dtype == "auto":
        return torch.bfloat16 if device.type == "cuda" else torch.float32
    return {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16,
            "float16": torch.float16, "fp32": torch.float32, "float32": torch.float32}[config.dtype]


class DeviceTimer:
    """Collects CUDA-event pairs around device work; `total_ms()` synchronises and sums them."""

    def __init__(self, stream=None):
        self.stream = stream
        self.pairs: List[Tuple[Any, Any]] = []
        self._open = None

    def start(self, stream=None) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream or self.stream)
        self._open = ev

    def stop(self, stream=None) -> None:
        if self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream or self.stream)
        self.pairs.append((self._open, ev))
        self._open = None

    def total_ms(self) -> float:
        torch.cuda.synchronize()
        return float(sum(a.elapsed_time(b) for a, b in self.pairs))


class ModelRunner:
    def __init__(self, config: Config, compressor_path: Optional[str] = None, compression_factor: int = 5,
                 enable_compression: bool = False, async_compression: bool = False,
                 compression_backend: str = "mlp", kvpress_method: str = "streaming_llm",
                 compression_pipeline: str = "auto", compression_streams: int = 2,
                 greenctx_enabled: bool = False, greenctx_compress_ratio: float = 0.25,
                 greenctx_main_ratio: float = 0.75, greenctx_main_stream: bool = False,
                 decode_layers_per_step: int = 4, compressor: Any = None, min_seq_len: int = 2,
                 kvpress_params: Optional[dict] = None):
        self.config = config
        self.device = _resolve_device(config)
        self.dtype = _resolve_dtype(config, self.device)
        self.block_size = config.kvcache_block_size
        self.enforce_eager = config.enforce_eager
        self.tp_size = tpmod.get_tp_size()
        self.tp_rank = tpmod.get_tp_rank()
        hf = config.hf_config
        if hf is None:
            hf = ModelConfig.from_pretrained(config.model)
            config.hf_config = hf
        self.hf_config = hf
        self.text_config = text_config_of(hf)
        self.model_type = detect_model_type(hf)
        self.is_multimodal = self.model_type in ("llava", "minicpm")

        prev = torch.get_default_dtype()
        torch.set_default_dtype(self.dtype)
        try:
            with torch.device(self.device):
                self.model = build_model(hf)
        finally:
            torch.set_default_dtype(prev)
        self.model.eval()
        self._load_weights()

        tc = self.text_config
        self.num_hidden_layers = tc.num_hidden_layers
        heads = tc.num_attention_heads
        kvh = getattr(tc, "num_key_value_heads", None) or heads
        self.head_dim = getattr(tc, "head_dim", None) or tc.hidden_size // heads
        self.total_kv_heads = kvh
        self.num_key_value_heads = max(1, kvh // self.tp_size)     # per rank
        self.num_heads_local = heads // self.tp_size
        self.image_token_len = int(getattr(self.model, "image_token_len", 0))
        self.image_token_id = getattr(self.model, "image_token_id", None)

        self.fused_comm = None
        if self.tp_size > 1 and self.device.type == "cuda" and not config.extra.get("disable_fused_comm", False):
            from ..parallel import symm
            big = 0 if config.extra.get("disable_fused_prefill", False) else config.max_num_batched_tokens
            self.fused_comm = symm.enable(int(config.extra.get("fused_comm_tokens", 512)), tc.hidden_size,
                                          self.device, max_tokens=big)
        self.sampler = Sampler(config.seed)
        # under tensor parallelism with the fused communication kernels the LM head keeps its vocabulary shard
        # and the sampler exchanges one candidate per rank: no gather of logits inside or outside the graphs
        self.local_logits = self.fused_comm is not None
        self.head = next((m for m in self.model.modules() if m.__class__.__name__ == "ParallelLMHead"), None)
        self.io = {"h2d_bytes": 0, "d2h_bytes": 0}      # host<->device traffic of the step loop
        self.timer: Optional[DeviceTimer] = None        # set by benchmarks to time device work only
        self.graph_launches: Dict[int, int] = {}
        self.last_status = 0
        self.allocate_kv_cache()

        # ------------------------------------------------------ compression
        self.enable_compression = enable_compression
        self.async_compression = async_compression
        self.compression_backend = compression_backend
        self.kvpress_method = kvpress_method
        self.kvpress_params = dict(kvpress_params or {})
        self.compression_factor = compression_factor
        self.min_seq_len = min_seq_len
        self.decode_layers_per_step = decode_layers_per_step
        self.compressor = None
        self.packed_compressor: Optional[PackedCCMWeights] = None
        self._compressed_lens: Dict[int, int] = {}
        self._window_q: Dict[int, Dict[int, torch.Tensor]] = {}
        if enable_compression and compression_backend == "kvpress":
            from ..compress.scorers import SCORERS
            if kvpress_method not in SCORERS:
                raise ValueError(f"unknown eviction method {kvpress_method!r}; have {sorted(SCORERS)}")
        if enable_compression:
            self._load_compressor(compressor_path, compressor)
        if not enable_compression or (compression_backend == "mlp" and self.packed_compressor is None):
            self.compression_pipeline = "none"
        elif compression_pipeline == "auto":
            # merge compression is GEMM work that hides under memory-bound decode;
            # eviction is cheap and goes with prefill
            self.compression_pipeline = "decode" if compression_backend == "mlp" else "prefill"
        else:
            self.compression_pipeline = compression_pipeline
        self.obs_window = int(self.kvpress_params.get("window", 64)) \
            if (enable_compression and compression_backend == "kvpress" and kvpress_method in NEEDS_QUERIES) else 0

        # ---------------------------------------------------------- streams
        self.greenctx_enabled = False
        self._greenctx_info: Dict[str, Any] = {}
        self.main_stream = None
        self.compress_streams: List[Any] = []
        self._rr = 0
        if self.device.type == "cuda":
            from ..utils.streams import build_streams
            pool = build_streams(self.device, n_compress=max(1, compression_streams),
                                 use_greenctx=greenctx_enabled, compress_ratio=greenctx_compress_ratio,
                                 main_on_greenctx=greenctx_main_stream)
            self.main_stream = pool.main
            self.compress_streams = pool.compress
            self.greenctx_enabled = pool.greenctx
            self._greenctx_info = pool.info
            self._stream_pool = pool

        # ------------------------------------------------------------ graphs
        self.graphs: Dict[int, Any] = {}
        self.graph_bs: List[int] = []
        self.graph_vars: Dict[str, torch.Tensor] = {}
        self.graph_pool = None
        if not self.enforce_eager:
            self.capture_cudagraph()

    # ------------------------------------------------------------------ setup
    def _load_weights(self) -> None:
        cfg = self.config
        random_init = bool(cfg.extra.get("random_init", False)) or not cfg.model
        if random_init:
            shapes = self.model.hf_weight_shapes(self.hf_config)
            init_random_weights(self.model, shapes, seed=cfg.seed, std=float(cfg.extra.get("init_std", 0.02)),
                                device=cfg.extra.get("init_device") or
                                (str(self.device) if self.device.type == "cuda" else "cpu"))
        else:
            load_model(self.model, cfg.model)

    def _load_compressor(self, path: Optional[str], module: Any) -> None:
        if self.compression_backend != "mlp":
            return
        try:
            if module is None:
                if path is None:
                    raise FileNotFoundError("compression_backend='mlp' needs compressor_path or a module")
                module = load_compressor(path, None, min_seq_len=self.min_seq_len,
                                         nhead=self.total_kv_heads)
            if module.n_layer != self.num_hidden_layers or module.head_dim != self.head_dim:
                raise ValueError(f"compressor is for {module.n_layer} layers x head_dim {module.head_dim}; "
                                 f"model has {self.num_hidden_layers} x {self.head_dim}")
            self.compressor = module
            self.compression_factor = module.compression_factor
            self.packed_compressor = module.pack(self.dtype, self.device)
        except Exception as exc:
            # same recovery as the reference: a compressor that cannot be loaded
            # turns compression off instead of failing the engine
            # ("kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:555-565)
            print(f"[fastcache_b200] compressor unavailable ({exc}); compression disabled")
            self.compressor = None
            self.packed_compressor = None

    def allocate_kv_cache(self) -> None:
        cfg = self.config
        L, H, D, bs = self.num_hidden_layers, self.num_key_value_heads, self.head_dim, self.block_size
        block_bytes = 2 * L * bs * H * D * torch.empty((), dtype=self.dtype).element_size()
        if cfg.num_kvcache_blocks <= 0:
            if self.device.type == "cuda":
                total, used, free = get_gpu_memory(self.device.index)
                budget = int(total * cfg.gpu_memory_utilization) - used
                need = -(-cfg.max_model_len // bs)
                if budget < need * block_bytes:
                    raise RuntimeError(
                        f"not enough device memory for the KV pool: {max(budget, 0) / 2**30:.1f} GiB left under "
                        f"gpu_memory_utilization={cfg.gpu_memory_utilization} ({used / 2**30:.1f} of "
                        f"{total / 2**30:.1f} GiB in use), one request of max_model_len={cfg.max_model_len} needs "
                        f"{need * block_bytes / 2**30:.1f} GiB; free other engines in this process "
                        f"(`llm.exit()`) or pass num_kvcache_blocks")
                cfg.num_kvcache_blocks = budget // block_bytes
            else:
                need = cfg.max_num_seqs * -(-cfg.max_model_len // bs)
                cfg.num_kvcache_blocks = max(1, min(need, (1 << 30) // block_bytes))
        self.num_blocks = cfg.num_kvcache_blocks
        self.kv_cache = torch.zeros(L, 2, self.num_blocks, H, bs, D, dtype=self.dtype, device=self.device)
        i = 0
        for module in self.model.modules():
            if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
                module.k_cache = self.kv_cache[i, 0]
                module.v_cache = self.kv_cache[i, 1]
                i += 1
        if i != L:
            raise RuntimeError(f"bound {i} attention layers, expected {L}")

    # --------------------------------------------------------------- metadata
    def _to_dev(self, arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
        t = torch.from_numpy(arr).to(dtype)
        if self.device.type == "cuda":
            self.io["h2d_bytes"] += t.numel() * t.element_size()
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def _block_table_array(self, seqs: Seq[Sequence], width: Optional[int] = None) -> np.ndarray:
        width = width or max(len(s.block_table) for s in seqs)
        bt = np.full((len(seqs), width), -1, dtype=np.int32)
        for i, s in enumerate(seqs):
            bt[i, : len(s.block_table)] = s.block_table
        return bt

    def prepare_prefill(self, seqs: Seq[Sequence]):
        bs = self.block_size
        ids: List[np.ndarray] = []
        pos: List[np.ndarray] = []
        slots: List[np.ndarray] = []
        cu_q = [0]
        kv_lens = []
        image_rows: List[Tuple[int, int, int]] = []      # (seq index, first flat row, count)
        max_q = max_k = 0
        for si, s in enumerate(seqs):
            toks = np.asarray(s.token_ids, dtype=np.int64)
            if s.has_image:
                p = s.image_token_pos
                toks = np.concatenate([toks[:p], np.full(s.num_image_tokens, toks[p], dtype=np.int64),
                                       toks[p + 1:]])
            start = s.prefill_start
            n = toks.shape[0] if s.prefill_end is None else int(s.prefill_end)     # a piece of a split prompt
            rows = np.arange(start, n, dtype=np.int64)
            if s.has_image:
                image_rows.append((si, cu_q[-1] + s.image_token_pos - start, s.num_image_tokens))
            ids.append(toks[start:n])
            pos.append(rows)
            table = np.asarray(s.block_table, dtype=np.int64)
            slots.append(table[rows // bs] * bs + rows % bs)
            cu_q.append(cu_q[-1] + n - start)
            kv_lens.append(n)
            max_q = max(max_q, n - start)
            max_k = max(max_k, n)
        input_ids = self._to_dev(np.concatenate(ids), torch.int64)
        positions = self._to_dev(np.concatenate(pos), torch.int64)
        slot_mapping = self._to_dev(np.concatenate(slots), torch.int32)
        cu = self._to_dev(np.asarray(cu_q, dtype=np.int32), torch.int32)
        kvl = self._to_dev(np.asarray(kv_lens, dtype=np.int32), torch.int32)
        block_tables = self._to_dev(self._block_table_array(seqs), torch.int32)
        window = None
        if self.obs_window > 0:
            idx = []
            for i in range(len(seqs)):
                q_len = cu_q[i + 1] - cu_q[i]
                w = min(self.obs_window, q_len)
                idx.append(np.arange(cu_q[i + 1] - w, cu_q[i + 1], dtype=np.int64))
            window = {"indices": self._to_dev(np.concatenate(idx), torch.int64), "q": {},
                      "counts": [len(x) for x in idx]}
        set_context(True, cu, cu, max_q, max_k, slot_mapping, kvl, block_tables, window_q=window,
                    obs_window=self.obs_window)
        return input_ids, positions, image_rows

    def prepare_decode(self, seqs: Seq[Sequence]):
        bs = self.block_size
        n = len(seqs)
        ids = np.empty(n, dtype=np.int64)
        pos = np.empty(n, dtype=np.int64)
        slots = np.empty(n, dtype=np.int32)
        lens = np.empty(n, dtype=np.int32)
        mode = self.config.position_mode
        for i, s in enumerate(seqs):
            ids[i] = s.last_token
            pos[i] = s.next_position(mode)
            kv = s.kv_cache_len
            lens[i] = kv
            slots[i] = s.block_table[(kv - 1) // bs] * bs + (kv - 1) % bs
        return ids, pos, slots, lens, self._block_table_array(seqs)

    # ------------------------------------------------------------------ forward
    def _forward(self, input_ids: torch.Tensor, positions: torch.Tensor,
                 seqs: Optional[Seq[Sequence]] = None, image_rows=None, local_logits: bool = False) -> torch.Tensor:
        if self.fused_comm is not None:
            self.fused_comm.begin_forward()
        if self.is_multimodal:
            pixel = None
            if image_rows:
                pixel = [(seqs[si].pixel_values, seqs[si].image_meta, row, cnt) for si, row, cnt in image_rows]
            hidden = self.model(input_ids, positions, images=pixel)
        else:
            hidden = self.model(input_ids, positions)
        return self._logits(hidden, local_logits)

    def _logits(self, hidden: torch.Tensor, local: bool) -> torch.Tensor:
        """Logits over the whole vocabulary, or (local) over this rank's vocabulary shard."""
        if not local:
            return self.model.compute_logits(hidden)
        from ..layers import embed_head
        prev = embed_head.set_local_logits(True)
        try:
            return self.model.compute_logits(hidden)
        finally:
            embed_head.set_local_logits(prev)

    @torch.inference_mode()
    def run_prefill(self, seqs: Seq[Sequence], local_logits: bool = False) -> torch.Tensor:
        input_ids, positions, image_rows = self.prepare_prefill(seqs)
        from ..utils.context import get_context
        ctx = get_context()
        if self.timer is not None:
            self.timer.start(self.main_stream)
        logits = self._forward(input_ids, positions, seqs, image_rows, local_logits=local_logits)
        if ctx.window_q is not None:
            counts = ctx.window_q["counts"]
            offs = np.concatenate([[0], np.cumsum(counts)])
            for i, s in enumerate(seqs):
                self._window_q[s.seq_id] = {l: q[offs[i]:offs[i + 1]] for l, q in ctx.window_q["q"].items()}
        return logits

    def _graph_bucket(self, n: int) -> Optional[int]:
        for b in self.graph_bs:
            if b >= n:
                return b
        return None

    @torch.inference_mode()
    def run_decode(self, seqs: Seq[Sequence], local_logits: bool = False) -> torch.Tensor:
        """Logits of one decode step.  `local_logits` (tensor parallelism with the fused kernels): this rank's
        vocabulary shard; the CUDA graphs are captured in that form."""
        ids, pos, slots, lens, bt = self.prepare_decode(seqs)
        n = len(seqs)
        bucket = None if self.enforce_eager else self._graph_bucket(n)
        if bucket is None or bt.shape[1] > self.graph_vars["block_tables"].shape[1]:
            set_context(False, slot_mapping=self._to_dev(slots, torch.int32),
                        context_lens=self._to_dev(lens, torch.int32),
                        block_tables=self._to_dev(bt, torch.int32),
                        attn_workspace=getattr(self, "attn_workspace", None))
            ids_d, pos_d = self._to_dev(ids, torch.int64), self._to_dev(pos, torch.int64)
            if self.timer is not None:
                self.timer.start(self.main_stream)
            return self._forward(ids_d, pos_d, local_logits=local_logits)
        gv = self.graph_vars
        h = self._staging
        h["input_ids"][:n] = torch.from_numpy(ids)
        h["input_ids"][n:bucket] = 0
        h["positions"][:n] = torch.from_numpy(pos)
        h["positions"][n:bucket] = 0
        h["slot_mapping"][:n] = torch.from_numpy(slots)
        h["slot_mapping"][n:bucket] = -1
        h["context_lens"][:n] = torch.from_numpy(lens)
        h["context_lens"][n:bucket] = 0
        h["block_tables"][:bucket].fill_(0)
        h["block_tables"][:n, : bt.shape[1]] = torch.from_numpy(np.maximum(bt, 0))
        for k in ("input_ids", "positions", "slot_mapping", "context_lens", "block_tables"):
            gv[k][:bucket].copy_(h[k][:bucket], non_blocking=True)
            if self.device.type == "cuda":
                self.io["h2d_bytes"] += h[k][:bucket].numel() * h[k].element_size()
        if self.timer is not None:
            self.timer.start(self.main_stream)
        self._replay(bucket)
        logits = gv["logits"][:n]
        if self.local_logits and not local_logits:          # the graphs hold shards: gather for a caller who asked
            logits = tpmod.tp_all_gather(logits, dim=-1)[:, : self.text_config.vocab_size]
        return logits

    def _replay(self, bucket: int) -> None:
        g = self.graphs[bucket]
        if g is None:                       # CPU: same static buffers, eager execution
            self._decode_on_static(bucket)
        else:
            g.replay()
            from .. import ops
            ops.COUNTERS["launches"] += self.graph_launches.get(bucket, 0)

    def _decode_on_static(self, bucket: int) -> None:
        gv = self.graph_vars
        set_context(False, slot_mapping=gv["slot_mapping"][:bucket], context_lens=gv["context_lens"][:bucket],
                    block_tables=gv["block_tables"][:bucket],
                    attn_workspace=getattr(self, "attn_workspace", None))
        gv["logits"][:bucket] = self._forward(gv["input_ids"][:bucket], gv["positions"][:bucket],
                                              local_logits=self.local_logits)

    @torch.inference_mode()
    def capture_cudagraph(self) -> None:
        cfg = self.config
        max_bs = min(cfg.max_num_seqs, cfg.decode_batch_size or cfg.max_num_seqs, 512)
        max_blocks = -(-cfg.max_model_len // self.block_size) + 1
        dev = self.device
        vocab = self.head.per_rank if (self.local_logits and self.head is not None) else self.text_config.vocab_size
        self.graph_vars = {
            "input_ids": torch.zeros(max_bs, dtype=torch.int64, device=dev),
            "positions": torch.zeros(max_bs, dtype=torch.int64, device=dev),
            "slot_mapping": torch.full((max_bs,), -1, dtype=torch.int32, device=dev),
            "context_lens": torch.zeros(max_bs, dtype=torch.int32, device=dev),
            "block_tables": torch.zeros(max_bs, max_blocks, dtype=torch.int32, device=dev),
            "logits": torch.zeros(max_bs, vocab, dtype=self.dtype, device=dev),
        }
        pin = dev.type == "cuda"
        self._staging = {k: torch.zeros(v.shape, dtype=v.dtype, pin_memory=pin)
                         for k, v in self.graph_vars.items() if k != "logits"}
        buckets = [b for b in (1, 2, 4, 8) if b <= max_bs] + list(range(16, max_bs + 1, 16))
        if max_bs not in buckets:
            buckets.append(max_bs)
        self.graph_bs = sorted(set(buckets))
        if dev.type != "cuda":
            self.graphs = {b: None for b in self.graph_bs}
            return
        stream = self.main_stream or torch.cuda.current_stream()
        with torch.cuda.stream(stream):
            for b in reversed(self.graph_bs):
                self._decode_on_static(b)            # warm-up (allocations, lazy init)
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                from .. import ops
                before = ops.COUNTERS["launches"]
                with torch.cuda.graph(g, pool=self.graph_pool, stream=stream):
                    self._decode_on_static(b)
                self.graph_launches[b] = ops.COUNTERS["launches"] - before
                if self.graph_pool is None:
                    self.graph_pool = g.pool()
                self.graphs[b] = g
        stream.synchronize()
        reset_context()

    # --------------------------------------------------------------------- run
    def _temperatures(self, seqs: Seq[Sequence]) -> torch.Tensor:
        return self._to_dev(np.asarray([s.temperature for s in seqs], dtype=np.float32), torch.float32)

    @torch.inference_mode()
    def run_decode_steps(self, seqs: Seq[Sequence], k: int) -> Optional[List[List[int]]]:
        """`k` decode steps launched back to back, one host synchronisation at the end: returns the k lists of
        sampled tokens, or None when the batch cannot take the static-buffer path (the caller then steps once).

        Positions, context lengths and slots of the later steps do not depend on the sampled tokens, so the host
        prepares them for all k steps at once; between the steps only device-side copies run (the sampled tokens
        become the next input ids, the step's metadata rows go into the graph's static buffers).  The block tables
        must already cover `k - 1` rows beyond the one the first step writes."""
        if self.enforce_eager or k < 2:
            return None
        n = len(seqs)
        bucket = self._graph_bucket(n)
        ids, pos, slots, lens, bt = self.prepare_decode(seqs)
        if bucket is None or bt.shape[1] > self.graph_vars["block_tables"].shape[1]:
            return None
        bs = self.block_size
        steps = np.arange(k, dtype=np.int64)[:, None]
        pos_k = np.zeros((k, bucket), dtype=np.int64)
        lens_k = np.zeros((k, bucket), dtype=np.int32)
        slots_k = np.full((k, bucket), -1, dtype=np.int32)
        pos_k[:, :n] = pos[None, :] + steps
        lens_k[:, :n] = lens[None, :].astype(np.int64) + steps
        rows = lens_k[:, :n].astype(np.int64) - 1
        slots_k[:, :n] = bt[np.arange(n)[None, :], rows // bs].astype(np.int64) * bs + rows % bs
        cm = torch.cuda.stream(self.main_stream) if self.main_stream is not None else _Null()
        with cm:
            local = self.local_logits and self.head is not None
            gv, h = self.graph_vars, self._staging
            h["input_ids"][:n] = torch.from_numpy(ids)
            h["input_ids"][n:bucket] = 0
            h["block_tables"][:bucket].fill_(0)
            h["block_tables"][:n, : bt.shape[1]] = torch.from_numpy(np.maximum(bt, 0))
            for key in ("input_ids", "block_tables"):
                gv[key][:bucket].copy_(h[key][:bucket], non_blocking=True)
                if self.device.type == "cuda":
                    self.io["h2d_bytes"] += h[key][:bucket].numel() * h[key].element_size()
            pos_d = self._to_dev(pos_k, torch.int64)
            lens_d = self._to_dev(lens_k, torch.int32)
            slots_d = self._to_dev(slots_k, torch.int32)
            temps = self._temperatures(seqs)
            if self.timer is not None:
                self.timer.start(self.main_stream)
            outs = []
            for j in range(k):
                gv["positions"][:bucket].copy_(pos_d[j], non_blocking=True)
                gv["context_lens"][:bucket].copy_(lens_d[j], non_blocking=True)
                gv["slot_mapping"][:bucket].copy_(slots_d[j], non_blocking=True)
                if j > 0:
                    gv["input_ids"][:n].copy_(outs[-1][:n], non_blocking=True)
                self._replay(bucket)
                logits = gv["logits"][:n]
                if local:
                    tokens = self.sampler.forward_sharded(logits, temps, self.fused_comm, self.head.vocab_start,
                                                          self.head.num_embeddings)
                else:
                    if self.local_logits:
                        logits = tpmod.tp_all_gather(logits, dim=-1)[:, : self.text_config.vocab_size]
                    tokens = self.sampler(logits, temps, with_status=True)
                outs.append(tokens)
            if self.timer is not None:
                self.timer.stop(self.main_stream)
            table = torch.stack(outs).tolist()
            self.io["d2h_bytes"] += 8 * k * (n + 1)
        reset_context()
        self.last_status = 0
        for row in table:
            code = int(row.pop())
            if code and not self.last_status:
                self.last_status = code
        return table

    def run(self, seqs: Seq[Sequence], is_prefill: bool, **_ignored) -> List[int]:
        """One model step for a batch; returns the sampled token per request."""
        cm = torch.cuda.stream(self.main_stream) if self.main_stream is not None else _Null()
        with cm:
            local = self.local_logits and self.head is not None
            logits = self.run_prefill(seqs, local) if is_prefill else self.run_decode(seqs, local)
            temps = self._temperatures(seqs)
            if local:
                tokens = self.sampler.forward_sharded(logits, temps, self.fused_comm, self.head.vocab_start,
                                                      self.head.num_embeddings)
            else:
                tokens = self.sampler(logits, temps, with_status=True)
            if self.timer is not None:
                self.timer.stop(self.main_stream)
            out = tokens.tolist()
            self.io["d2h_bytes"] += 8 * len(out)
        reset_context()
        # the last entry is the device status word: a kernel wait that ran out, or an index that was out of
        # range, since the status was last cleared (0 on the CPU and in a clean step)
        self.last_status = int(out.pop())
        return out

    # ------------------------------------------------------------- compression
    def compressed_len_for(self, seq: Sequence) -> int:
        n = seq.kv_cache_len
        if self.compression_backend == "mlp":
            img = self._image_rows_of(seq)
            if self.packed_compressor.single_segment:
                img = 0
            from ..compress.ccm import ccm_output_len
            return ccm_output_len(n, img, self.compression_factor, self.min_seq_len)
        return n_kept_for(n, ratio_from_factor(self.compression_factor))

    @staticmethod
    def _image_rows_of(seq: Sequence) -> int:
        return seq.image_token_pos + seq.num_image_tokens if seq.has_image else 0

    @torch.inference_mode()
    def compress_kv_cache_batch(self, seqs: Seq[Sequence], layer_start: int = 0,
                                layer_end: Optional[int] = None, stream: Any = None,
                                dst_tables: Optional[List[List[int]]] = None) -> List[int]:
        """Compress the pool rows of `seqs` in place; returns the new row counts.  With `dst_tables` (merge
        compression only) the result goes to those blocks and the requests' own rows stay as they are.

        Does not touch scheduler state: the engine updates `seq.kv_cache_len`
        and frees the tail blocks once the work is ordered before their reuse.
        """
        if not seqs:
            return []
        tables = [s.block_table for s in seqs]
        lens = [s.kv_cache_len for s in seqs]
        cm = torch.cuda.stream(stream) if stream is not None else _Null()
        timed = self.timer is not None and (stream is None or stream is self.main_stream)
        if timed:
            self.timer.start(stream)
        with cm:
            if self.compression_backend == "mlp":
                if self.packed_compressor is None:
                    raise RuntimeError("no compressor loaded")
                imgs = [self._image_rows_of(s) for s in seqs]
                new = ccm_compress_in_pool(self.kv_cache, tables, lens, imgs, self.packed_compressor,
                                           layer_start, layer_end, dst_tables)
            else:
                if dst_tables is not None:
                    raise ValueError("eviction compacts in place: no destination blocks")
                ratio = ratio_from_factor(self.compression_factor)
                kept = [n_kept_for(n, ratio) for n in lens]
                wq = None
                if self.kvpress_method in NEEDS_QUERIES:
                    wq = [self._window_q.get(s.seq_id) for s in seqs]
                new = evict_in_pool(self.kv_cache, tables, lens, self.kvpress_method, kept, wq,
                                    self.kvpress_params, layer_start, layer_end)
        if timed:
            self.timer.stop(stream)
        full = (layer_start == 0 and (layer_end is None or layer_end >= self.num_hidden_layers))
        for s, n in zip(seqs, new):
            if full or (layer_end is not None and layer_end >= self.num_hidden_layers):
                self._compressed_lens[s.seq_id] = n
                self._window_q.pop(s.seq_id, None)
        return new

    def get_compressed_block_count(self, seq_id: int) -> int:
        n = self._compressed_lens.get(seq_id)
        return 0 if n is None else -(-n // self.block_size)

    def copy_block(self, src: int, dst: int) -> None:
        self.kv_cache[:, :, dst].copy_(self.kv_cache[:, :, src])

    def copy_rows(self, src_table: Seq[int], src_row: int, dst_table: Seq[int], dst_row: int, count: int) -> None:
        """Rows [src_row, src_row + count) of one request (all layers, K and V) to rows [dst_row, ...) of another
        block table.  Used once per request when an out-of-place compression is switched in: the few rows decoded
        meanwhile move behind the compressed ones."""
        if count <= 0:
            return
        bs = self.block_size
        dev = self.kv_cache.device
        r = torch.arange(count)
        src, dst = r + src_row, r + dst_row
        sb = torch.as_tensor(src_table, dtype=torch.long)[src // bs].to(dev)
        db = torch.as_tensor(dst_table, dtype=torch.long)[dst // bs].to(dev)
        so, do = (src % bs).to(dev), (dst % bs).to(dev)
        self.kv_cache[:, :, db, :, do] = self.kv_cache[:, :, sb, :, so]

    def read_device_status(self) -> int:
        """Status word the kernels write when a bounded wait runs out or an index is out of range
        (0 = clean).  Reading it synchronises with the device and clears it."""
        dev = torch.device(self.device)
        if dev.type != "cuda":
            return 0
        from .. import ops
        return int(ops.ext().read_status(dev.index if dev.index is not None else torch.cuda.current_device()))

    def reset_sync_state(self) -> None:
        """After a device wait ran out: wait for the device, then zero the in-kernel barrier words and split-K
        counters of this device's streams (a kernel that gave up may have left them mid-count)."""
        dev = torch.device(self.device)
        if dev.type != "cuda":
            return
        from .. import ops
        torch.cuda.synchronize(dev)
        ops.ext().reset_sync_state(dev.index if dev.index is not None else torch.cuda.current_device())

    def release(self, seq: Sequence) -> None:
        self._compressed_lens.pop(seq.seq_id, None)
        self._window_q.pop(seq.seq_id, None)

    def next_compress_stream(self):
        if not self.compress_streams:
            return None
        s = self.compress_streams[self._rr % len(self.compress_streams)]
        self._rr += 1
        return s

    def update_streams(self, use_greenctx: bool, sm_compress_ratio: float, sm_main_ratio: float = 0.0,
                       num_streams: Optional[int] = None) -> None:
        """Rebuild the compression streams for a new SM split (controller decision)."""
        if self.device.type != "cuda":
            return
        from ..utils.streams import build_streams
        info = self._greenctx_info
        same = (use_greenctx == self.greenctx_enabled and
                abs(info.get("compress_ratio", -1.0) - sm_compress_ratio) < 1e-3 and
                (num_streams is None or num_streams == len(self.compress_streams)))
        if same:
            return
        torch.cuda.synchronize(self.device)
        pool = build_streams(self.device, n_compress=num_streams or max(1, len(self.compress_streams)),
                             use_greenctx=use_greenctx, compress_ratio=sm_compress_ratio,
                             main_on_greenctx=False, reuse_main=self.main_stream)
        self.compress_streams = pool.compress
        self.greenctx_enabled = pool.greenctx
        self._greenctx_info = pool.info
        self._stream_pool = pool

    # ------------------------------------------------- reference runner surface
    # Method names of the reference's multimodal runner ("kv-cache pipeline"/nanovllm/engine/
    # llava_model_runner.py:621-629, :756-790, :879-891, :998-1005, :1140-1352).  The policies they
    # drive (side-stream and layer-chunked compression) live in the engine here, because they
    # change scheduler and block-manager state; the runner methods forward to the engine that
    # owns this runner.
    def _owner(self):
        mgr = getattr(self, "_async_manager", None)
        if mgr is None:
            raise RuntimeError("this runner is not attached to an engine")
        return mgr.engine

    def preare_block_tables(self, seqs: Seq[Sequence]) -> torch.Tensor:      # (sic) the reference's spelling
        return self._to_dev(self._block_table_array(seqs), torch.int32)

    prepare_block_tables = preare_block_tables

    def prepare_sample(self, seqs: Seq[Sequence]) -> torch.Tensor:
        return self._temperatures(seqs)

    @torch.inference_mode()
    def run_model(self, input_ids: torch.Tensor, positions: torch.Tensor, is_prefill: bool,
                  pixel_values: Any = None) -> torch.Tensor:
        """Eager forward to logits on metadata already set by `prepare_prefill` / `prepare_decode`.
        `pixel_values`: the `images` list the multimodal models take ((pixels, meta, row, count))."""
        if self.fused_comm is not None:
            self.fused_comm.begin_forward()
        if self.is_multimodal:
            hidden = self.model(input_ids, positions, images=pixel_values)
        else:
            hidden = self.model(input_ids, positions)
        return self.model.compute_logits(hidden)

    def get_blocks_to_free(self, seq_id: int) -> List[int]:
        """Tail blocks a compressed request no longer needs (empty once the engine has freed them)."""
        keep = self.get_compressed_block_count(seq_id)
        if keep <= 0:
            return []
        for s in self._owner().scheduler.running:
            if s.seq_id == seq_id:
                return list(s.block_table[max(keep, s.kv_num_blocks):])
        return []

    def reset_graph_vars(self) -> None:
        for name, t in getattr(self, "graph_vars", {}).items():
            if name == "slot_mapping":
                t.fill_(-1)
            elif name != "logits":
                t.zero_()

    def start_background_compression(self, seqs: Seq[Sequence], compress_stream: Any = None):
        """Whole-request compression on a compression stream; returns (start_event, end_event) of the
        launch, or None when nothing was eligible or the device has no streams."""
        eng = self._owner()
        before = set(eng._pending)
        if compress_stream is not None and compress_stream in self.compress_streams:
            self._rr = self.compress_streams.index(compress_stream)
        eng._launch_async(list(seqs))
        new = [p for sid, p in eng._pending.items() if sid not in before]
        return (new[0].start_event, new[0].event) if new else None

    def update_decode_overlap_engine(self, layers_per_step: int) -> bool:
        """Layers compressed per engine step in the decode pipeline.  Refused (False) while chunked
        compressions are in flight, as in the reference."""
        layers_per_step = max(1, int(layers_per_step))
        if layers_per_step == self.decode_layers_per_step:
            return True
        mgr = getattr(self, "_async_manager", None)
        if mgr is not None and any(p.seq.hold or (p.shadow and p.next_layer < self.num_hidden_layers)
                                   for p in mgr.engine._pending.values()):
            return False
        if self.compression_backend == "mlp" and self.packed_compressor is None:
            return False
        self.decode_layers_per_step = layers_per_step
        return True

    def get_next_compress_stream(self):
        return self.next_compress_stream()

    def start_decode_overlap_compression(self, seqs: Seq[Sequence]) -> None:
        self._owner()._start_chunked(list(seqs))

    def step_decode_overlap_compression(self, seqs: Seq[Sequence]) -> List[Sequence]:
        """Launch the next layer chunk of every held request; returns those of `seqs` whose last
        chunk has now been launched (their blocks are freed when they next decode)."""
        eng = self._owner()
        L = self.num_hidden_layers

        def running(s):
            p = eng._pending.get(s.seq_id)
            return s.hold or (p is not None and p.shadow and p.next_layer < L)

        before = {s.seq_id for s in seqs if running(s)}
        eng._advance_chunked()
        return [s for s in seqs if s.seq_id in before and not running(s)]

    @staticmethod
    def wait_compression(event: Any) -> None:
        if event is not None:
            event.synchronize()

    def clear_compressed_lens(self, seq_ids: Optional[Seq[int]] = None) -> None:
        if seq_ids is None:
            self._compressed_lens.clear()
        else:
            for sid in seq_ids:
                self._compressed_lens.pop(sid, None)

    def exit(self) -> None:
        """Wait for the device, then drop everything that holds device memory: graphs and their
        static buffers, the KV pool (and the layers' views of it), the weights."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.graphs.clear()
        self.graph_pool = None
        self.graph_vars = {}
        self._staging = {}
        model = getattr(self, "model", None)
        if model is not None:
            for module in model.modules():
                if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
                    module.k_cache = module.v_cache = None
        self.kv_cache = None
        self.model = None
        self.packed_compressor = None
        self._window_q.clear()


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# name used by the reference's multimodal engine
LlavaModelRunner = ModelRunner
