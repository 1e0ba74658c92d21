"""Three-queue scheduler: prefill, compress, decode.

Parity
  * text scheduler with prefill-first batching, token / sequence caps,
    decode-time preemption and the `prefer_decode` flip used for dual-batch
    alternation: "kv-cache pipeline"/nanovllm/engine/scheduler.py:9-95
  * multimodal rule (an image request is prefetched alone):
    "kv-cache pipeline"/nanovllm/engine/llava_scheduler.py:65-86 — kept as an
    option (`one_image_per_prefill`), off by default because this build's
    vision tower takes a batch of images
  * per-stage batch caps [prefill, compress, decode] of the HF harness
    (scripts/llava_testcon2.6.py:2095-2100, configs/experiments.yaml:38)
  * lazy trigger "compress every uncompressed running request when the pool is
    nearly full" (nanovllm_fastapi_server.py:98-145)

The compress queue is explicit here: a request that finished prefill and is
eligible for compression is parked in `compress_queue` (`enqueue_compress`,
called by the engine after every prefill step) until the engine takes a
compression batch of at most `compress_batch_size` requests
(`schedule_compress`, once per engine step).  A queued request can decode
meanwhile — the runner orders the pool accesses — so the queue is a work
list, not a state that blocks the request.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, Deque, List, Optional, Tuple

from ..config import Config
from .block_manager import BlockManager
from .sequence import CompressionState, Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config: Config):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.prefill_cap = config.prefill_batch_size or config.max_num_seqs
        self.compress_cap = config.compress_batch_size or config.max_num_seqs
        self.decode_cap = config.decode_batch_size or config.max_num_seqs
        self.lazy_threshold = config.lazy_occupancy_threshold
        self.chunk_min = int(getattr(config, "chunked_prefill_tokens", 0) or 0)
        # rows kept for the last piece of a split prompt (the scorers' observation window reads them)
        self.chunk_tail = 64
        self._piece_last = False         # the previous step ran a piece of a split prompt
        self.one_image_per_prefill = bool(config.extra.get("one_image_per_prefill", False))
        self.block_manager = BlockManager(config.num_kvcache_blocks, config.kvcache_block_size,
                                          prefix_caching=config.prefix_caching)
        self.waiting: Deque[Sequence] = deque()
        self.running: Deque[Sequence] = deque()
        self.compress_queue: Deque[Sequence] = deque()
        self.num_preemptions = 0
        # called with a sequence that loses its blocks (lets the runner drop
        # per-request device state)
        self.on_release: Optional[Callable[[Sequence], None]] = None

    # ------------------------------------------------------------------ queues
    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    # ----------------------------------------------------------------- prefill
    def _schedule_prefill(self) -> List[Sequence]:
        """Requests from the head of `waiting` while they fit the step's token budget.  With
        `chunked_prefill_tokens` set, a text prompt that does not fit the rest of the budget is split: the
        piece that fits runs now, the request keeps its blocks and its place at the head of `waiting`, and
        later steps continue where it stopped (`Sequence.num_computed_tokens`); only the last piece samples
        a token and moves the request to `running`."""
        picked: List[Sequence] = []
        tokens = 0
        while self.waiting and len(picked) < self.prefill_cap \
                and len(self.running) + len(picked) < self.max_num_seqs:
            seq = self.waiting[0]
            if self.one_image_per_prefill and seq.has_image and picked:
                break
            room = self.max_num_batched_tokens - tokens
            rows = seq.prompt_rows + seq.num_completion_tokens
            cost = rows - seq.prefill_start
            if cost > room and self._piece(seq, cost, room) <= 0:
                break
            if not seq.block_table:             # first time: a request whose earlier pieces ran keeps its blocks
                if not self.block_manager.can_allocate(seq):
                    break
                self.block_manager.allocate(seq)
                cost = rows - seq.prefill_start             # prefix-cache hits shorten it
            piece = self._piece(seq, cost, room) if cost > room else 0
            if cost > room and piece <= 0:
                break                            # the blocks stay with the request; it is tried again next step
            if piece > 0:
                seq.prefill_end = seq.prefill_start + piece
                # rows beyond this piece do not exist yet: their blocks must not be found through the prefix cache
                self.block_manager.unpublish_unwritten(seq, seq.prefill_end)
                self.running.extend(picked)
                return picked + [seq]
            seq.prefill_end = None
            tokens += cost
            seq.status = SequenceStatus.RUNNING
            self.waiting.popleft()
            picked.append(seq)
            if self.one_image_per_prefill and seq.has_image:
                break
        self.running.extend(picked)
        return picked

    def _piece(self, seq: Sequence, cost: int, room: int) -> int:
        """Rows of `seq` to prefetch now when its `cost` rows exceed the `room` left in the step (0: do not
        split).  The last `chunk_tail` rows are kept for the final piece where possible.  A piece shorter
        than `chunked_prefill_tokens` is only cut when the step would otherwise be empty (the request has
        the whole budget to itself and still cannot finish)."""
        if self.chunk_min <= 0 or seq.has_image:
            return 0
        take = min(room, cost - self.chunk_tail)
        if take >= self.chunk_min:
            return take
        if room < self.max_num_batched_tokens:       # other requests share the step: wait for an emptier one
            return 0
        return take if take > 0 else min(room, cost - 1)

    # ------------------------------------------------------------------ decode
    def _schedule_decode(self) -> List[Sequence]:
        picked: List[Sequence] = []
        skipped: List[Sequence] = []
        while self.running and len(picked) < self.decode_cap:
            seq = self.running.popleft()
            if seq.hold:
                skipped.append(seq)
                continue
            while not self.block_manager.can_append(seq):
                if self.running:
                    self.preempt(self.running.pop())
                else:
                    self.preempt(seq)
                    break
            else:
                self.block_manager.may_append(seq)
                picked.append(seq)
        # keep arrival order: visited requests go back to the front
        visited = sorted(picked + skipped, key=lambda s: s.seq_id)
        self.running.extendleft(reversed(visited))
        return picked

    def schedule(self, prefer_decode: bool = False) -> Tuple[List[Sequence], bool]:
        """Pick the next batch.  Returns (sequences, is_prefill)."""
        # between two pieces of a split prompt the running requests get a decode step, so a long prompt
        # costs them one piece of latency per token instead of its whole prefill
        if self._piece_last and self.running and self.waiting and self.waiting[0].block_table:
            prefer_decode = True
        self._piece_last = False
        if prefer_decode and self.running:
            seqs = self._schedule_decode()
            if seqs:
                return seqs, False
        seqs = self._schedule_prefill()
        if seqs:
            self._piece_last = seqs[-1].prefill_end is not None
            return seqs, True
        seqs = self._schedule_decode()
        if not seqs and (self.waiting or self.running) and not any(s.hold for s in self.running):
            head = self.waiting[0] if self.waiting else self.running[0]
            raise RuntimeError(
                f"request {head.seq_id} needs {head.num_blocks} blocks but the pool has "
                f"{self.block_manager.num_blocks}; raise num_kvcache_blocks or shorten the request")
        return seqs, False

    def preempt(self, seq: Sequence) -> None:
        """Take a running request's blocks away; it is prefetched again later."""
        self.num_preemptions += 1
        seq.status = SequenceStatus.WAITING
        if self.on_release is not None:          # orders work in flight on the request's rows before the blocks go
            self.on_release(seq)
        self.block_manager.deallocate(seq)
        seq.reset_for_recompute()
        try:
            self.compress_queue.remove(seq)
        except ValueError:
            pass
        if self.waiting and self.waiting[0].block_table:
            # a split prompt whose first pieces are in the pool keeps the head of the queue: it owns all the
            # blocks it needs, so it always finishes, whereas a preempted request put in front of it could
            # wait forever for the blocks that it holds
            head = self.waiting.popleft()
            self.waiting.appendleft(seq)
            self.waiting.appendleft(head)
        else:
            self.waiting.appendleft(seq)

    def abort(self, seq: Sequence) -> bool:
        """Cancel a request wherever it is queued; its blocks return to the pool.  False if it had
        already finished."""
        if seq.is_finished:
            return False
        was_running = seq in self.running
        try:
            self.waiting.remove(seq)
        except ValueError:
            pass
        if was_running:
            self.finish(seq)
        else:
            seq.status = SequenceStatus.FINISHED
            if seq.block_table:                      # a split prompt whose first pieces are in the pool
                if self.on_release is not None:
                    self.on_release(seq)
                self.block_manager.deallocate(seq)
            try:
                self.compress_queue.remove(seq)
            except ValueError:
                pass
        return True

    def requeue_running(self) -> int:
        """Recovery after an aborted step: every running request gives its blocks back and is
        prefilled again from its tokens so far (arrival order kept).  Returns how many moved."""
        for seq in self.waiting:                 # split prompts whose first pieces are in the pool start over
            if seq.block_table:
                self.block_manager.unpublish_unwritten(seq, seq.num_computed_tokens)
                self.block_manager.deallocate(seq)
                seq.reset_for_recompute()
        moved = sorted(self.running, key=lambda s: s.seq_id, reverse=True)
        self.running.clear()
        for seq in moved:
            seq.hold = False
            # the failed step may have been this request's prefill or a compression of its rows: what its
            # own blocks hold is not to be trusted, so they leave the prefix cache before they are freed
            self.block_manager.unpublish_unwritten(seq, 0)
            self.preempt(seq)
        return len(moved)

    # ---------------------------------------------------------------- compress
    def enqueue_compress(self, seqs: List[Sequence]) -> None:
        for seq in seqs:
            if seq.compression_state is CompressionState.NONE and not seq.is_finished:
                seq.compression_state = CompressionState.PENDING
                self.compress_queue.append(seq)

    def schedule_compress(self, limit: Optional[int] = None) -> List[Sequence]:
        cap = self.compress_cap if limit is None else min(limit, self.compress_cap)
        picked: List[Sequence] = []
        while self.compress_queue and len(picked) < cap:
            seq = self.compress_queue.popleft()
            if seq.is_finished or seq.compression_state is not CompressionState.PENDING:
                continue
            picked.append(seq)
        return picked

    def lazy_compress_due(self) -> bool:
        return self.block_manager.occupancy > self.lazy_threshold

    def lazy_candidates(self) -> List[Sequence]:
        """Uncompressed running requests, largest KV first."""
        cands = [s for s in self.running
                 if s.compression_state is CompressionState.NONE and not s.is_finished]
        cands.sort(key=lambda s: -s.kv_cache_len)
        return cands

    # ------------------------------------------------------------- postprocess
    def postprocess(self, seqs: List[Sequence], token_ids: List[int]) -> List[Sequence]:
        """Append sampled tokens; retire finished requests.  Returns the finished ones."""
        done: List[Sequence] = []
        for seq, token_id in zip(seqs, token_ids):
            if seq.prefill_end is not None:          # a piece of a split prompt: nothing was sampled for it
                seq.num_computed_tokens, seq.prefill_end = seq.prefill_end, None
                continue
            seq.num_computed_tokens = 0
            seq.append_token(int(token_id))
            hit_eos = (not seq.ignore_eos) and token_id == self.eos
            if hit_eos or seq.num_completion_tokens >= seq.max_tokens:
                self.finish(seq)
                done.append(seq)
        return done

    def finish(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.FINISHED
        if self.on_release is not None:
            self.on_release(seq)
        self.block_manager.deallocate(seq)
        try:
            self.running.remove(seq)
        except ValueError:
            pass
        try:
            self.compress_queue.remove(seq)
        except ValueError:
            pass


# the reference exposes a second class for multimodal requests
class LlavaScheduler(Scheduler):
    def __init__(self, config: Config):
        super().__init__(config)
