"""Per-request state.

Parity: nanovllm/engine/sequence.py:8-98 (token list, prompt length, prefix
cache hit count, block table, compression state) and the multimodal subclass
in "kv-cache pipeline"/nanovllm/engine/llava_engine.py:28-41.

Differences by design: the KV length of a request is tracked explicitly
(`kv_len`) from the start instead of being derived from the number of text
tokens, so an image placeholder that expands to hundreds of KV rows is
accounted for in block allocation (the reference sizes blocks by text tokens
only and pads block tables with indices it never allocated).
"""
from __future__ import annotations

import itertools
import time
from copy import copy
from enum import Enum, auto
from typing import Any, List, Optional

from ..sampling_params import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class CompressionState(Enum):
    NONE = auto()         # never compressed
    PENDING = auto()      # chosen for compression, not launched
    IN_PROGRESS = auto()  # launched on a side stream, event outstanding
    COMPLETED = auto()
    FAILED = auto()       # the compressor raised; the request keeps its full KV and is not retried


class Sequence:
    block_size = 256
    _ids = itertools.count()

    def __init__(self, token_ids: List[int], sampling_params: Optional[SamplingParams] = None,
                 num_image_tokens: int = 0, image_token_pos: int = -1):
        sp = sampling_params or SamplingParams()
        self.seq_id = next(Sequence._ids)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.last_token = self.token_ids[-1]
        self.num_tokens = len(self.token_ids)
        self.num_prompt_tokens = self.num_tokens
        self.num_cached_tokens = 0
        # chunked prefill: rows already in the pool from earlier pieces, and where this step's piece ends
        # (None: at the end of the request)
        self.num_computed_tokens = 0
        self.prefill_end: Optional[int] = None
        self.block_table: List[int] = []
        self.temperature = sp.temperature
        self.max_tokens = sp.max_tokens
        self.ignore_eos = sp.ignore_eos
        # multimodal: one placeholder token expands to `num_image_tokens` rows
        self.num_image_tokens = int(num_image_tokens)
        self.image_token_pos = int(image_token_pos)
        self.pixel_values: Any = None
        self.image_meta: Any = None
        # compression
        self._kv_cache_len: Optional[int] = None     # None = tracks the logical length
        self.compression_state = CompressionState.NONE
        self.compression_event: Any = None
        self.hold = False             # kept out of decode batches (chunked compression running)
        # blocks that receive this request's compressed rows while it keeps decoding over the original ones
        self.shadow_table: List[int] = []
        self._pending_row = False     # the newest token's K/V row is not in the pool yet
        # timestamps (host seconds, monotonic) for TTFT / TPOT
        self.arrival_time = time.perf_counter()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None

    # ------------------------------------------------------------------ lengths
    def __len__(self) -> int:
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def extra_image_rows(self) -> int:
        """KV rows added by expanding the image placeholder (0 for text)."""
        return max(0, self.num_image_tokens - 1) if self.num_image_tokens > 0 else 0

    @property
    def logical_len(self) -> int:
        """Number of KV rows the request would occupy without compression."""
        return self.num_tokens + self.extra_image_rows

    @property
    def prefill_start(self) -> int:
        """First row the next prefill step has to compute (after prefix-cache hits and earlier pieces)."""
        return max(self.num_cached_tokens, self.num_computed_tokens)

    @property
    def prompt_rows(self) -> int:
        return self.num_prompt_tokens + self.extra_image_rows

    @property
    def kv_cache_len(self) -> int:
        return self.logical_len if self._kv_cache_len is None else self._kv_cache_len

    @kv_cache_len.setter
    def kv_cache_len(self, value: int) -> None:
        self._kv_cache_len = int(value)

    # short alias used throughout this package
    kv_len = kv_cache_len

    @property
    def is_compressed(self) -> bool:
        return self._kv_cache_len is not None

    @property
    def has_image(self) -> bool:
        return self.num_image_tokens > 0

    @property
    def image_token_len(self) -> int:
        return self.num_image_tokens

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return self.num_tokens - self.num_prompt_tokens

    @property
    def prompt_token_ids(self) -> List[int]:
        return self.token_ids[: self.num_prompt_tokens]

    @property
    def completion_token_ids(self) -> List[int]:
        return self.token_ids[self.num_prompt_tokens:]

    # ------------------------------------------------------------------- blocks
    @property
    def num_cached_blocks(self) -> int:
        return self.num_cached_tokens // self.block_size

    @property
    def num_blocks(self) -> int:
        """Blocks needed for the logical (uncompressed) length."""
        return -(-self.logical_len // self.block_size)

    @property
    def kv_num_blocks(self) -> int:
        """Blocks needed for the rows really held in the pool."""
        return -(-self.kv_cache_len // self.block_size)

    def last_block(self) -> List[int]:
        """Token ids of the last (possibly partial) block, counted over the token ids like `block(i)`."""
        n = -(-len(self.token_ids) // self.block_size)
        return self.token_ids[max(0, n - 1) * self.block_size:]

    @property
    def last_block_num_tokens(self) -> int:
        return self.kv_cache_len - (self.kv_num_blocks - 1) * self.block_size

    def block(self, i: int) -> List[int]:
        """Token ids of logical block `i` (text-only requests; used for prefix hashing)."""
        return self.token_ids[i * self.block_size:(i + 1) * self.block_size]

    # ------------------------------------------------------------------ mutation
    def append_token(self, token_id: int) -> None:
        self.token_ids.append(token_id)
        self.last_token = token_id
        self.num_tokens += 1
        if self._kv_cache_len is not None:
            self._kv_cache_len += 1
        self._pending_row = True

    @property
    def rows_in_pool(self) -> int:
        """Rows whose K/V are really stored (a sampled token is stored by the next decode step)."""
        return self.kv_cache_len - int(self._pending_row)

    def next_position(self, mode: str = "compressed") -> int:
        """Position id of the token that the next decode step feeds.

        The reference engine uses the (possibly compressed) KV length for both
        the context length and the rotary position
        ("kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:731-745).
        """
        if mode == "compressed":
            return self.kv_cache_len - 1
        return self.logical_len - 1

    def reset_for_recompute(self) -> None:
        """Drop pool state after preemption; the request is prefetched again."""
        self._kv_cache_len = None
        self.compression_state = CompressionState.NONE
        self.compression_event = None
        self.hold = False
        self._pending_row = False
        self.num_cached_tokens = 0
        self.num_computed_tokens = 0
        self.prefill_end = None
        self.block_table = []
        self.shadow_table = []

    # pickling for the optional driver->worker plan broadcast keeps messages small
    def __getstate__(self):
        state = copy(self.__dict__)
        state["pixel_values"] = None
        state["compression_event"] = None
        return state


# name used by the reference's multimodal engine
LlavaSequence = Sequence
