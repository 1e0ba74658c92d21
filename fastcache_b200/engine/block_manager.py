"""Accounting for the paged KV pool.

Parity: nanovllm/engine/block_manager.py:9-169 — free list, used set,
reference counts, chained content hashes for prefix caching, append rules
keyed on the *stored* KV length so compressed requests grow correctly, and
`free_blocks_after_compression` / `free_specific_blocks` (:134-169).

This build adds pool-occupancy queries (the lazy policy triggers on them) and
`check_invariants`, a host-side ownership audit used by the tests in place of
a device memory checker.
"""
from __future__ import annotations

import hashlib
import struct
from collections import deque
from typing import Deque, Dict, Iterable, List, Optional, Set

from .sequence import Sequence


class Block:
    __slots__ = ("block_id", "ref_count", "hash", "token_ids")

    def __init__(self, block_id: int):
        self.block_id = block_id
        self.ref_count = 0
        self.hash = -1
        self.token_ids: List[int] = []

    def update(self, h: int, token_ids: List[int]) -> None:
        self.hash = h
        self.token_ids = token_ids

    def reset(self) -> None:
        self.ref_count = 1
        self.hash = -1
        self.token_ids = []


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int, prefix_caching: bool = True):
        if num_blocks <= 0:
            raise ValueError("the KV pool needs at least one block")
        self.block_size = block_size
        self.prefix_caching = prefix_caching
        self.blocks: List[Block] = [Block(i) for i in range(num_blocks)]
        self.hash_to_block_id: Dict[int, int] = {}
        self.free_block_ids: Deque[int] = deque(range(num_blocks))
        self.used_block_ids: Set[int] = set()

    # ------------------------------------------------------------------ hashing
    @staticmethod
    def compute_hash(token_ids: List[int], prefix: int = -1) -> int:
        """64-bit chained content hash of one full block."""
        h = hashlib.blake2b(digest_size=8)
        if prefix != -1:
            h.update(struct.pack("<q", prefix))
        h.update(struct.pack(f"<{len(token_ids)}i", *token_ids))
        return int.from_bytes(h.digest(), "little", signed=True)

    # --------------------------------------------------------------- occupancy
    @property
    def num_blocks(self) -> int:
        return len(self.blocks)

    @property
    def num_free_blocks(self) -> int:
        return len(self.free_block_ids)

    @property
    def occupancy(self) -> float:
        return 1.0 - len(self.free_block_ids) / len(self.blocks)

    # ------------------------------------------------------------- block moves
    def _allocate_block(self, block_id: int) -> Block:
        block = self.blocks[block_id]
        if block.ref_count != 0:
            raise RuntimeError(f"block {block_id} handed out twice")
        block.reset()
        self.free_block_ids.remove(block_id)
        self.used_block_ids.add(block_id)
        return block

    def _pop_free(self) -> Block:
        block_id = self.free_block_ids.popleft()
        block = self.blocks[block_id]
        if block.ref_count != 0:
            raise RuntimeError(f"block {block_id} on the free list with references")
        if block.hash != -1 and self.hash_to_block_id.get(block.hash) == block_id:
            del self.hash_to_block_id[block.hash]
        block.reset()
        self.used_block_ids.add(block_id)
        return block

    def _deallocate_block(self, block_id: int) -> None:
        block = self.blocks[block_id]
        if block.ref_count != 0:
            raise RuntimeError(f"block {block_id} freed while referenced")
        self.used_block_ids.discard(block_id)
        self.free_block_ids.append(block_id)

    def _release(self, block_id: int) -> None:
        block = self.blocks[block_id]
        block.ref_count -= 1
        if block.ref_count == 0:
            self._deallocate_block(block_id)

    # -------------------------------------------------------------- allocation
    def can_allocate(self, seq: Sequence) -> bool:
        return len(self.free_block_ids) >= seq.num_blocks

    def allocate(self, seq: Sequence) -> None:
        """Give `seq` blocks for its whole prompt, reusing cached prefix blocks.

        Prefix reuse is limited to text-only requests: the rows of an image
        request depend on pixels that the token ids do not identify.
        """
        if seq.block_table:
            raise RuntimeError("sequence already holds blocks")
        use_cache = self.prefix_caching and not seq.has_image
        h = -1
        cache_miss = not use_cache
        for i in range(seq.num_blocks):
            token_ids = seq.block(i) if use_cache else []
            full = len(token_ids) == self.block_size
            h = self.compute_hash(token_ids, h) if (use_cache and full) else -1
            block_id = self.hash_to_block_id.get(h, -1) if h != -1 else -1
            if block_id == -1 or self.blocks[block_id].token_ids != token_ids:
                cache_miss = True
            if cache_miss:
                block = self._pop_free()
            else:
                seq.num_cached_tokens += self.block_size
                if block_id in self.used_block_ids:
                    block = self.blocks[block_id]
                    block.ref_count += 1
                else:
                    block = self._allocate_block(block_id)
            if h != -1:
                block.update(h, token_ids)
                self.hash_to_block_id[h] = block.block_id
            seq.block_table.append(block.block_id)
        # never report the whole prompt as cached: the last token must run
        if seq.num_cached_tokens >= seq.num_prompt_tokens:
            seq.num_cached_tokens -= self.block_size

    def deallocate(self, seq: Sequence) -> None:
        for block_id in reversed(seq.block_table):
            self._release(block_id)
        seq.num_cached_tokens = 0
        seq.block_table.clear()

    # ------------------------------------------------------------------- decode
    def can_append(self, seq: Sequence) -> bool:
        """A decode step needs a fresh block when the new row opens one."""
        needs_new = (seq.kv_cache_len % self.block_size == 1) or self.block_size == 1
        return len(self.free_block_ids) >= int(needs_new)

    def blocks_short_for(self, seq: Sequence, extra_rows: int) -> int:
        """Blocks still missing from the table of `seq` if it is to hold `extra_rows` rows beyond the one its next
        decode step writes (several decode steps launched back to back)."""
        need = -(-(seq.kv_cache_len + extra_rows) // self.block_size)
        return max(0, need - len(seq.block_table))

    def reserve_rows(self, seq: Sequence, extra_rows: int) -> None:
        """Grow the block table for `extra_rows` more rows (the caller has checked that the pool has the blocks)."""
        for _ in range(self.blocks_short_for(seq, extra_rows)):
            seq.block_table.append(self._pop_free().block_id)

    def may_append(self, seq: Sequence) -> None:
        """Grow the block table for the row that this decode step writes.

        `seq.kv_cache_len` already counts that row (the token was appended in
        postprocess), so a remainder of 1 means "first row of a new block".
        """
        table = seq.block_table
        need = seq.kv_num_blocks
        while len(table) < need:
            table.append(self._pop_free().block_id)
        if seq.is_compressed or seq.has_image or not self.prefix_caching:
            return
        if seq.kv_cache_len % self.block_size == 0:
            # a block just filled with real token ids: publish it for prefix reuse
            last = self.blocks[table[-1]]
            if last.hash == -1:
                token_ids = seq.block(seq.num_blocks - 1)
                prefix = self.blocks[table[-2]].hash if len(table) > 1 else -1
                if len(table) > 1 and prefix == -1:
                    return
                h = self.compute_hash(token_ids, prefix)
                last.update(h, token_ids)
                self.hash_to_block_id[h] = last.block_id

    # -------------------------------------------------------------- compression
    def _unpublish(self, block_id: int) -> None:
        block = self.blocks[block_id]
        if block.hash != -1 and self.hash_to_block_id.get(block.hash) == block_id:
            del self.hash_to_block_id[block.hash]
        block.hash = -1
        block.token_ids = []

    def unpublish_unwritten(self, seq: Sequence, rows_written: int) -> int:
        """Take the blocks of `seq` that are not completely written yet (block index >= rows_written //
        block_size) out of the prefix cache, unless another request shares them (then their first owner
        wrote them).  Used for prompts that are prefetched in pieces: a block must not be found by its
        content hash before its rows exist.  Returns how many blocks were unpublished."""
        n = 0
        for block_id in seq.block_table[rows_written // self.block_size:]:
            block = self.blocks[block_id]
            if block.ref_count == 1 and block.hash != -1:
                self._unpublish(block_id)
                n += 1
        return n

    def private_copy_needed(self, seq: Sequence) -> List[int]:
        """Indices into the block table whose block is shared with another request.

        Compression rewrites the leading blocks in place, which must not be
        visible to a request that shares them through the prefix cache.
        """
        return [i for i, b in enumerate(seq.block_table) if self.blocks[b].ref_count > 1]

    def make_private(self, seq: Sequence, index: int) -> tuple:
        """Swap a shared block for a fresh one; returns (old_id, new_id) so the
        runner can copy the rows."""
        old = seq.block_table[index]
        new = self._pop_free().block_id
        self.blocks[old].ref_count -= 1
        seq.block_table[index] = new
        return old, new

    def free_blocks_after_compression(self, seq: Sequence, blocks_to_keep: int) -> int:
        """Return the tail of `seq`'s block table to the pool.

        The kept blocks now hold rewritten rows, so they leave the prefix
        cache.  Returns the number of blocks released.
        """
        blocks_to_keep = max(0, min(blocks_to_keep, len(seq.block_table)))
        tail = seq.block_table[blocks_to_keep:]
        for block_id in reversed(tail):
            self._release(block_id)
        del seq.block_table[blocks_to_keep:]
        for block_id in seq.block_table:
            if self.blocks[block_id].ref_count == 1:
                self._unpublish(block_id)
        seq.num_cached_tokens = 0
        return len(tail)

    # ------------------------------------------------- blocks outside a block table
    def take_blocks(self, n: int) -> List[int]:
        """`n` fresh private blocks that belong to no block table yet (the destination of an out-of-place
        compression; the caller keeps them in `Sequence.shadow_table`).  Raises if the pool cannot give them."""
        if n > len(self.free_block_ids):
            raise RuntimeError(f"asked for {n} blocks, {len(self.free_block_ids)} are free")
        return [self._pop_free().block_id for _ in range(n)]

    def release_blocks(self, block_ids: Iterable[int]) -> int:
        """Give back blocks obtained with `take_blocks` or a block table that a request no longer uses."""
        n = 0
        for block_id in reversed(list(block_ids)):
            self._release(block_id)
            n += 1
        return n

    def free_specific_blocks(self, block_ids: Iterable[int]) -> int:
        n = 0
        for block_id in block_ids:
            if block_id in self.used_block_ids:
                self._release(block_id)
                n += 1
        return n

    # --------------------------------------------------------------------- audit
    def check_invariants(self, live: Optional[Iterable[Sequence]] = None) -> None:
        """Raise if the ownership bookkeeping is inconsistent."""
        free = list(self.free_block_ids)
        if len(set(free)) != len(free):
            raise AssertionError("duplicate id on the free list")
        if set(free) & self.used_block_ids:
            raise AssertionError("block both free and used")
        if len(free) + len(self.used_block_ids) != len(self.blocks):
            raise AssertionError("blocks leaked")
        for b in self.blocks:
            if b.ref_count < 0:
                raise AssertionError("negative reference count")
            if (b.ref_count > 0) != (b.block_id in self.used_block_ids):
                raise AssertionError(f"block {b.block_id}: refs and used set disagree")
        if live is not None:
            refs: Dict[int, int] = {}
            for s in live:
                for b in list(s.block_table) + list(getattr(s, "shadow_table", ())):
                    refs[b] = refs.get(b, 0) + 1
            for b, n in refs.items():
                if self.blocks[b].ref_count != n:
                    raise AssertionError(f"block {b}: {n} holders, ref_count {self.blocks[b].ref_count}")
            if set(refs) != self.used_block_ids:
                raise AssertionError("used set differs from the union of live block tables")


# module-level name used by the reference (nanovllm/engine/block_manager.py:9-14)
compute_hash = BlockManager.compute_hash
