"""Property tests: random operation sequences never break the block manager's ownership bookkeeping,
and the scheduler serves every request under any pool size that can hold the largest one."""
import random

from hypothesis import HealthCheck, given, settings, strategies as st

from fastcache_b200.config import Config
from fastcache_b200.engine.block_manager import BlockManager
from fastcache_b200.engine.scheduler import Scheduler
from fastcache_b200.engine.sequence import CompressionState, Sequence
from fastcache_b200.sampling_params import SamplingParams

BS = 8


def _seq(tokens):
    Sequence.block_size = BS
    return Sequence(list(tokens), SamplingParams(max_tokens=64))


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.data())
def test_random_allocate_append_compress_free_keeps_invariants(data):
    rng = random.Random(data.draw(st.integers(0, 10 ** 6)))
    prefix_caching = data.draw(st.booleans())
    bm = BlockManager(num_blocks=48, block_size=BS, prefix_caching=prefix_caching)
    live = []
    shared_prefix = [rng.randrange(3, 50) for _ in range(3 * BS)]
    for _ in range(data.draw(st.integers(5, 60))):
        op = rng.choice(["alloc", "alloc_shared", "append", "compress", "free", "private"])
        if op in ("alloc", "alloc_shared"):
            n = rng.randrange(1, 5 * BS)
            toks = (shared_prefix + [rng.randrange(3, 50) for _ in range(n)]) if op == "alloc_shared" else \
                [rng.randrange(3, 50) for _ in range(n)]
            s = _seq(toks)
            if bm.can_allocate(s):
                bm.allocate(s)
                assert len(s.block_table) == s.num_blocks
                assert s.num_cached_tokens < s.num_prompt_tokens
                live.append(s)
        elif op == "append" and live:
            s = rng.choice(live)
            s.append_token(rng.randrange(3, 50))
            if bm.can_append(s):
                bm.may_append(s)
                assert len(s.block_table) >= s.kv_num_blocks
            else:                                    # no room: the scheduler would preempt; undo here
                bm.deallocate(s)
                live.remove(s)
        elif op == "compress" and live:
            s = rng.choice(live)
            if s.compression_state is CompressionState.NONE and s.kv_cache_len >= 8:
                for i in bm.private_copy_needed(s):
                    if i < s.kv_num_blocks and bm.num_free_blocks > 0:
                        bm.make_private(s, i)
                if not bm.private_copy_needed(s):
                    s.kv_cache_len = max(1, s.kv_cache_len // 4)
                    s.compression_state = CompressionState.COMPLETED
                    freed = bm.free_blocks_after_compression(s, s.kv_num_blocks)
                    assert freed >= 0 and len(s.block_table) == s.kv_num_blocks
        elif op == "private" and live:
            s = rng.choice(live)
            need = bm.private_copy_needed(s)
            if need and bm.num_free_blocks > 0:
                old, new = bm.make_private(s, need[0])
                assert old != new and s.block_table[need[0]] == new
        elif op == "free" and live:
            s = live.pop(rng.randrange(len(live)))
            bm.deallocate(s)
            assert not s.block_table
        bm.check_invariants(live)
        assert 0.0 <= bm.occupancy <= 1.0
    for s in live:
        bm.deallocate(s)
    bm.check_invariants([])
    assert bm.num_free_blocks == bm.num_blocks


@settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(0, 10 ** 6), st.integers(12, 40), st.integers(1, 6))
def test_scheduler_serves_every_request_under_pressure(seed, num_blocks, max_seqs):
    """A trace of schedule / postprocess steps with random prompt lengths and output lengths: every request
    finishes, nothing is scheduled twice in one step, preempted requests come back, no block leaks."""
    rng = random.Random(seed)
    Sequence.block_size = BS
    cfg = Config.from_kwargs("", kvcache_block_size=BS, num_kvcache_blocks=num_blocks, max_num_seqs=max_seqs,
                             max_num_batched_tokens=64, max_model_len=96, eos=-1)
    sch = Scheduler(cfg)
    seqs = []
    for _ in range(rng.randrange(3, 12)):
        n = rng.randrange(1, 40)
        s = Sequence([rng.randrange(3, 50) for _ in range(n)],
                     SamplingParams(max_tokens=rng.randrange(1, 20), ignore_eos=True))
        sch.add(s)
        seqs.append(s)
    steps = 0
    while not sch.is_finished():
        batch, is_prefill = sch.schedule()
        assert batch and len({s.seq_id for s in batch}) == len(batch)
        assert len(batch) <= max_seqs
        if is_prefill:
            assert sum(s.logical_len - s.num_cached_tokens for s in batch) <= 64
        for s in batch:
            assert len(s.block_table) >= s.kv_num_blocks
        sch.postprocess(batch, [rng.randrange(3, 50) for _ in batch])
        sch.block_manager.check_invariants(list(sch.running))
        steps += 1
        assert steps < 5000
    assert all(s.is_finished and s.num_completion_tokens == s.max_tokens for s in seqs)
    bm = sch.block_manager
    assert bm.num_free_blocks == bm.num_blocks


@settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(0, 10 ** 6), st.integers(24, 60), st.integers(1, 6), st.integers(4, 24))
def test_scheduler_with_split_prompts_serves_every_request(seed, num_blocks, max_seqs, chunk):
    """The same trace with chunked prefill and prompts longer than a step's budget: a step never exceeds the
    budget, every piece starts where the last one ended, every request finishes, no block leaks."""
    rng = random.Random(seed)
    Sequence.block_size = BS
    budget = 48
    cfg = Config.from_kwargs("", kvcache_block_size=BS, num_kvcache_blocks=num_blocks, max_num_seqs=max_seqs,
                             max_num_batched_tokens=budget, max_model_len=200, eos=-1, chunked_prefill_tokens=chunk)
    sch = Scheduler(cfg)
    sch.chunk_tail = 8
    seqs = []
    for _ in range(rng.randrange(3, 10)):
        n = rng.randrange(1, min(150, (num_blocks - 4) * BS))
        s = Sequence([rng.randrange(3, 50) for _ in range(n)],
                     SamplingParams(max_tokens=rng.randrange(1, 12), ignore_eos=True))
        sch.add(s)
        seqs.append(s)
    computed = {s.seq_id: 0 for s in seqs}
    steps = 0
    while not sch.is_finished():
        batch, is_prefill = sch.schedule()
        assert batch and len({s.seq_id for s in batch}) == len(batch)
        if is_prefill:
            rows = 0
            for s in batch:
                end = s.logical_len if s.prefill_end is None else s.prefill_end
                # a request that comes back after preemption may find its first blocks in the prefix cache
                assert s.prefill_start == max(computed[s.seq_id], s.num_cached_tokens) and end > s.prefill_start
                assert len(s.block_table) * BS >= end
                rows += end - s.prefill_start
                computed[s.seq_id] = end if s.prefill_end is not None else 0
            assert rows <= budget
            assert sum(s.prefill_end is not None for s in batch) <= 1
        before = {s.seq_id: s.num_completion_tokens for s in batch}
        partial = {s.seq_id for s in batch if s.prefill_end is not None}
        sch.postprocess(batch, [rng.randrange(3, 50) for _ in batch])
        for s in batch:
            grew = s.num_completion_tokens - before[s.seq_id]
            assert grew == (0 if s.seq_id in partial else 1)
        for s in seqs:                               # a preempted request starts over
            if not s.block_table and not s.is_finished:
                computed[s.seq_id] = 0
        sch.block_manager.check_invariants(list(sch.running) + [s for s in sch.waiting if s.block_table])
        steps += 1
        assert steps < 8000
    assert all(s.is_finished and s.num_completion_tokens == s.max_tokens for s in seqs)
    bm = sch.block_manager
    assert bm.num_free_blocks == bm.num_blocks
