"""Layer-chunked (decode pipeline) compression on the CPU: eviction and merge give the same tokens whether the
layers are compressed in one call or a few per engine step, and a request whose chunks are in flight can lose its
blocks safely."""
import pytest

import torch

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
from helpers import random_compressor, tiny_llama_config


def _prompts(n=3, length=96, vocab=1024, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _engine(pipeline, layers_per_step, backend="kvpress", method="knorm", **kw):
    cfg = tiny_llama_config(num_hidden_layers=4)
    comp = random_compressor(KVCacheLinearDecoupleCompressor, 4, 64, 2) if backend == "mlp" else None
    return LLM(cfg, kvcache_block_size=16, num_kvcache_blocks=kw.pop("blocks", 128), max_model_len=512, device="cpu",
               enforce_eager=True, enable_compression=True, compression_backend=backend, kvpress_method=method,
               compression_factor=2, compressor=comp, compression_pipeline=pipeline,
               decode_layers_per_step=layers_per_step, **kw)


@pytest.mark.parametrize("method", ["knorm", "snapkv", "streaming_llm"])
@pytest.mark.parametrize("layers_per_step", [1, 2, 4])
def test_eviction_in_layer_chunks_matches_one_call(method, layers_per_step):
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = _engine("prefill", 4, method=method).generate(_prompts(), sp)
    got = _engine("decode", layers_per_step, method=method).generate(_prompts(), sp)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]


@pytest.mark.parametrize("layers_per_step", [1, 3])
def test_merge_in_layer_chunks_matches_one_call(layers_per_step):
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = _engine("prefill", 4, backend="mlp").generate(_prompts(), sp)
    got = _engine("decode", layers_per_step, backend="mlp", decode_overlap="hold").generate(_prompts(), sp)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]


def test_shadow_compression_with_all_layers_in_one_chunk_matches_the_prefill_pipeline():
    """Out-of-place compression whose only chunk runs before the request's first decode step switches in with no
    rows decoded meanwhile: the same tokens as compressing right after prefill."""
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = _engine("prefill", 4, backend="mlp").generate(_prompts(), sp)
    llm = _engine("decode", 4, backend="mlp", decode_overlap="shadow")
    got = llm.generate(_prompts(), sp)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]
    bm = llm.scheduler.block_manager
    bm.check_invariants([])
    assert bm.num_free_blocks == bm.num_blocks and llm.stats.compressions == 3


def test_shadow_compression_keeps_the_request_decoding():
    """One layer per engine step: the request gets a token at every step while its layers are compressed into a
    second set of blocks, then continues over [compressed rows | rows decoded meanwhile]."""
    from fastcache_b200.compress.inpool import _rows, ccm_compress_reference
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    llm = _engine("decode", 1, backend="mlp", decode_overlap="shadow")
    r, bm = llm.model_runner, llm.scheduler.block_manager
    seq = llm.add_request(_prompts(1)[0], sp)
    llm.step()                                             # prefill: 96 rows in 6 blocks
    assert not seq.hold and len(seq.shadow_table) >= 4 and seq.seq_id in llm._pending
    pool0 = r.kv_cache.clone()
    old_table = list(seq.block_table)
    produced = []
    while seq.seq_id in llm._pending:
        before = seq.num_completion_tokens
        llm.step()
        produced.append(seq.num_completion_tokens - before)
        bm.check_invariants([seq])
    assert produced and all(n == 1 for n in produced)      # never held out of a decode batch
    assert len(produced) == 4                              # a chunk per step; the switch comes in the step of the last
    tail = len(produced) - 1                               # rows decoded over the full KV before the switch
    n_out = 96 // 2
    assert seq.is_compressed and seq.kv_cache_len == n_out + tail + 1 + 1 and not seq.shadow_table
    # the compressed rows are what compressing the prefill rows gives; the rows decoded meanwhile follow them
    want_pool = pool0.clone()
    ccm_compress_reference(want_pool, old_table, 96, 0, r.packed_compressor)
    new_blocks = torch.tensor(seq.block_table)
    for layer in range(4):
        for kv in (0, 1):
            got = _rows(r.kv_cache[layer, kv], new_blocks, n_out)
            want = _rows(want_pool[layer, kv], torch.tensor(old_table), n_out)
            torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    while not llm.is_finished():
        llm.step()
    bm.check_invariants([])
    assert bm.num_free_blocks == bm.num_blocks and seq.num_completion_tokens == 10


def test_shadow_falls_back_to_hold_without_free_blocks_and_survives_preemption():
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm = _engine("decode", 1, backend="mlp", decode_overlap="shadow", blocks=8)   # 96 rows = 6 of 8 blocks
    seq = llm.add_request(_prompts(1)[0], sp)
    llm.step()
    assert seq.hold and not seq.shadow_table               # no room for a second copy: in place
    while not llm.is_finished():
        llm.step()
    # a request that loses its blocks between chunks gives its shadow blocks back too
    llm2 = _engine("decode", 1, backend="mlp", decode_overlap="shadow")
    s2 = llm2.add_request(_prompts(1)[0], sp)
    llm2.step()
    llm2.step()
    assert s2.shadow_table
    llm2.scheduler.running.remove(s2)
    llm2.scheduler.preempt(s2)
    bm = llm2.scheduler.block_manager
    assert not s2.shadow_table and bm.num_free_blocks == bm.num_blocks
    bm.check_invariants([])
    while not llm2.is_finished():
        llm2.step()
    assert s2.num_completion_tokens == 6


def test_chunks_of_one_request_stay_on_one_stream_and_leave_an_event_each():
    """The engine pins every layer chunk of a request to the stream chosen when its compression started and
    records an event after each chunk (checked with stand-in streams: the CPU device has none)."""
    import fastcache_b200.engine.llm_engine as eng_mod

    class FakeStream:
        def __init__(self, name):
            self.name, self.waits = name, 0

        def wait_event(self, ev):
            self.waits += 1

    class FakeEvent:
        made = []

        def __init__(self, *a, **k):
            self.stream = None
            FakeEvent.made.append(self)

        def record(self, stream=None):
            self.stream = stream

    llm = _engine("decode", 1)
    r = llm.model_runner
    r.compress_streams = [FakeStream("a"), FakeStream("b")]
    r.main_stream = FakeStream("main")
    used = []
    real = r.compress_kv_cache_batch

    def spy(seqs, first=0, last=None, stream=None, dst_tables=None):
        used.append((tuple(s.seq_id for s in seqs), first, stream.name))
        return real(seqs, first, last, stream=None, dst_tables=dst_tables)

    r.compress_kv_cache_batch = spy
    orig_event = eng_mod.torch.cuda.Event
    eng_mod.torch.cuda.Event = FakeEvent
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
        seqs = [llm.add_request(p, sp) for p in _prompts(2)]
        llm.step()                                           # prefill of both, chunked compression starts
        streams = {sid: p.stream.name for sid, p in llm._pending.items()}
        assert sorted(streams.values()) == ["a", "b"]        # one request per stream
        for _ in range(4):
            llm.step()
        per_seq = {}
        for ids, first, name in used:
            for sid in ids:
                per_seq.setdefault(sid, []).append((first, name))
        for s in seqs:
            assert [f for f, _ in per_seq[s.seq_id]] == [0, 1, 2, 3]
            assert {n for _, n in per_seq[s.seq_id]} == {streams[s.seq_id]}
        chunk_events = [e for e in FakeEvent.made if e.stream is not None and e.stream.name in ("a", "b")]
        assert len(chunk_events) == 8                        # 2 requests x 4 chunks
    finally:
        eng_mod.torch.cuda.Event = orig_event
        r.main_stream = None
        r.compress_streams = []


def test_preempting_a_request_between_chunks_orders_the_main_stream_first():
    import fastcache_b200.engine.llm_engine as eng_mod
    waited = []

    class FakeStream:
        def wait_event(self, ev):
            waited.append(ev)

    class FakeEvent:
        def __init__(self, *a, **k):
            pass

        def record(self, stream=None):
            self.stream = stream

    llm = _engine("decode", 1)
    r = llm.model_runner
    side = FakeStream()
    r.compress_streams = [side]
    r.main_stream = FakeStream()
    real = r.compress_kv_cache_batch
    r.compress_kv_cache_batch = lambda seqs, first=0, last=None, stream=None, dst_tables=None: \
        real(seqs, first, last, stream=None, dst_tables=dst_tables)
    orig_event = eng_mod.torch.cuda.Event
    eng_mod.torch.cuda.Event = FakeEvent
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
        seq = llm.add_request(_prompts(1)[0], sp)
        llm.step()
        llm._advance_chunked()                               # first chunk launched, three to go
        p = llm._pending[seq.seq_id]
        assert seq.hold and p.event is not None and p.next_layer == 1
        waited.clear()
        llm.scheduler.running.remove(seq)
        llm.scheduler.preempt(seq)
        assert waited == [p.event]                           # the main stream waits for the newest chunk
        assert seq.seq_id not in llm._pending and not seq.hold and not seq.block_table
        llm.scheduler.block_manager.check_invariants([])
    finally:
        eng_mod.torch.cuda.Event = orig_event
        r.main_stream = None
        r.compress_streams = []
