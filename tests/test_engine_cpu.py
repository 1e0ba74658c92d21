"""CPU plumbing: tiny Llama, 4 x 128-token prompts, CCM ratio 4, block 16, greedy 32."""
import torch

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
from helpers import random_compressor, tiny_llama_config


def _prompts(n=4, length=128, vocab=1024, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _engine(enforce_eager, compress, **kw):
    cfg = tiny_llama_config()
    comp = random_compressor(KVCacheLinearDecoupleCompressor, 2, 64, 4) if compress else None
    return LLM(cfg, kvcache_block_size=16, num_kvcache_blocks=256, max_model_len=512, device="cpu",
               enforce_eager=enforce_eager, enable_compression=compress, compressor=comp,
               compression_backend="mlp", compression_pipeline="prefill", **kw)


def test_graph_path_matches_eager_with_ccm():
    sp = SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True)
    a = _engine(True, True).generate(_prompts(), sp)
    b = _engine(False, True).generate(_prompts(), sp)
    assert [x["token_ids"] for x in a] == [x["token_ids"] for x in b]
    assert all(len(x["token_ids"]) == 32 for x in a)


def test_compression_frees_blocks_and_changes_lengths():
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    llm = _engine(True, True)
    for p in _prompts():
        llm.add_request(p, sp)
    free0 = llm.scheduler.block_manager.num_free_blocks
    llm.step()                                        # prefill + eager compression
    bm = llm.scheduler.block_manager
    seqs = list(llm.scheduler.running)
    assert all(s.is_compressed for s in seqs)
    # 128 rows -> 32 rows = 2 blocks of 16; the sampled token's row opens a third at the next decode
    assert all(s.kv_cache_len == 33 and len(s.block_table) == 2 for s in seqs)
    assert free0 - bm.num_free_blocks == 4 * 2
    bm.check_invariants(seqs)
    assert llm.stats.blocks_freed == 4 * (8 - 2)
    llm.step()
    assert all(len(s.block_table) == 3 for s in seqs)
    while not llm.is_finished():
        llm.step()
    bm.check_invariants([])
    assert bm.num_free_blocks == bm.num_blocks


def test_uncompressed_matches_dense_forward():
    """Paged engine output == plain dense causal forward of the same weights."""
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    llm = _engine(True, False)
    prompts = _prompts(2, 40)
    out = llm.generate(prompts, sp)
    out2 = _engine(False, False).generate(prompts, sp)
    assert [x["token_ids"] for x in out] == [x["token_ids"] for x in out2]


def test_step_trace_records_every_step_and_exports_chrome_trace(tmp_path):
    import json
    from fastcache_b200.utils import tracing
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    llm = _engine(True, True)
    trace = llm.enable_trace(capacity=64)
    with tracing.nvtx_range("no-op without a GPU"):
        llm.generate(_prompts(), sp)
    kinds = [r.kind for r in trace.records]
    assert kinds[0] == "prefill" and kinds.count("decode") == 3 and len(kinds) == llm.stats.steps
    first = trace.records[0]
    assert first.num_seqs == 4 and first.tokens == 4 * 128 and first.total_blocks == 256
    assert trace.records[1].compressions == 4 and trace.records[1].free_blocks == 256 - 4 * 3
    s = trace.summary()
    assert s["prefill"]["tokens"] == 512 and s["decode"]["steps"] == 3 and s["decode"]["device_ms"] is None
    path = tmp_path / "trace.json"
    trace.dump(str(path))
    blob = json.loads(path.read_text())
    assert sum(e["ph"] == "X" for e in blob["traceEvents"]) == len(kinds)
    assert not tracing.nvtx_enabled() or torch.cuda.is_available()


def test_exit_releases_the_engine_and_a_second_one_runs():
    """`exit()` drops the interpreter-exit hook, the pool and the weights, so the engine object and its
    tensors can be collected; another engine built afterwards in the same process works."""
    import gc
    import weakref
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    llm = _engine(True, True)
    first = llm.generate(_prompts(2, 40), sp)
    pool, engine = weakref.ref(llm.model_runner.kv_cache), weakref.ref(llm)
    llm.exit()
    llm.exit()                                           # idempotent
    assert llm.model_runner.kv_cache is None and llm.model_runner.model is None
    del llm
    gc.collect()
    assert pool() is None and engine() is None
    again = _engine(True, True).generate(_prompts(2, 40), sp)
    assert [o["token_ids"] for o in again] == [o["token_ids"] for o in first]


def test_compress_queue_meters_compression_by_the_compress_cap():
    """The three-queue batching of the harness ([prefill, compress, decode] caps): requests that finished prefill
    wait in the scheduler's compress queue and at most `compress_batch_size` of them are compressed per engine
    step; the others decode uncompressed until their turn."""
    from fastcache_b200.engine.sequence import CompressionState
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm = _engine(True, True, compress_batch_size=1)
    seqs = [llm.add_request(p, sp) for p in _prompts(3)]
    llm.step()                                             # one prefill step for all three, one compression
    assert [s.is_compressed for s in seqs] == [True, False, False]
    assert list(llm.scheduler.compress_queue) == seqs[1:]
    assert all(s.compression_state is CompressionState.PENDING for s in seqs[1:])
    llm.step()                                             # a decode step for all three, the second compression
    assert [s.is_compressed for s in seqs] == [True, True, False]
    llm.step()
    assert all(s.is_compressed for s in seqs) and not llm.scheduler.compress_queue
    while not llm.is_finished():
        llm.step()
    assert llm.stats.compressions == 3
    llm.scheduler.block_manager.check_invariants([])
