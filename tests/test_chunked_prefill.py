"""Chunked prefill: prompts split over several prefill steps give the tokens of unsplit prefill."""
import pytest
import torch

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
from helpers import random_compressor, tiny_llama_config


def _prompts(lengths, seed=4):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, 1000, (n,), generator=g).tolist() for n in lengths]


def _engine(budget, chunk, **kw):
    return LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=256, max_model_len=1024, device="cpu",
               enforce_eager=True, max_num_batched_tokens=budget, chunked_prefill_tokens=chunk, prefix_caching=False,
               **kw)


@pytest.mark.parametrize("kind", ["none", "ccm", "snapkv"])
def test_split_prompts_generate_the_same_tokens(kind):
    kw = {}
    if kind == "ccm":
        kw = dict(enable_compression=True, compression_backend="mlp", compression_pipeline="prefill",
                  compressor=random_compressor(KVCacheLinearDecoupleCompressor, 2, 64, 4))
    elif kind == "snapkv":
        kw = dict(enable_compression=True, compression_backend="kvpress", kvpress_method="snapkv",
                  compression_factor=2, compression_pipeline="prefill",
                  kvpress_params={"window": 16, "kernel_size": 5})
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = _prompts([300, 40, 150, 90, 260])
    whole = _engine(4096, 0, **kw)
    ref = [o["token_ids"] for o in whole.generate(prompts, sp)]
    assert whole.stats.prefill_steps == 1

    llm = _engine(128, 32, **kw)
    seqs = [llm.add_request(p, sp) for p in prompts]
    pieces = 0
    while not llm.is_finished():
        head = llm.scheduler.waiting[0] if llm.scheduler.waiting else None
        llm.step()
        if head is not None and head.num_computed_tokens > 0 and head.status.name == "WAITING":
            pieces += 1
            assert head.block_table and head.num_completion_tokens == 0      # keeps its blocks, sampled nothing
        llm.scheduler.block_manager.check_invariants(list(llm.scheduler.running) +
                                                     [s for s in llm.scheduler.waiting if s.block_table])
    assert pieces >= 4 and llm.stats.prefill_steps > 5
    assert [s.completion_token_ids for s in seqs] == ref
    assert llm.stats.prefill_tokens == sum(len(p) for p in prompts)
    if kind != "none":
        assert llm.stats.compressions == len(prompts)
    bm = llm.scheduler.block_manager
    assert bm.num_free_blocks == bm.num_blocks


def test_unsplittable_cases_and_abort():
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)
    # splitting off: a prompt over the step budget is refused, as before
    llm = _engine(64, 0)
    llm.add_request(_prompts([100])[0], sp)
    with pytest.raises(RuntimeError):
        llm.step()
    # a request cancelled between its pieces returns its blocks
    llm = _engine(64, 16)
    seq = llm.add_request(_prompts([200])[0], sp)
    llm.step()
    assert seq.num_computed_tokens == 64 and seq.block_table
    bm = llm.scheduler.block_manager
    assert bm.num_free_blocks < bm.num_blocks
    assert llm.abort_request(seq.seq_id) and bm.num_free_blocks == bm.num_blocks
    assert llm.is_finished()
    # recovery restarts a half-prefetched request from its first row
    seq = llm.add_request(_prompts([200])[0], sp)
    llm.step()
    llm.recover()
    assert seq.num_computed_tokens == 0 and not seq.block_table and bm.num_free_blocks == bm.num_blocks
    out = []
    while not llm.is_finished():
        out += llm.step()[0]
    assert len(out[0][1]) == 2


def test_unwritten_blocks_of_a_split_prompt_are_not_in_the_prefix_cache():
    """With prefix caching on, a second request with the same prompt must not hit blocks of a request that is
    still between its pieces; after the first has finished, the written blocks (up to the first piece's end)
    may be shared, and both requests generate the same tokens as an engine without prefix caching."""
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    prompt = _prompts([200])[0]
    plain = LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=256, max_model_len=1024, device="cpu",
                enforce_eager=True, max_num_batched_tokens=4096, prefix_caching=False)
    want = plain.generate([prompt], sp)[0]["token_ids"]
    llm = LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=256, max_model_len=1024, device="cpu",
              enforce_eager=True, max_num_batched_tokens=64, chunked_prefill_tokens=16, prefix_caching=True)
    a = llm.add_request(prompt, sp)
    llm.step()                                           # first piece: rows [0, 64)
    bm = llm.scheduler.block_manager
    published = [i for i, b in enumerate(a.block_table) if bm.blocks[b].hash != -1]
    assert published == [0, 1, 2, 3]                     # only the four blocks the piece fills
    b = llm.add_request(prompt, sp)
    while not llm.is_finished():
        llm.step()
    assert a.completion_token_ids == want and b.completion_token_ids == want
    assert bm.num_free_blocks == bm.num_blocks


def test_decode_steps_run_between_the_pieces_of_a_long_prompt():
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    short, long_ = _prompts([20, 400], seed=9)
    want = [o["token_ids"] for o in _engine(4096, 0).generate([short, long_], sp)]
    llm = _engine(64, 16)
    a = llm.add_request(short, sp)
    llm.step()                                           # the short request is running before the long one arrives
    b = llm.add_request(long_, sp)
    kinds = []
    while not llm.is_finished():
        _, n = llm.step()
        kinds.append("P" if n > 0 else "D")
    trace = "".join(kinds)
    assert "PP" not in trace[: trace.rindex("P")]        # while the short request decodes, no two pieces in a row
    assert trace.count("P") >= 6
    assert [a.completion_token_ids, b.completion_token_ids] == want
