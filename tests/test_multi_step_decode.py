"""Several decode steps per engine step (`decode_steps_per_call`): the same tokens as one step at a time."""
import pytest
import torch

from fastcache_b200 import LLM, SamplingParams
from helpers import tiny_llama_config


def _prompts(n=5, seed=3, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, vocab, (int(torch.randint(20, 90, (1,), generator=g)),), generator=g).tolist()
            for _ in range(n)]


def _engine(k, **kw):
    kw.setdefault("prefix_caching", False)
    return LLM(tiny_llama_config(num_hidden_layers=2), kvcache_block_size=16, num_kvcache_blocks=96, max_model_len=256,
               device="cpu", enforce_eager=False, seed=7, decode_steps_per_call=k, **kw)


@pytest.mark.parametrize("temperature", [0.0, 0.8])
@pytest.mark.parametrize("k", [2, 4, 7])
def test_same_tokens_as_single_steps(k, temperature):
    sps = [SamplingParams(temperature=temperature, max_tokens=m, ignore_eos=True) for m in (23, 5, 16, 1, 30)]
    want = _engine(1).generate(_prompts(), sps)
    llm = _engine(k)
    got = llm.generate(_prompts(), sps)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]
    assert llm.stats.decode_steps > 0 and llm.stats.steps < _steps_of(want, 5)      # fewer engine steps
    bm = llm.scheduler.block_manager
    bm.check_invariants([])
    assert bm.num_free_blocks == bm.num_blocks


def _steps_of(outs, n_prefill_steps):
    return n_prefill_steps + max(len(o["token_ids"]) for o in outs)


def test_end_of_sequence_token_inside_a_launch_discards_the_rest():
    """A request that samples its end token in the middle of a multi-step launch keeps nothing after it."""
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    base = _engine(1).generate(_prompts(3), sp)
    eos = base[1]["token_ids"][9]                       # the tenth token of request 1 becomes the end token
    sp2 = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=False)
    want = _engine(1, eos=eos).generate(_prompts(3), sp2)
    got = _engine(4, eos=eos).generate(_prompts(3), sp2)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]
    assert len(want[1]["token_ids"]) <= 10


def test_with_compression_and_with_requests_still_waiting():
    """Compression right after prefill, more requests than one prefill step takes: multi-step launches only start
    once nothing is waiting, and give the same tokens."""
    kw = dict(enable_compression=True, compression_backend="kvpress", kvpress_method="knorm", compression_factor=2,
              compression_pipeline="prefill", max_num_batched_tokens=128, max_num_seqs=8)
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = _engine(1, **kw).generate(_prompts(6), sp)
    llm = _engine(3, **kw)
    got = llm.generate(_prompts(6), sp)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]
    assert llm.stats.compressions == 6


def test_not_enough_blocks_falls_back_to_single_steps():
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    prompts = _prompts(4)
    want = _engine(1).generate(prompts, sp)
    # a pool that holds the prompts and little more: reservations fail, requests are preempted as usual
    tight = LLM(tiny_llama_config(num_hidden_layers=2), kvcache_block_size=16, num_kvcache_blocks=22, max_model_len=256,
                device="cpu", enforce_eager=False, seed=7, decode_steps_per_call=8, prefix_caching=False)
    got = tight.generate(prompts, sp)
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]
