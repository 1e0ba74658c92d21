"""Rotary position of the tokens decoded after compression: `position_mode` "compressed" (the KV length, as the
reference engine does it: "kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:731-745) or "original" (the
true index of the token)."""
import pytest
import torch

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.config import Config
from helpers import tiny_llama_config


def _engine(mode, **kw):
    return LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=128, max_model_len=512, device="cpu",
               enforce_eager=True, prefix_caching=False, enable_compression=True, compression_backend="kvpress",
               kvpress_method="knorm", compression_factor=2, compression_pipeline="prefill", position_mode=mode, **kw)


def _decode_positions(llm, prompts, max_tokens):
    """Run the job and return, per decode step, the (request id, position, KV length) triples that were fed."""
    seen = []
    inner = llm.model_runner.prepare_decode

    def spy(seqs):
        out = inner(seqs)
        seen.append([(s.seq_id, int(p), int(n)) for s, p, n in zip(seqs, out[1], out[3])])
        return out

    llm.model_runner.prepare_decode = spy
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))
    return seen, [o["token_ids"] for o in out]


@pytest.mark.parametrize("mode", ["compressed", "original"])
def test_positions_after_compression_follow_the_mode(mode):
    g = torch.Generator().manual_seed(3)
    lengths = [100, 64, 37]
    prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in lengths]
    llm = _engine(mode)
    steps, tokens = _decode_positions(llm, prompts, 6)
    assert llm.stats.compressions == len(prompts) and all(len(t) == 6 for t in tokens)
    first = {}
    for step in steps:
        for sid, pos, kv in step:
            first.setdefault(sid, []).append((pos, kv))
    assert len(first) == len(prompts)
    for n, (sid, rows) in zip(lengths, sorted(first.items())):
        kept = n // 2
        for j, (pos, kv) in enumerate(rows):
            # the j-th decode step stores the token sampled by the step before it: row kept + j of the pool
            assert kv == kept + j + 1
            assert pos == (kv - 1 if mode == "compressed" else n + j)


def test_modes_agree_without_compression_and_unknown_mode_is_refused():
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (50, 21)]
    outs = []
    for mode in ("compressed", "original"):
        llm = LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=64, max_model_len=256, device="cpu",
                  enforce_eager=True, position_mode=mode)
        outs.append([o["token_ids"] for o in
                     llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))])
    assert outs[0] == outs[1]
    with pytest.raises(ValueError):
        Config(model=tiny_llama_config(), position_mode="absolute")
