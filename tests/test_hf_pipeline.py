"""The HuggingFace-style three-stage pipeline on a tiny random Llama (CPU): batched, left-padded,
pooled and compressed serving must give the tokens of serving each request alone."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from fastcache_b200.compress import KVCacheLinearDecoupleCompressor  # noqa: E402
from fastcache_b200.compress.kvpress_compat import KVPressCompressor  # noqa: E402
from fastcache_b200.serving.hf_pipeline import (HFPipelineTester, TransformersBackend, cache_to_pairs,  # noqa: E402
                                                create_attention_mask_from_padding, left_pad, merge_kv_cache,
                                                pairs_to_cache)
from helpers import random_compressor  # noqa: E402


def _model():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=300, max_position_embeddings=512)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval()


def _alone(model, prompt, n_new, compressor=None, it_len=(0, 0)):
    """One request, no padding: prefill, optional compression of its cache, greedy decode."""
    ids = torch.tensor([prompt])
    with torch.no_grad():
        out = model(input_ids=ids, use_cache=True)
        kv = [(k, v) for k, v in cache_to_pairs(out.past_key_values)]
        if compressor is not None:
            kv = compressor(kv, list(it_len))
        cache = pairs_to_cache([(k.contiguous(), v.contiguous()) for k, v in kv])
        n = kv[0][0].shape[2]
        toks = [int(out.logits[0, -1].argmax())]
        for step in range(n_new - 1):
            o = model(input_ids=torch.tensor([[toks[-1]]]), past_key_values=cache, use_cache=True,
                      attention_mask=torch.ones(1, n + step + 1, dtype=torch.long),
                      position_ids=torch.tensor([[n + step]]))
            toks.append(int(o.logits[0, -1].argmax()))
    return toks


def _prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(3, 300, (n,), generator=g).tolist() for n in (9, 23, 14, 31, 17, 12, 26)]


@pytest.mark.parametrize("kind", ["none", "ccm", "knorm"])
def test_pipeline_equals_serving_each_request_alone(kind):
    model = _model()
    comp, split = None, [0] * 7
    if kind == "ccm":
        comp = random_compressor(KVCacheLinearDecoupleCompressor, 2, 16, 2, min_seq_len=2)
        split = [4, 0, 6, 8, 0, 5, 10]                  # image rows differ per request
    elif kind == "knorm":
        comp = KVPressCompressor("knorm", 0.5)
    prompts = _prompts()
    tester = HFPipelineTester(TransformersBackend(model), comp, batching=[3, 2, 5], req_per_sec=400.0,
                              max_wait_time=0.02)
    res = tester.run_concurrent_test(prompts, max_new_tokens=6, image_rows=split)
    assert res.completed == 7 and res.failed == 0 and not res.compression["errors"]
    for r, p, img in zip(tester.requests, prompts, split):
        assert r.output == _alone(model, p, 6, comp, (img, len(p) - img)), (kind, r.request_id)
    if comp is not None:
        assert res.compression["calls"] == 7 and res.compression["rows_out"] < res.compression["rows_in"]
    assert tester.pool.get_stats()["entries"] == 0                      # every cache left the pool
    summary, _ = tester.timestamps.analyze_timestamps()
    assert summary["total_generated_lens"] == 42 and summary["average_times"]["ttft"] > 0
    assert res.ttft["p50"] > 0 and res.throughput_tok_s > 0


def test_padding_helpers():
    ids, mask = left_pad([[1, 2, 3], [4]], 0, "cpu")
    assert ids.tolist() == [[1, 2, 3], [0, 0, 4]] and mask.tolist() == [[1, 1, 1], [0, 0, 1]]
    assert create_attention_mask_from_padding([2, 3], 3, "cpu").tolist() == [[0, 1, 1], [1, 1, 1]]
    a = [(torch.ones(1, 2, 3, 4), torch.ones(1, 2, 3, 4))]
    b = [(torch.ones(1, 2, 5, 4), torch.ones(1, 2, 5, 4))]
    merged, lens = merge_kv_cache([a, b])
    assert lens == [3, 5] and merged[0][0].shape == (2, 2, 5, 4) and float(merged[0][0][0, :, :2].abs().sum()) == 0


def test_a_failing_batch_is_reported_not_raised():
    model = _model()

    def broken(kv, it_len):
        raise RuntimeError("compressor down")

    tester = HFPipelineTester(TransformersBackend(model), broken, batching=[4, 4, 8], req_per_sec=400.0,
                              max_wait_time=0.02)
    res = tester.run_concurrent_test(_prompts()[:3], max_new_tokens=3)
    assert res.failed == 3 and res.completed == 0 and "compressor down" in res.compression["errors"][0]


def test_cli_runs_the_hf_pipeline():
    from fastcache_b200.serving import testcon
    rows = testcon.main(["--engine", "hf", "--device", "cpu", "--use_compression", "--comp_mode", "ccm",
                         "--num_samples", "4", "--max_new_tokens", "4", "--req_per_sec", "300", "--no_log",
                         "--prefill_batch_size", "2", "--compress_batch_size", "2", "--decoding_batch_size", "4"])
    r = rows[0]
    assert r["engine"] == "hf" and r["result"]["completed"] == 4 and r["result"]["output_tokens"] == 16
    assert r["result"]["compression"]["calls"] == 4 and r["stage_averages"]["generated_lens"] == 4.0


def test_quantiser_as_the_compression_stage():
    from fastcache_b200.compress.quant import SimpleKVQuantizer
    model = _model()
    q = SimpleKVQuantizer(8)
    tester = HFPipelineTester(TransformersBackend(model), q, batching=[4, 4, 8], req_per_sec=400.0, max_wait_time=0.02)
    res = tester.run_concurrent_test(_prompts()[:4], max_new_tokens=4)
    assert res.completed == 4 and res.compression["calls"] == 4
    assert res.compression["rows_in"] == res.compression["rows_out"]          # precision, not length
    assert q.totalTime > 0
