"""Green contexts on the GPU: the SM split comes up, kernels run on both groups, and an engine whose
compression streams live on the small group generates the same tokens as one without the split."""
import pytest
import torch

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
from helpers import random_compressor, tiny_llama_config

pytestmark = pytest.mark.gpu


def _partition(compress_sms):
    from fastcache_b200.ops.loader import ext
    try:
        return ext().greenctx_create(0, compress_sms, 0, 0)
    except RuntimeError as exc:
        if "not available" in str(exc):
            pytest.skip(f"driver without green contexts: {exc}")
        raise


def test_partition_and_kernels_on_both_groups():
    from fastcache_b200 import ops
    from fastcache_b200.ops.loader import ext
    got = _partition(36)
    total = got["total_sms"]
    assert got["main_sms"] + got["compress_sms"] <= total and 16 <= got["compress_sms"] <= 48
    assert got["main_sms"] >= total - 48
    main = torch.cuda.ExternalStream(got["main_stream"], device="cuda:0")
    comp = torch.cuda.ExternalStream(got["compress_stream"], device="cuda:0")
    ext().register_stream_sms(got["main_stream"], got["main_sms"])
    ext().register_stream_sms(got["compress_stream"], got["compress_sms"])
    torch.manual_seed(0)
    x = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16) * 0.03
    ref = (x.float() @ w.float().T)
    torch.cuda.synchronize()
    outs = []
    for s in (main, comp):
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            outs.append(ops.linear(x, w))
    torch.cuda.synchronize()
    for y in outs:
        assert torch.allclose(y.float(), ref, atol=0.25, rtol=0.02)
    assert ext().read_status(0) == 0


def test_engine_with_compression_on_the_small_group():
    _partition(36)                                    # skips when the driver has no green contexts
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, 1000, (96,), generator=g).tolist() for _ in range(4)]

    def run(green):
        comp = random_compressor(KVCacheLinearDecoupleCompressor, 2, 64, 4)
        llm = LLM(tiny_llama_config(), device="cuda:0", kvcache_block_size=32, num_kvcache_blocks=128,
                  max_model_len=512, max_num_seqs=8, enable_compression=True, async_compression=True,
                  compressor=comp, compression_backend="mlp", compression_pipeline="prefill",
                  greenctx_enabled=green, greenctx_compress_ratio=36 / 148)
        active, info = llm.model_runner.greenctx_enabled, dict(llm.model_runner._greenctx_info)
        out = [o["token_ids"] for o in llm.generate(prompts, sp)]
        n = llm.stats.compressions
        status = llm.model_runner.read_device_status()
        llm.exit()
        return active, info, out, n, status

    active, info, out, n, status = run(True)
    assert active and info["compress_sms"] >= 16 and info["main_sms"] > info["compress_sms"]
    assert n == 4 and status == 0
    _, _, plain, n2, _ = run(False)
    assert n2 == 4 and out == plain
