"""The host-side race detector for the KV pool (utils/stream_check.py) on stand-in streams and events."""
import pytest

from fastcache_b200.utils.stream_check import StreamOrderChecker, StreamOrderError


class _Obj:
    pass


def _setup():
    c = StreamOrderChecker()
    main, side = _Obj(), _Obj()
    c.name_stream(main, "main")
    c.name_stream(side, "compress")
    return c, main, side


def test_read_after_write_on_another_stream_needs_an_event():
    c, main, side = _setup()
    c.launch(main, writes=[3, 4], what="prefill")
    with pytest.raises(StreamOrderError, match="reads .* block 3 .* prefill on main"):
        c.launch(side, reads=[3], what="compression")
    ev = _Obj()
    c.record(ev, main)
    c.wait(side, ev)
    c.launch(side, reads=[3], writes=[4], what="compression")          # ordered now
    with pytest.raises(StreamOrderError, match="writes"):
        c.launch(main, writes=[4], what="decode")                      # main never waited for the compression
    done = _Obj()
    c.record(done, side)
    c.wait(main, done)
    c.launch(main, reads=[3], writes=[4], what="decode")


def test_event_carries_only_what_came_before_it():
    c, main, side = _setup()
    ev = _Obj()
    c.record(ev, side)                       # recorded BEFORE the side stream's write
    c.launch(side, writes=[7], what="chunk 1")
    c.wait(main, ev)
    with pytest.raises(StreamOrderError):
        c.launch(main, reads=[7], what="decode")


def test_write_after_read_and_freed_block_reuse():
    """A block that one request's compression still reads must not be rewritten by its next owner's prefill."""
    c, main, side = _setup()
    c.launch(main, writes=[1], what="prefill of request A")
    c.wait_stream(side, main)
    c.launch(side, reads=[1], writes=[2], what="compression of request A into its shadow blocks")
    # the request is aborted, block 1 goes back to the pool and to request B without an event wait
    with pytest.raises(StreamOrderError, match="writes .* block 1 .* reads"):
        c.launch(main, writes=[1], what="prefill of request B")


def test_row_ranges_and_concurrent_readers():
    c, main, side = _setup()
    c.launch(main, writes=[(5, 0, 10)], what="prefill")
    c.wait_stream(side, main)
    c.launch(side, reads=[(5, 0, 10)], what="compression")             # reads rows 0-9
    c.launch(main, reads=[(5, 0, 10)], writes=[(5, 10, 11)], what="decode")   # appends row 10: no overlap, fine
    c.launch(main, reads=[(5, 0, 11)], writes=[(5, 11, 12)], what="decode")
    with pytest.raises(StreamOrderError):
        c.launch(main, writes=[(5, 9, 10)], what="rewrite of a row the compression reads")


def test_host_synchronisation_orders_everything_before_it():
    c, main, side = _setup()
    c.launch(side, writes=[9], what="compression")
    c.synchronize()                                                     # torch.cuda.synchronize()
    c.launch(main, reads=[9], writes=[9], what="decode")
    c.launch(side, writes=[8], what="compression")
    c.synchronize(main)                                                 # only the main stream was waited for
    with pytest.raises(StreamOrderError):
        c.launch(main, reads=[8], what="decode")


def test_collecting_mode_and_unknown_event():
    c = StreamOrderChecker(raise_on_violation=False)
    a, b = _Obj(), _Obj()
    c.launch(a, writes=[1])
    c.launch(b, reads=[1])
    c.wait(b, _Obj())
    assert len(c.violations) == 2 and "never recorded" in c.violations[1]


def test_engine_runs_clean_under_the_checker_and_a_dropped_wait_is_caught():
    """Tiny CPU engine (no streams: everything is one stream) passes; the checker sees every step."""
    from fastcache_b200 import LLM, SamplingParams
    hf = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=128, max_position_embeddings=512,
              rms_norm_eps=1e-6, rope_theta=10000.0, torch_dtype="float32")
    llm = LLM(hf, device="cpu", kvcache_block_size=16, num_kvcache_blocks=64, max_model_len=256,
              enable_compression=True, compression_factor=2, compression_backend="kvpress", kvpress_method="knorm",
              check_streams=True)
    outs = llm.generate([[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12] * 3, [5, 6, 7, 8] * 6],
                        SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert len(outs) == 2 and llm.stream_check.launches > 6 and not llm.stream_check.violations


@pytest.mark.parametrize("pipeline,overlap", [("decode", "shadow"), ("decode", "hold"), ("prefill", "shadow")])
def test_cpu_engine_pipelines_under_the_checker(pipeline, overlap):
    import torch
    from fastcache_b200 import LLM, SamplingParams
    from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
    from helpers import random_compressor, tiny_llama_config
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (96,), generator=g).tolist() for _ in range(3)]
    llm = LLM(tiny_llama_config(num_hidden_layers=4), kvcache_block_size=16, num_kvcache_blocks=128,
              max_model_len=512, device="cpu", enforce_eager=True, enable_compression=True, compression_backend="mlp",
              compression_factor=2, compressor=random_compressor(KVCacheLinearDecoupleCompressor, 4, 64, 2),
              compression_pipeline=pipeline, decode_layers_per_step=1, decode_overlap=overlap, check_streams=True)
    llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    assert llm.stats.compressions == 3 and not llm.stream_check.violations


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["async", "decode-shadow", "decode-hold"])
def test_gpu_engine_side_stream_compression_is_ordered(mode):
    """Real CUDA streams: compression on side streams while other requests prefill and decode, blocks freed and
    reused, requests finishing at different steps.  Every launch is ordered after the accesses it conflicts with."""
    import torch
    from fastcache_b200 import LLM, SamplingParams
    from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
    from helpers import random_compressor, tiny_qwen3_config
    cfg = tiny_qwen3_config(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                            intermediate_size=1024, vocab_size=2048, num_hidden_layers=4)
    comp = random_compressor(KVCacheLinearDecoupleCompressor, 4, 128, 2)
    kw = dict(compression_pipeline="prefill", async_compression=True) if mode == "async" else \
        dict(compression_pipeline="decode", decode_layers_per_step=1, decode_overlap=mode.split("-")[1])
    llm = LLM(cfg, device="cuda", kvcache_block_size=32, num_kvcache_blocks=96, max_model_len=512, max_num_seqs=4,
              max_num_batched_tokens=512, enable_compression=True, compression_backend="mlp", compression_factor=2,
              compressor=comp, check_streams=True, init_device="cpu", **kw)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 2048, (int(n),), generator=g).tolist() for n in (180, 64, 200, 96, 150, 130, 70, 190)]
    sps = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=True) for m in (10, 3, 14, 6, 9, 12, 4, 8)]
    out = llm.generate(prompts, sps)
    assert len(out) == 8 and llm.stats.compressions >= 6
    assert not llm.stream_check.violations and llm.stream_check.launches > 15
    llm.scheduler.block_manager.check_invariants([])
    llm.exit()
