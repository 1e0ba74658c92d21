"""Names that scripts written against the reference import or call: the async-compression manager,
the MiniCPM compressor loader, the quantised-cache context, the model unwrapping helper, the
multimodal merge helpers and the import paths of the helper package."""
import os
from types import SimpleNamespace

import pytest
import torch

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.compress import (KVCacheLinearDecoupleCompressor, MiniCPMKVCompressor, load_minicpm_compressor,
                                     save_compressor)
from fastcache_b200.compress.kvpress_compat import get_underlying_model
from fastcache_b200.compress.quant import QuantizedCacheWrapper
from fastcache_b200.engine.async_compression import AsyncCompressionManager
from fastcache_b200.engine.sequence import CompressionState
from helpers import random_compressor, tiny_llama_config
from test_vision_cpu import _llava_cfg, _minicpm_cfg


def _engine():
    comp = random_compressor(KVCacheLinearDecoupleCompressor, 2, 64, 4)
    return LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=128, max_model_len=512, device="cpu",
               enforce_eager=True, enable_compression=True, compressor=comp, compression_backend="mlp",
               compression_pipeline="prefill")


def test_async_manager_views_engine_state():
    llm = _engine()
    mgr = llm.async_manager
    assert isinstance(mgr, AsyncCompressionManager) and llm.model_runner._async_manager is mgr
    from nanovllm.engine.llava_model_runner import AsyncCompressionManager as Aliased
    from nanovllm.engine.llava_model_runner import CompressionState as AliasedState     # llava_model_runner.py:43
    assert Aliased is AsyncCompressionManager and AliasedState is CompressionState
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    g = torch.Generator().manual_seed(0)
    seqs = [llm.add_request(torch.randint(3, 1000, (64,), generator=g).tolist(), sp) for _ in range(2)]
    assert mgr.get_state(seqs[0].seq_id) is CompressionState.NONE
    llm.step(apply_compression=False)                       # prefill only
    assert all(not s.is_compressed and mgr.get_effective_kv_len(s) == 65 for s in seqs)
    launched = mgr.start_async_compression(seqs)
    assert launched == [s.seq_id for s in seqs]
    # no side stream on the CPU: the launch degrades to the synchronous path and is complete at once
    assert all(mgr.is_compression_complete(s.seq_id) for s in seqs)
    assert mgr.wait_all_compressions(100.0) and mgr.wait_for_compression(seqs[0].seq_id, 10.0)
    assert all(mgr.get_state(s.seq_id) is CompressionState.COMPLETED for s in seqs)
    assert all(mgr.get_effective_kv_len(s) == 16 + 1 for s in seqs)
    assert mgr.start_async_compression(seqs) == []          # not eligible twice
    llm.scheduler.block_manager.check_invariants(seqs)
    while not llm.is_finished():
        llm.step()
    mgr.cleanup_seq(seqs[0].seq_id)
    assert mgr.get_state(seqs[0].seq_id) is CompressionState.NONE


def test_load_minicpm_compressor_strict(tmp_path):
    cfg = SimpleNamespace(num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, hidden_size=32,
                          head_dim=8)
    src = MiniCPMKVCompressor(cfg, 5, 2)
    for p in src.parameters():
        torch.nn.init.normal_(p, std=0.1)
    path = os.path.join(tmp_path, "minicpm_mlp.pth")
    save_compressor(src, path)
    got = load_minicpm_compressor(path, cfg, compression_factor=5)
    assert isinstance(got, MiniCPMKVCompressor) and not got.training and got.min_seq_len == 2
    for (n1, a), (n2, b) in zip(src.state_dict().items(), got.state_dict().items()):
        assert n1 == n2 and torch.equal(a, b)
    with pytest.raises(FileNotFoundError):
        load_minicpm_compressor(os.path.join(tmp_path, "absent.pth"), cfg)
    with pytest.raises(ValueError):
        load_minicpm_compressor(path, cfg, compression_factor=4)


def test_quantized_cache_context_restores_config():
    model = SimpleNamespace(config=SimpleNamespace())
    with QuantizedCacheWrapper(nbits=4)(model) as m:
        assert m is model and m.config.cache_implementation == "quantized"
        assert m.config.cache_config == {"backend": "quanto", "nbits": 4}
    assert not hasattr(model.config, "cache_implementation") and not hasattr(model.config, "cache_config")
    model.config.cache_implementation = "static"
    with QuantizedCacheWrapper(2)(model):
        pass
    assert model.config.cache_implementation == "static"


def test_get_underlying_model_shapes():
    stack = SimpleNamespace(layers=[1, 2])
    assert get_underlying_model(SimpleNamespace(language_model=stack)) is stack
    assert get_underlying_model(SimpleNamespace(language_model=SimpleNamespace(model=stack))) is stack
    assert get_underlying_model(SimpleNamespace(llm=SimpleNamespace(model=stack))) is stack
    assert get_underlying_model(SimpleNamespace(model=stack)) is stack
    with pytest.raises(AttributeError):
        get_underlying_model(SimpleNamespace(foo=1))


def test_llava_merge_helper_positions():
    llm = LLM(_llava_cfg(), device="cpu", kvcache_block_size=16, num_kvcache_blocks=32, max_model_len=128,
              enforce_eager=True)
    model = llm.model_runner.model
    ids = torch.tensor([5, 6, 500, 7, 8])
    pos = torch.arange(5)
    feats = model.get_image_features(torch.rand(1, 3, 56, 56))
    assert feats.shape[:2] == (1, 16)
    emb, p2 = model.merge_input_ids_with_image_features(ids, feats, pos)
    assert emb.shape[0] == 5 + 15 and p2.tolist() == list(range(20))
    assert torch.equal(emb[2:18], feats[0].to(emb.dtype))
    text = model.language_model.get_input_embeddings(ids)
    assert torch.equal(emb[:2], text[:2]) and torch.equal(emb[18:], text[3:])
    e0, p0 = model.merge_input_ids_with_image_features(torch.tensor([5, 6]), feats, torch.arange(2))
    assert e0.shape[0] == 2 and p0.tolist() == [0, 1]


def test_minicpm_get_vllm_embedding_scatter():
    llm = LLM(_minicpm_cfg(), device="cpu", kvcache_block_size=16, num_kvcache_blocks=32, max_model_len=256,
              enforce_eager=True)
    model = llm.model_runner.model
    q = model.query_num
    ids = torch.full((2, 16), 7)
    slices = [torch.rand(3, 28, 42), torch.rand(3, 42, 28)]
    data = {"input_ids": ids, "pixel_values": [slices, []],
            "tgt_sizes": [torch.tensor([[2, 3], [3, 2]]), torch.zeros(0, 2)],
            "image_bound": [torch.tensor([[1, 1 + q], [8, 8 + q]]), torch.zeros(0, 2)]}
    emb, vis = model.get_vllm_embedding(data)
    assert emb.shape[:2] == (2, 16) and vis[0].shape[:2] == (2, q) and vis[1].shape[0] == 0
    text = model.llm.get_input_embeddings(ids.reshape(-1)).reshape(2, 16, -1)
    assert torch.equal(emb[1], text[1]) and torch.equal(emb[0, 0], text[0, 0])
    assert torch.equal(emb[0, 1:1 + q], vis[0][0].to(emb.dtype)) and torch.equal(emb[0, 8:8 + q], vis[0][1].to(emb.dtype))


def test_reference_import_paths_resolve():
    import fastcache_paths
    from utils_ccm.module_ccm_v11 import (KVCacheCompressionLoss, KVCacheHybridCompressor,  # noqa: F401
                                          KVCacheLinearDecoupleCompressor as K1)
    from utils_ccm.utils_compress import press_select, exec_compression_methods, TimeTik  # noqa: F401
    from utils_ccm.utils_kvcachePool import KVCachePool  # noqa: F401
    from utils_ccm.utils_schedule_v11 import DynamicScheduler, TimestampManager, GPUMonitor  # noqa: F401
    from utils_ccm.utils_requests import Request, RequestStatus  # noqa: F401
    from utils_ccm.utils_profiler import LLaVAIntensityAnalyzer  # noqa: F401
    from nanovllm.kernels.zero_overhead_compress import ZeroOverheadCompressEngine  # noqa: F401
    from nanovllm.kernels.fused_compress import FusedCompressor  # noqa: F401
    assert K1 is KVCacheLinearDecoupleCompressor
    assert hasattr(fastcache_paths, "REPO_ROOT") and callable(fastcache_paths.ensure_sys_paths)


def test_runner_surface_drives_chunked_compression():
    comp = random_compressor(KVCacheLinearDecoupleCompressor, 2, 64, 4)
    llm = LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=128, max_model_len=512, device="cpu",
              enforce_eager=True, enable_compression=True, compressor=comp, compression_backend="mlp",
              compression_pipeline="decode", decode_layers_per_step=1, decode_overlap="hold")
    r = llm.model_runner
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    g = torch.Generator().manual_seed(3)
    seqs = [llm.add_request(torch.randint(3, 1000, (64,), generator=g).tolist(), sp) for _ in range(2)]
    llm.step(apply_compression=False)
    assert r.preare_block_tables(seqs).shape == (2, 4) and r.prepare_sample(seqs).tolist() == [0.0, 0.0]
    assert r.get_compressed_block_count(seqs[0].seq_id) == 0 and r.get_blocks_to_free(seqs[0].seq_id) == []
    r.start_decode_overlap_compression(seqs)
    assert all(s.hold for s in seqs) and not r.update_decode_overlap_engine(2)     # refused while in flight
    assert r.step_decode_overlap_compression(seqs) == []                           # layer 0 of 2
    done = r.step_decode_overlap_compression(seqs)
    assert done == seqs and all(not s.hold and s.kv_cache_len == 17 for s in seqs)
    llm.async_manager.finalize(seqs)
    assert all(len(s.block_table) == 2 for s in seqs)
    llm.scheduler.block_manager.check_invariants(seqs)
    assert r.update_decode_overlap_engine(2) and r.decode_layers_per_step == 2
    r.clear_compressed_lens([seqs[0].seq_id])
    assert r.get_compressed_block_count(seqs[0].seq_id) == 0 and r.get_compressed_block_count(seqs[1].seq_id) == 1
    while not llm.is_finished():
        llm.step()
    # run_model: logits from metadata prepared by the caller
    seq = llm.add_request([5, 6, 7, 8], sp)
    llm.scheduler.schedule()
    ids, pos, _ = r.prepare_prefill([seq])
    assert r.run_model(ids, pos, True).shape[-1] == 1024


def test_harness_reference_method_names():
    import fastcache_b200.serving.harness as h
    from fastcache_b200.compress.kvpress_compat import create_kvpress_compressor
    from fastcache_b200.engine.block_manager import BlockManager, compute_hash
    from fastcache_b200.utils.streams import StreamPool

    r = h.Request(1, [1, 2, 3])
    for step in (r.enter_queue, r.start_processing, r.start_prefill, r.end_prefill, r.start_decode, r.end_decode):
        step()
    r.complete("ok")
    d = r.to_dict()
    assert d["status"] == "completed" and d["metrics"]["total_time"] >= 0 and r.result == "ok"
    t = h.TimestampManager()
    t.create_request(["a", "b"])
    for i, st in enumerate(["prefill_queueing_start", "prefill_start", "prefill_finish", "compress_queueing",
                            "compress_start", "compress_finish", "decoding_queueing", "decode_start",
                            "decoding_finish"]):
        t.record_timestamp(["a"], st, float(i))
    t.record_timestamp(["a"], "generated_lens", 4)
    summary, durations = t.analyze_timestamps()
    assert summary["total_generated_lens"] == 4 and summary["average_times"]["ttft"] == 2.0
    assert durations["tpot"] == [0.25] and t.get_timestamps("b") == {}
    t.remove_request("a")
    assert t.analyze_timestamps()[0]["total_generated_lens"] == 0
    pool = h.KVCachePool()
    kv = [(torch.zeros(2, 1, 3, 4), torch.zeros(2, 1, 3, 4))]
    pool.store_kvcache([7, 8], kv)
    assert pool.get_kvcache(7)[0][0].shape == (1, 1, 3, 4) and len(pool.get_kvcache([7, 8])) == 2
    assert pool.release_kvcache([7]) and not pool.release_kvcache(7)
    pool.clear_kvcache()
    assert pool.get_stats()["entries"] == 0
    sch = h.DynamicScheduler(max_batch_size=2, std_batch_threshold_decoding=5, max_wait_time=0.0)
    from types import SimpleNamespace as NS
    sch.add_request(NS(batch={"input_ids": torch.zeros(1, 9)}), "prefill")
    sch.add_request(NS(batch={"request_size": 3}), "decoding")
    sch.add_request(NS(batch={"request_size": 3}), "decoding")
    assert sch.get_queue_status()["prefill_count"] == 1 and sch.adaptive_batch_size("decoding") == 1
    assert sch.binary_search_last_le([1, 2, 5], 3) == 1 and sch.binary_search_last_le([4], 3) == -1
    sch.update_performance({"batch_size": 4})
    assert sch.get_current_performance() == 4
    kind, batch = sch.select_batch()
    assert kind == "prefill" and sch.get_queue_status()["current_mode"] == "prefill"
    mon = h.GPUMonitor(period=0.01)
    mon.accum_state_round("prefill")
    mon.accum_state_round("prefill")
    assert mon.get_state_round_info() == "prefill 2" and mon.check_gpu_stats() == {}
    c = create_kvpress_compressor("knorm", 4)
    assert abs(c.compression_factor - 4) < 1e-9 and c.get_compressed_length(100) == 25
    out = c.forward([(torch.randn(1, 2, 16, 8), torch.randn(1, 2, 16, 8))])
    assert out[0][0].shape == (1, 2, 4, 8)
    assert compute_hash([1, 2, 3], 5) == BlockManager.compute_hash([1, 2, 3], 5)
    sp_ = StreamPool(None, [])
    assert sp_.streams == [] and not sp_.greenctx_info.available


def test_layer_level_helpers():
    from fastcache_b200.layers.attention import store_kvcache
    from fastcache_b200.layers.layernorm import RMSNorm
    from fastcache_b200.layers.rotary_embedding import apply_rotary_emb, get_rope
    from fastcache_b200.parallel.tp import get_tp_device

    torch.manual_seed(0)
    k_cache, v_cache = torch.zeros(3, 2, 4, 8), torch.zeros(3, 2, 4, 8)     # [blocks, Hkv, block, D]
    k, v = torch.randn(3, 2, 8), torch.randn(3, 2, 8)
    store_kvcache(k, v, k_cache, v_cache, torch.tensor([5, -1, 9]))
    assert torch.equal(k_cache[1, :, 1], k[0]) and torch.equal(v_cache[2, :, 1], v[2])
    assert float(k_cache.abs().sum()) == float(k[0].abs().sum() + k[2].abs().sum())     # slot -1 skipped
    norm = RMSNorm(8)
    x, res = torch.randn(4, 8), torch.randn(4, 8)
    assert torch.equal(norm.rms_forward(x), norm(x))
    a, b = norm.add_rms_forward(x, res)
    a2, b2 = norm(x, res)
    assert torch.equal(a, a2) and torch.equal(b, b2)
    rope = get_rope(8, 8, 64, 10000.0)
    pos = torch.tensor([0, 3, 7])
    q = torch.randn(3, 2, 8)
    cs = rope.cos_sin_cache[pos]
    q_rot, _ = rope(pos, q, q)
    assert torch.allclose(apply_rotary_emb(q, cs[:, None, :4], cs[:, None, 4:]), q_rot)
    assert torch.allclose(apply_rotary_emb(q[:1], cs[:1, None, :4], cs[:1, None, 4:]), q[:1])     # position 0
    assert get_tp_device().type in ("cpu", "cuda")


def test_green_context_partitions_are_created_once_per_split(monkeypatch):
    """Against a fake extension: the same SM split asked for twice reuses its partition; more compression
    streams are added to it on demand; another split is another partition."""
    import fastcache_b200.ops.loader as loader
    import fastcache_b200.utils.streams as streams

    class FakeExt:
        def __init__(self):
            self.created, self.extra, self.registered = [], 0, {}

        def sm_count(self, index):
            return 148

        def greenctx_create(self, index, want, a, b):
            self.created.append(want)
            base = 1000 * len(self.created)
            return {"main_stream": base + 1, "compress_stream": base + 2, "main_sms": 148 - want,
                    "compress_sms": want, "total_sms": 148}

        def greenctx_extra_stream(self, compress_stream, prio):
            self.extra += 1
            return compress_stream + 10 * self.extra

        def register_stream_sms(self, ptr, sms):
            self.registered[ptr] = sms

    class FakeStream:
        def __init__(self, ptr, device=None):
            self.cuda_stream = ptr

    fake = FakeExt()
    monkeypatch.setattr(loader, "ext", lambda: fake)
    monkeypatch.setattr(loader, "ext_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "ExternalStream", FakeStream)
    monkeypatch.setattr(streams, "_PARTITIONS", {})
    dev = torch.device("cuda", 0)
    a = streams.try_create_greenctx_streams(dev, 36 / 148, 1)
    b = streams.try_create_greenctx_streams(dev, 36 / 148, 2)
    c = streams.try_create_greenctx_streams(dev, 36 / 148, 1)
    assert fake.created == [36] and a["main"] is b["main"] is c["main"]
    assert len(a["compress"]) == 1 and len(b["compress"]) == 2 and len(c["compress"]) == 1 and fake.extra == 1
    assert b["compress"][0] is a["compress"][0] and fake.registered[b["compress"][1].cuda_stream] == 36
    d = streams.try_create_greenctx_streams(dev, 0.40, 1)
    assert fake.created == [36, 59] and d["compress_sms"] == 59 and d["main"] is not a["main"]


def test_alias_submodules_are_the_same_module_objects():
    """`nanovllm.<pkg>.<module>` must be the module of this package itself (not a second copy whose classes
    differ and whose relative imports point into the alias package)."""
    import importlib
    import fastcache_b200.autocompress.cost_model as cm
    import fastcache_b200.layers.linear as lin
    assert importlib.import_module("nanovllm.layers.linear") is lin
    assert importlib.import_module("nanovllm.autocompress.cost_model") is cm
    from nanovllm.layers.layernorm import RMSNorm as A
    from fastcache_b200.layers.layernorm import RMSNorm as B
    from nanovllm.models.qwen3 import Qwen3ForCausalLM  # noqa: F401
    from nanovllm.utils.streams import GreenCtxInfo  # noqa: F401
    assert A is B
    with pytest.raises(ImportError):
        importlib.import_module("nanovllm.no_such_module")
