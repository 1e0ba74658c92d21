"""HF-tensor front ends: batched / chunked / stream-pipelined merge compression and the eviction presses."""
import torch

from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
from fastcache_b200.compress.batched import (BatchedGEMMCompressor, PipelineAsyncCompressor,
                                             create_zero_overhead_compressor)
from fastcache_b200.compress.kvpress_compat import (KVPressCompressor, exec_compression_methods, press_select)
from fastcache_b200.compress.scorers import score_keys, select_keep
from helpers import random_compressor


def _kv(L=4, B=2, H=2, S=50, D=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B, H, S, D, generator=g), torch.randn(B, H, S, D, generator=g)) for _ in range(L)]


def test_batched_equals_module_and_chunks_equal_whole():
    m = random_compressor(KVCacheLinearDecoupleCompressor, 4, 16, 4)
    kv = _kv()
    want = m(kv, [13, 37])
    b = BatchedGEMMCompressor().load_from_original_compressor(m)
    got = b(kv, [13, 37])
    for (k1, v1), (k2, v2) in zip(want, got):
        assert torch.allclose(k1, k2, atol=1e-5) and torch.allclose(v1, v2, atol=1e-5)
    eng = create_zero_overhead_compressor(m, layers_per_decode_step=3)
    eng.start_compression(5, kv, [13, 37])
    steps = 0
    while not eng.step_compression(5):
        steps += 1
    assert steps == 1 and eng.get_stats()["completed"] == 1
    out = eng.get_compressed_cache(5)
    assert len(out) == 4 and torch.allclose(out[3][1], want[3][1], atol=1e-5)
    p = PipelineAsyncCompressor(b, num_streams=2)
    p.submit_compression(1, kv, [13, 37])
    assert p.is_compression_ready(1) and p.get_compressed_len(1) == want[0][0].shape[2]
    assert torch.allclose(p.wait_compression(1)[0][0], want[0][0], atol=1e-5)
    p.cleanup(1)
    assert p.get_compressed_len(1) is None


def test_scorers_basic_properties():
    g = torch.Generator().manual_seed(1)
    k, v = torch.randn(2, 40, 8, generator=g), torch.randn(2, 40, 8, generator=g)
    k[0, 7] *= 100.0                                      # huge norm: knorm (kvpress) drops it, knorm_ref keeps it
    idx = select_keep(score_keys("knorm", k), 20)
    assert 7 not in idx[0].tolist() and idx.shape == (2, 20) and (idx[:, 1:] > idx[:, :-1]).all()
    assert 7 in select_keep(score_keys("knorm_ref", k), 5)[0].tolist()
    s = select_keep(score_keys("streaming_llm", k, n_sink=4), 10)[0].tolist()
    assert s == [0, 1, 2, 3] + list(range(34, 40))
    q = torch.randn(4, 8, 8, generator=g)
    sk = score_keys("snapkv", k, v, q, window=8, kernel_size=5)
    assert torch.isinf(sk[:, -8:]).all() and sk.shape == (2, 40)
    kept = select_keep(sk, 12)
    assert set(range(32, 40)) <= set(kept[0].tolist())     # the observation window is always kept
    ea = score_keys("expected_attention", k, v, q, n_sink=2)
    assert torch.isinf(ea[:, :2]).all() and (ea[:, 2:] >= 0).all()
    assert score_keys("tova", k, v, q).shape == (2, 40)


def test_presses_and_engine_side_compressor():
    kv = _kv(L=2, S=64)
    out, secs = exec_compression_methods(kv, "Knorm", 0.5)
    assert out[0][0].shape[2] == 32 and secs >= 0.0
    c = KVPressCompressor("streaming_llm", 0.75, n_sink=4)
    o = c(kv)
    assert o[1][1].shape[2] == 16 and torch.equal(o[0][0][:, :, :4], kv[0][0][:, :, :4])
    assert torch.equal(o[0][0][:, :, 4:], kv[0][0][:, :, -12:]) and c.get_stats()["calls"] == 1
    # a query-based method without queries degrades to uniform striding, like the reference engine
    u = KVPressCompressor("snapkv", 0.5)(kv)
    assert u[0][0].shape[2] == 32
    assert press_select("ExpectedAttention", 0.5).method == "expected_attention"


def test_self_benchmarks_agree_with_the_modules():
    from fastcache_b200.compress.batched import benchmark_batched_vs_original, benchmark_fused_vs_pytorch
    r = benchmark_batched_vs_original(num_layers=2, num_heads=2, seq_len=50, head_dim=16, image_len=20, iters=2,
                                      warmup=1, device="cpu", verbose=False)
    assert r["max_abs_diff"] < 1e-4 and r["compressed_len"] == 20 // 5 + 30 // 5 and r["speedup"] > 0
    r = benchmark_fused_vs_pytorch(64, 32, 16, iters=2, warmup=1, device="cpu", verbose=False)
    assert r["max_abs_diff"] < 1e-4
