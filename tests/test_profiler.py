"""Analytic FLOP / byte model of the serving phases (utils_ccm/utils_profiler.py:163-428, :520-908) against numbers
worked out by hand for the Qwen3-8B and LLaVA-1.5-7B shapes."""
from types import SimpleNamespace

import pytest
import torch

from fastcache_b200.serving.profiler import (ComputeStats, LLaVAIntensityAnalyzer, LLMIntensityAnalyzer, PhaseCost,
                                             VisionEncoderAnalyzer, format_number)


def _qwen3_8b(tp=1):
    return LLMIntensityAnalyzer(4096, 36, 32, 8, 128, 12288, 151936, 2, tp)


def test_weight_and_kv_bytes_of_the_qwen3_8b_shape():
    a = _qwen3_8b()
    per_layer = 4096 * (32 + 16) * 128 + 32 * 128 * 4096 + 3 * 4096 * 12288
    assert a.layer_weight_params() == per_layer == 192_937_984
    assert a.weight_bytes() == (36 * per_layer + 151936 * 4096) * 2
    assert a.kv_bytes_per_token() == 2 * 36 * 8 * 128 * 2 == 147_456
    # 8 ranks: one KV head and an eighth of every projection per rank
    b = _qwen3_8b(tp=8)
    assert b.kv_bytes_per_token() == 147_456 / 8 and b.layer_weight_params() == per_layer / 8
    assert b.tp_message_bytes(128) == 128 * 4096 * 2


def test_prefill_is_compute_bound_and_decode_memory_bound():
    a = _qwen3_8b()
    pre = a.prefill(8, 4096)
    T = 8 * 4096
    gemm = 2.0 * T * 36 * 192_937_984
    attn = 4.0 * 8 * 32 * 128 * 4096 * 4096 / 2 * 36
    head = 2.0 * 8 * 4096 * 151936
    assert pre.flops == pytest.approx(gemm + attn + head)
    dec = a.decode(128, 2304)
    assert dec.bytes == pytest.approx(a.weight_bytes() + 128 * 2304 * 147_456)
    assert dec.flops == pytest.approx(2.0 * 128 * (36 * 192_937_984 + 4096 * 151936) + 4.0 * 128 * 32 * 128 * 2304 * 36)
    # ridge of a B200 at the measured peaks: about 1590e12 / 6650e9 = 239 FLOP per byte
    assert pre.intensity > 239 > dec.intensity
    # the roofline time is the slower of the two limits
    assert pre.time_ms(1590.0, 6650.0) == pytest.approx(pre.flops / 1590e12 * 1e3)
    assert dec.time_ms(1590.0, 6650.0) == pytest.approx(dec.bytes / 6650e9 * 1e3)
    both = pre + dec
    assert isinstance(both, PhaseCost) and both.flops == pre.flops + dec.flops and both.bytes == pre.bytes + dec.bytes


def test_compression_costs():
    a = _qwen3_8b()
    kv = 16 * 4096 * 147_456
    ev = a.eviction(16, 4096, 0.5)
    assert ev.bytes == pytest.approx(0.5 * kv + 2 * 0.5 * kv)           # K read once, kept K and V read and written
    assert ev.flops == pytest.approx(2.0 * 16 * 4096 * 36 * 8 * 128)
    m = a.compression_mlp(15, 640, 4)
    rows = 15 * 8 * 160 * 36 * 2
    assert m.flops == pytest.approx(2.0 * rows * (128 * 4 * 128 + 2 * 128 * 128))
    assert m.bytes == pytest.approx(15 * 640 * 147_456 * 1.25)


def test_tensor_driven_interface_from_a_config():
    cfg = SimpleNamespace(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2,
                          vocab_size=1024, intermediate_size=512, torch_dtype="bfloat16")
    a = LLMIntensityAnalyzer.from_config(cfg, peak_tflops=1000.0)
    assert (a.h, a.L, a.hq, a.hkv, a.d, a.ffn, a.vocab, a.b) == (256, 2, 4, 2, 64, 512, 1024, 2)
    ids = torch.zeros(3, 50, dtype=torch.long)
    rep = a.analyze_prefill(ids)
    c = a.prefill(3, 50)
    assert rep["phase"] == "prefill" and rep["batch_size"] == 3 and rep["seq_length"] == 50
    assert rep["flops"] == c.flops and rep["total_memory"] == pytest.approx(c.bytes)
    assert rep["theoretical_time"] == pytest.approx(c.flops / 1e15)
    assert rep["compute_intensity"] == pytest.approx(c.flops / c.bytes)
    past = [(torch.zeros(3, 2, 70, 64), torch.zeros(3, 2, 70, 64))] * 2
    dec = a.analyze_decode(ids[:, :1], past)
    assert dec["phase"] == "decode" and dec["seq_length"] == 71 and dec["flops"] == a.decode(3, 70).flops


def test_llava_request_breakdown_and_compression_report():
    a = LLaVAIntensityAnalyzer()
    assert isinstance(a.vision, VisionEncoderAnalyzer) and a.vision.n == 577
    r = a.request(text_tokens=64, out_tokens=128, factor=4)
    assert set(r) == {"vision", "projection", "prefill", "compress", "decode_per_token"}
    rows = 576 + 64
    assert r["prefill"].flops == a.llm.prefill(1, rows).flops
    assert r["compress"].flops == a.llm.compression_mlp(1, rows, 4).flops
    assert r["decode_per_token"].bytes == a.llm.decode(1, rows // 4 + 64).bytes
    assert "compress" not in a.request(factor=0)
    # the projector: two GEMMs 1024 -> 4096 -> 4096 over 576 rows per image
    assert a.projection(2).flops == 2.0 * 2 * 576 * (1024 * 4096 + 4096 * 4096)
    cache = [(torch.zeros(2, 32, 640, 128, dtype=torch.bfloat16),) * 2] * 3
    rep = a.analyze_kv_cache_compression(cache, image_len=576, text_len=64, compression_factor=4)
    per_seg = lambda n: 2.0 * 2 * 32 * (n // 4) * (128 * 4 * 128 + 2 * 128 * 128)          # noqa: E731
    assert rep["phase"] == "kv_cache_compression"
    assert rep["flops"] == pytest.approx(3 * 2 * (per_seg(576) + per_seg(64)))
    # a segment shorter than the factor is not merged
    short = a.analyze_kv_cache_compression(cache, image_len=576, text_len=3, compression_factor=4)
    assert short["flops"] == pytest.approx(3 * 2 * per_seg(576))
    ids = torch.zeros(1, 65, dtype=torch.long)
    mm = a.analyze_multimodal_prefill(ids, pixel_values=[torch.zeros(3, 336, 336)])
    text_only = a.analyze_multimodal_prefill(ids)
    assert mm["flops"] > text_only["flops"] and mm["seq_length"] == 65 + 575


def test_compute_stats_and_number_format():
    s = ComputeStats(100.0, 30.0, 10.0, 4, 7) + ComputeStats(50.0, 5.0, 5.0, 2, 9)
    assert (s.flops, s.memory_read, s.memory_write, s.batch_size, s.seq_length) == (150.0, 35.0, 15.0, 4, 9)
    assert s.total_memory == 50.0 and s.compute_intensity == 3.0
    assert s.per_sample_flops == 37.5 and s.per_sample_memory == 12.5
    assert format_number(1536) == "1.50K" and format_number(3 * 1024 ** 3) == "3.00G" and format_number(12) == "12.00"
    assert format_number(2_500_000, base=1000) == "2.50M"
