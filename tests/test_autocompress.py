"""Planning package and online controller (CPU only)."""
import torch

import fastcache_b200.autocompress as ac
from fastcache_b200.engine.auto_compress_controller import AutoCompressionController


def test_profiles_and_hardware_table():
    assert "mlp" in ac.list_profiles() and ac.get_profile("kvpress_snapkv").requires_attention
    b200 = ac.get_hardware_profile("NVIDIA B200")
    assert b200.gpu_arch is ac.GPUArch.BLACKWELL and b200.sm_count == 148
    assert b200.is_decode_memory_bound(128, 4096, 36, 8, 128, 4096)


def test_cost_model_prefers_compression_for_long_outputs(tmp_path):
    cm = ac.CostModel(ac.get_hardware_profile("B200"))
    long_w = ac.WorkloadContext(batch_size=128, seq_len=4096, expected_output_len=512, num_layers=36)
    short_w = ac.WorkloadContext(batch_size=1, seq_len=64, expected_output_len=2, num_layers=36)
    assert cm.compute_speedup("knorm", long_w) > 1.2
    assert cm.compute_speedup("mlp", short_w) < cm.compute_speedup("mlp", long_w)
    assert cm.get_break_even_output_len("mlp", long_w) < 512
    cal = ac.CalibrationData("B200")
    cal.update_decode(1.0, 2.0)
    cal.save(str(tmp_path / "c.json"))
    assert abs(ac.CalibrationData.load(str(tmp_path / "c.json")).decode_scale - cal.decode_scale) < 1e-9


def test_scheduler_plans_and_executor_trace():
    s = ac.AutoCompressScheduler(ac.get_hardware_profile("B200"))
    w = ac.WorkloadContext(batch_size=32, seq_len=4096, expected_output_len=256, num_layers=32)
    plan = s.schedule("mlp", w)
    assert plan.should_compress and plan.timing is ac.ExecutionTiming.ASYNC_DECODE and plan.chunking.enabled
    assert sum(len(plan.chunking.get_layers(c)) for c in range(plan.chunking.num_chunks)) == 32
    tiny = s.schedule("mlp", ac.WorkloadContext(batch_size=1, seq_len=32, expected_output_len=4))
    assert not tiny.should_compress
    ex = ac.PipelineExecutor()
    seen = []
    ex.on(ac.StepType.COMPRESS_CHUNK, lambda st: seen.append(st.chunk))
    ex.run(plan)
    assert seen == list(range(plan.chunking.num_chunks))
    assert s.schedule("snapkv", w).timing is ac.ExecutionTiming.INLINE_PREFILL


def test_methods_eviction_and_quantisation_round_trip():
    kv = [(torch.randn(2, 2, 64, 32), torch.randn(2, 2, 64, 32)) for _ in range(2)]
    out = ac.get_method("kvpress_knorm", compression_ratio=0.5).compress(kv)
    assert out[0][0].shape == (2, 2, 32, 32)
    q = [torch.randn(2, 4, 8, 32) for _ in range(2)]
    out = ac.get_method("snapkv", compression_ratio=0.75, window=8).compress(kv, queries=q)
    assert out[1][1].shape == (2, 2, 16, 32)
    for mode, tol in [("int8", 0.05), ("int8_asym", 0.05), ("int4", 0.6), ("nf4", 0.6), ("fp8_e4m3", 0.3)]:
        m = ac.get_method(f"quant_{mode}", group_size=32)
        back = m.decompress(m.compress(kv))
        assert (back[0][0] - kv[0][0]).abs().max() < tol, mode


def test_composed_pipeline_orders_memory_before_gemm():
    o = ac.PipelineOrchestrator(ac.get_hardware_profile("B200"))
    w = ac.WorkloadContext(batch_size=16, seq_len=8192, expected_output_len=256)
    c = o.create_composed_pipeline(["mlp", "streaming_llm"], w)
    assert [s.method for s in c.stages] == ["streaming_llm", "mlp"] and c.total_compression_ratio == 8.0


def _controller(**kw):
    return AutoCompressionController(compression_backend="mlp", kvpress_method=None, compression_factor=4,
                                     num_layers=32, num_kv_heads=32, head_dim=128, greenctx_enabled=True,
                                     decision_interval=1, **kw)


def test_controller_thresholds_and_sm_ratio_adaptation():
    c = _controller()
    assert c.decide(batch_size=4, seq_len=100, expected_output_len=512).pipeline == "none"
    d = c.decide(batch_size=32, seq_len=2048, expected_output_len=512)
    assert d.pipeline == "decode" and d.greenctx_enabled and abs(d.sm_compress_ratio - 0.40) < 1e-9
    for _ in range(5):
        c.update_decode(5.0)
        c.update_compress(20.0)
    d2 = c.decide(batch_size=32, seq_len=2048, expected_output_len=512)
    assert d2.sm_compress_ratio > d.sm_compress_ratio
    assert 1 <= d2.decode_layers_per_step <= 8


def test_controller_dual_batch_choice():
    c = _controller()
    assert c.decide_batch_type(waiting=0, running=5) == "decode"
    assert c.decide_batch_type(waiting=5, running=0) == "prefill"
    c.decide(batch_size=32, seq_len=2048, expected_output_len=512)     # pipeline -> decode
    picks = [c.decide_batch_type(waiting=10, running=10) for _ in range(16)]
    assert "decode" in picks and "prefill" in picks
    assert c.decide_batch_type(waiting=100, running=10) == "prefill"
