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


def test_reference_named_planning_surface(tmp_path):
    """Factories, step-wise executor, measurement-keyed calibration, timing rules and the
    argument-style manager calls that scripts written against the reference use."""
    import torch
    from fastcache_b200.autocompress import (AutoCompressManager, CompressionConfig, WorkloadContext,
                                             AdaptiveCompressionWrapper)
    from fastcache_b200.autocompress.context import get_hardware_profile
    from fastcache_b200.autocompress.cost_model import CalibrationData, CostModel
    from fastcache_b200.autocompress.execution import (ChunkingConfig, ExecutionPlan, ExecutionTiming,
                                                       PipelineExecutor, StepType, StreamManager)
    from fastcache_b200.autocompress.kernels import TileLangKernelGenerator
    from fastcache_b200.autocompress.methods import MethodRegistry, get_method

    plan = ExecutionPlan.create_async_plan("mlp", 3.0, 1.2, chunk_size=8, num_layers=36)
    assert plan.chunking.num_chunks == 5 and plan.is_valid() and "5 x 8 layers" in plan.summary()
    assert [s.type for s in plan.to_schedule()].count(StepType.COMPRESS_CHUNK) == 5
    assert ExecutionPlan.create_sync_plan("mlp", 1.0, 0.9).is_valid() is False
    assert ExecutionPlan.create_inline_plan("snapkv", 0.5, 1.1).timing is ExecutionTiming.INLINE_PREFILL
    none = ExecutionPlan.create_no_compress_plan()
    assert not none.should_compress and [s.type for s in none.steps] == [StepType.PREFILL, StepType.DECODE]
    assert ChunkingConfig.create(30, 4).num_chunks == 8 and ChunkingConfig.create(30, 4).chunk_size == 4
    seen = []
    ex = PipelineExecutor()
    ex.register_callback(StepType.COMPRESS_CHUNK, lambda st: seen.append(st.chunk))
    ex.register_callback(StepType.FREE_BLOCKS, lambda st: 1 / 0)
    ex.set_plan(plan)
    assert ex.execute_all() is False and seen == [0, 1, 2, 3, 4]
    st = ex.get_statistics()
    assert st["total_steps"] == len(plan.steps) and len(st["warnings"]) == 1
    sm = StreamManager()
    sm.initialize()
    assert sm.get_main_stream() is sm.main and sm.get_compress_stream() is sm.compress
    sm.synchronize_compress_to_main()

    hw = get_hardware_profile("B200")
    cal = CalibrationData(gpu_name="B200")
    cal.add_decode_measurement(8, 1024, 7.5)
    cal.add_compress_measurement("mlp", 1024, 8, 2.25)
    path = str(tmp_path / "cal.json")
    cal.save(path)
    cm = CostModel(hw, CalibrationData.load(path))
    w = WorkloadContext(batch_size=8, seq_len=1024, expected_output_len=128)
    assert cm.estimate_decode_latency(w) == 7.5 and cm.estimate_compress_latency("mlp", w) == 2.25
    assert cm.estimate_decode_latency(w, compressed=True, compression_ratio=4.0) < 7.5
    total, parts = cm.estimate_total_time(w, "mlp", async_mode=True)
    base, _ = cm.estimate_total_time(w)
    assert parts["compress_ms"] == 2.25 and 0.0 <= parts["overlap"] <= 1.0 and total < base

    small = WorkloadContext(batch_size=2, seq_len=2048)
    big = WorkloadContext(batch_size=16, seq_len=2048)
    assert get_method("mlp").get_optimal_timing(small, hw) is ExecutionTiming.AFTER_PREFILL
    assert get_method("mlp").get_optimal_timing(big, hw) is ExecutionTiming.ASYNC_DECODE
    assert get_method("snapkv").get_optimal_timing(big, hw) in (ExecutionTiming.INLINE_PREFILL,
                                                                ExecutionTiming.AFTER_PREFILL)
    assert get_method("quant_int8").get_optimal_timing(small, hw) is ExecutionTiming.ASYNC_DECODE
    assert "mlp" in MethodRegistry.list_methods()

    mgr = AutoCompressManager(CompressionConfig(method="knorm", compression_ratio=0.5), hardware=hw)
    plan2 = mgr.get_plan(16, 4096, 512)
    assert isinstance(mgr.should_compress(16, 4096, 512), bool) and plan2 is not None
    kv = [(torch.randn(1, 2, 32, 8), torch.randn(1, 2, 32, 8))]
    assert mgr.execute_sync(kv)[0][0].shape[2] == 16
    got = []
    h = mgr.execute_async(kv, callback=got.append)
    assert h.is_ready() and h.get_result()[0][0].shape[2] == 16 and len(got) == 1
    assert mgr.get_statistics()["compressed"] == 2
    wrap = AdaptiveCompressionWrapper(lambda kv_, it_len=(0, 0): kv_)
    assert wrap.compress(kv, expected_output_len=4) is not None and wrap.get_last_plan() is not None
    gen = TileLangKernelGenerator()
    q = gen.generate_quantize_kernel(8)(torch.randn(4, 128))
    assert torch.allclose(gen.generate_dequantize_kernel(8)(q), gen.generate_dequantize_kernel()(q))
    assert gen.generate_sparse_gather_kernel()(torch.arange(6.).reshape(3, 2), torch.tensor([2, 0])).tolist() == \
        [[4.0, 5.0], [0.0, 1.0]]


def test_examples_run(capsys):
    import runpy
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    old = sys.argv
    try:
        sys.argv = ["autocompress_demo.py"]
        runpy.run_path(str(root / "examples" / "autocompress_demo.py"), run_name="__main__")
    finally:
        sys.argv = old
    out = capsys.readouterr().out
    assert "hardware: NVIDIA B200" in out and "ExecutionPlan for 'mlp'" in out and "best of three" in out


def test_cached_decision_does_not_outlive_a_change_of_the_size_gate():
    from fastcache_b200.engine.auto_compress_controller import AutoCompressionController
    c = AutoCompressionController(compression_backend="kvpress", kvpress_method="knorm", compression_factor=2,
                                  num_layers=36, num_kv_heads=8, head_dim=128, greenctx_enabled=False,
                                  decision_interval=4, min_seq_len=256, min_output_len=64, min_speedup=1.05,
                                  force_compress=False, dual_batch_enabled=False, dual_batch_interval=4)
    assert c.decide(batch_size=8, seq_len=3072, expected_output_len=4).pipeline == "none"      # warm-up: 4 tokens
    first = c.decide(batch_size=10, seq_len=3072, expected_output_len=512)                      # inside the interval
    assert first.pipeline == "prefill"
    assert c.decide(batch_size=10, seq_len=3072, expected_output_len=512) is first              # cached now
    assert c.decide(batch_size=10, seq_len=64, expected_output_len=512).pipeline == "none"      # gate flips back
