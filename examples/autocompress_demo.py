"""What the planning package decides, printed for a few workloads.  Runs on a CPU.

    python examples/autocompress_demo.py [GPU name, default B200]

(Reference counterpart: demo_autocompress.py.)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fastcache_b200.autocompress import (AutoCompressManager, AutoCompressScheduler, CompressionConfig,  # noqa: E402
                                         CostModel, WorkloadContext, analyze_all_methods, get_hardware_profile,
                                         get_method, get_profile, list_methods, list_profiles)


def header(title: str) -> None:
    print(f"\n{'=' * 78}\n{title}\n{'=' * 78}")


def main() -> None:
    hw = get_hardware_profile(sys.argv[1] if len(sys.argv) > 1 else "B200")
    header(f"hardware: {hw.gpu_name}")
    print(f"memory bandwidth {hw.memory_bandwidth_gbps:.0f} GB/s, bf16 {hw.fp16_tflops:.0f} TFLOP/s, "
          f"roofline knee {hw.roofline_intensity:.0f} FLOP/B, {hw.sm_count} SMs")

    header("methods")
    print("profiles:", ", ".join(list_profiles()))
    print("constructible:", ", ".join(list_methods()))
    for name in list_profiles():
        p = get_profile(name)
        print(f"  {name:14s} {p.compute_type.name:7s} ratio {p.compression_ratio:4.1f}  "
              f"decode compatibility {p.decode_compatibility:.2f}  needs attention: {p.requires_attention}")

    cost, sched = CostModel(hw), AutoCompressScheduler(hw)
    workloads = [("short chat", WorkloadContext(batch_size=8, seq_len=256, expected_output_len=64)),
                 ("image + question", WorkloadContext(batch_size=45, seq_len=640, expected_output_len=128,
                                                      num_layers=32, num_kv_heads=32)),
                 ("long prompts", WorkloadContext(batch_size=128, seq_len=4096, expected_output_len=512,
                                                  num_layers=36, num_kv_heads=8)),
                 ("32k prompts", WorkloadContext(batch_size=32, seq_len=32768, expected_output_len=256,
                                                 num_layers=64, num_kv_heads=8, hidden_size=5120))]
    for label, w in workloads:
        header(f"{label}: batch {w.batch_size}, {w.seq_len} prompt rows, {w.expected_output_len} output tokens")
        print(f"decode step {cost.decode_latency_ms(w):.3f} ms "
              f"({'memory' if hw.is_decode_memory_bound(w.batch_size, w.seq_len, w.num_layers, w.num_kv_heads, w.head_dim, w.hidden_size) else 'compute'}-bound)")
        for method in ("mlp", "snapkv", "streaming_llm", "int8_quant"):
            a = sched.analyze(method, w)
            plan = sched.schedule(method, w)
            timing = get_method(method if method != "mlp" else "mlp").get_optimal_timing(w, hw).name
            print(f"  {method:14s} compress {a['compress_ms']:8.3f} ms  speed-up x{plan.estimated_speedup:5.2f}  "
                  f"break-even {cost.get_break_even_output_len(method, w):>6} tokens  "
                  f"{'compress' if plan.should_compress else 'skip    '}  {plan.timing.name:14s} (method rule: {timing})")
        best = sched.schedule_multi(["mlp", "snapkv", "streaming_llm"], w)
        print(f"  best of three: {best.method} ({best.reason or 'highest predicted speed-up'})")
        strategies = {m: c.strategy.name for m, c in analyze_all_methods(w, hw).items()}
        print("  pipeline strategies:", ", ".join(f"{m}={s}" for m, s in strategies.items()))

    header("manager")
    mgr = AutoCompressManager(CompressionConfig(method="mlp", compression_ratio=4.0), hardware=hw)
    plan = mgr.get_plan(batch_size=90, seq_len=640, expected_output_len=128, num_layers=32, num_kv_heads=32)
    print(plan.summary())
    print("should compress 4 x 128 -> 16:", mgr.should_compress(4, 128, 16))
    print(mgr.get_statistics())


if __name__ == "__main__":
    main()
