"""Serving harness pieces on the CPU engine."""
import time

import torch

from fastcache_b200 import LLM
from fastcache_b200.serving.harness import (ConcurrentTester, DynamicScheduler, KVCachePool, PerformanceMonitor,
                                            Request, RequestStatus, TimestampManager)
from helpers import tiny_llama_config


def test_dynamic_scheduler_prefill_priority_and_decode_budget():
    s = DynamicScheduler(max_batch_size=3, std_batch_threshold_decoding=10, max_wait_time=0.05)
    for i, n in enumerate([50, 10, 30]):
        s.add_prefill(f"p{i}", n)
    kind, batch = s.select_batch()
    assert kind == "prefill" and batch[0] == "p1" and len(batch) == 3      # shortest first, full batch
    s.add_prefill("late", 5)
    for i, n in enumerate([4, 4, 4, 4]):
        s.add_decoding(f"d{i}", n)
    kind, batch = s.select_batch()                                          # prefill not full, not waited long
    assert kind == "decoding" and len(batch) == 2                           # 4 + 4 <= 10 < 12
    time.sleep(0.06)
    kind, batch = s.select_batch()
    assert kind == "prefill" and batch == ["late"]                          # waited max_wait_time


def test_kv_pool_and_timestamps():
    pool = KVCachePool()
    kv = [(torch.randn(2, 2, 6, 4), torch.randn(2, 2, 6, 4))]
    pool.store_kvcache([7, 8], kv, lengths=[6, 4])
    assert pool.get(8)[0][0].shape == (1, 2, 4, 4) and pool.get_stats()["entries"] == 2
    merged, lens = pool.merge_and_pop([7, 8])
    assert merged[0][0].shape == (2, 2, 6, 4) and lens == [6, 4] and pool.get_stats()["entries"] == 0
    assert torch.equal(merged[0][0][1, :, 2:], kv[0][0][1, :, 2:])
    t = TimestampManager()
    for i, st in enumerate(["arrival", "prefill_queueing_start", "prefill_start", "prefill_finish",
                            "decoding_start", "decoding_finish"]):
        t.record(1, st, float(i))
    a = t.analyze(1, generated_len=4)
    assert a["ttft"] == 2.0 and a["tpot"] == 0.25 and a["latency"] == 5.0
    p = PerformanceMonitor.percentiles([1.0, 2.0, 3.0, 4.0, 100.0])
    assert p["p50"] == 3.0 and p["max"] == 100.0
    r = Request(0, [1, 2, 3])
    r.fail("boom")
    assert r.status is RequestStatus.FAILED and r.input_len == 3


def test_concurrent_tester_poisson_arrivals_with_compression():
    llm = LLM(tiny_llama_config(), device="cpu", kvcache_block_size=16, num_kvcache_blocks=256, max_model_len=256,
              enforce_eager=True, enable_compression=True, compression_backend="kvpress", kvpress_method="knorm",
              compression_factor=2, compression_pipeline="prefill")
    tester = ConcurrentTester(llm, batching=[3, 9, 18], req_per_sec=200.0, seed=1)
    assert ConcurrentTester.ccm_intensity_rule(135) == [15, 45, 135]
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 1000, (40,), generator=g).tolist() for _ in range(12)]
    res = tester.run(prompts, max_tokens=6)
    assert res.completed == 12 and res.output_tokens == 72 and res.failed == 0
    assert res.ttft["p50"] > 0 and res.latency["p99"] >= res.ttft["p99"]
    assert res.compression["compressions"] == 12 and res.compression["blocks_freed"] > 0
    assert llm.stats.prefill_steps >= 4                     # prefill cap 3 -> at least 4 prefill batches


def test_testcon_cli_single_run_and_yaml(tmp_path):
    """The harness command line on a CPU: one merge-compressor run (MiniCPM batching rule), then a YAML batch."""
    from fastcache_b200.serving import testcon
    common = ["--device", "cpu", "--num_samples", "4", "--max_new_tokens", "4", "--req_per_sec", "500",
              "--block_size", "16", "--kv_blocks", "256", "--max_model_len", "512"]
    out = tmp_path / "single"
    rows = testcon.main(["--model_mode", "minicpm", "--arch", "tiny-minicpm", "--use_compression", "--comp_mode",
                         "ccm", "--folder_path", str(out), "--gpu_info_path", str(tmp_path / "gpu.csv")] + common)
    assert rows[0]["batching"] == [15, 45, 135] and rows[0]["result"]["completed"] == 4
    assert rows[0]["result"]["compression"]["compressions"] == 4
    av = rows[0]["stage_averages"]
    assert 0 <= av["ttft"] <= av["latency"] and av["generated_lens"] == 4.0
    assert (tmp_path / "gpu.csv").exists() and (out / "summary.json").exists()
    assert "throughput_tok_s" in open(rows[0]["log"]).read()

    cfg = tmp_path / "experiments.yaml"
    cfg.write_text("global_settings:\n  num_samples: 3\n  req_per_sec: 500\n  max_new_tokens: 3\n"
                   "experiments:\n"
                   "  - {name: base, use_compression: false, comp_mode: orig, batching: [5, 5, 5]}\n"
                   "  - {name: knorm, use_compression: true, comp_mode: Knorm, batching: [5, 5, 5]}\n"
                   "  - {name: broken, use_compression: true, comp_mode: nonsense, batching: [5, 5, 5]}\n")
    rows = testcon.main(["--config", str(cfg), "--model_mode", "llava", "--arch", "tiny-llava", "--no_log"] + common)
    assert [r["name"] for r in rows] == ["base", "knorm", "broken"]
    assert rows[0]["result"]["completed"] == 3 and rows[0]["batching"] == [5, 5, 5]
    assert rows[1]["result"]["compression"]["compressions"] == 3 and "error" in rows[2]


def test_monitor_accumulates_batches_and_reports(tmp_path, capsys):
    from types import SimpleNamespace as NS
    import fastcache_b200.serving.harness as h
    m = h.PerformanceMonitor()
    m.add_result(NS(method="comp", latency=(1.0, 0.2, 0.01), throughput=100.0, memory_usage=5.0, request_id=[1, 2],
                    request_size=2, valid_tokens=64, success=True, compression_ratio=4.0, compression_time=0.01))
    m.add_result(NS(method="comp", latency=(1.5, 0.4, 0.02), throughput=120.0, memory_usage=6.0, request_id=[3],
                    request_size=1, valid_tokens=32, success=False))
    assert m.proc_latencies() == ([0.2, 0.2, 0.4], [0.01, 0.01, 0.02])
    met = m.calculate_metrics(system_completion_times=2.0)
    row = met["comp"]
    assert "orig" not in met and row["total_requests"] == 2 and row["success_rate"] == 50.0
    assert row["median_ttft"] == 0.2 and row["p99_ttft"] == 0.4 and abs(row["avg_throughput"] - 48.0) < 0.01
    assert row["avg_compression_ratio"] == 4.0 and row["throughput_stddev"] > 0
    h.print_metrics(met)
    assert "p90 0.4000" in capsys.readouterr().out
    path = h.generate_results_txt(met, {"ttft": 0.2}, 2.0, 96, "ccm", str(tmp_path / "r.txt"))
    assert "throughput: 48.00 tokens/s" in open(path).read()
    m.reset()
    assert m.calculate_metrics(system_completion_times=1.0) == {}
