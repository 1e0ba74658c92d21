"""The models x workloads x variants sweep on the CPU at tiny scale: rows, resume, error rows, trace input."""
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))

import matrix_bench as mb  # noqa: E402


def test_sweep_rows_resume_and_errors(tmp_path, monkeypatch):
    out = str(tmp_path / "m.json")
    base = ["--scale", "tiny", "--device", "cpu", "--models", "qwen3-8b", "--workloads", "light-dataset",
            "--batch-sizes", "2", "--output", out]
    rows = mb.main(base + ["--variants", "baseline,compression-only"])
    assert [r["variant"] for r in rows] == ["baseline", "compression-only"]
    assert all("error" not in r and r["throughput_tok_s"] > 0 and r["generated_tokens"] == 2 * 4 for r in rows)
    assert rows[0]["backend"] == "none" and rows[1]["backend"] == "kvpress" and rows[1]["compressions"] == 2
    assert rows[1]["speedup_vs_baseline"] > 0
    assert json.load(open(out)) == json.loads(json.dumps(rows))

    # resume: finished cells are kept and not run again; a failing cell is recorded and the sweep goes on
    calls, fail = [], [True]
    real = mb.run_cell

    def flaky(llm, reqs, batch, warmup_waves=1):
        calls.append(batch)
        if fail.pop() if fail else False:
            raise RuntimeError("injected")
        return real(llm, reqs, batch, warmup_waves)

    monkeypatch.setattr(mb, "run_cell", flaky)
    rows2 = mb.main(base + ["--resume", "--variants", "baseline,compression-only,auto-tune+greenctx,triad"])
    assert len(calls) == 2 and [r["variant"] for r in rows2] == ["baseline", "compression-only",
                                                                 "auto-tune+greenctx", "triad"]
    assert rows2[2]["error"] == "RuntimeError: injected" and "error" not in rows2[3]
    # a second resume retries only the failed cell
    calls.clear()
    rows3 = mb.main(base + ["--resume", "--variants", "baseline,compression-only,auto-tune+greenctx,triad"])
    assert len(calls) == 1 and all("error" not in r for r in rows3) and len(rows3) == 4


def test_trace_csv_filters(tmp_path):
    path = tmp_path / "trace.csv"
    path.write_text("TIMESTAMP,ContextTokens,GeneratedTokens\n0,100,10\n1,2000,300\n2,1500,900\n3,4000,100\n")
    assert mb.read_trace(str(path), 1024, 256, 512, 10) == [(2000, 300), (1500, 512)]
    spec = mb.WorkloadSpec("heavy-trace", "trace", 1, 64, trace_path=str(path), trace_min_context=1024,
                           trace_min_output=256, trace_max_output=512)
    reqs = mb.requests_for(spec, 3, 1000, 4096, seed=1)
    assert [len(p) for p, _ in reqs] == [2000, 1500, 2000] and all(n == 64 for _, n in reqs)


def test_cell_in_a_child_process(tmp_path):
    out = str(tmp_path / "iso.json")
    rows = mb.main(["--scale", "tiny", "--device", "cpu", "--models", "llava-mlp", "--workloads", "synthetic-long",
                    "--batch-sizes", "2", "--variants", "baseline,compression-only", "--isolate", "on",
                    "--output", out])
    assert [r.get("error") for r in rows] == [None, None]
    assert rows[1]["backend"] == "mlp" and rows[1]["compressions"] == 2 and rows[1]["speedup_vs_baseline"] > 0
    # a child that dies is an error row, not an exception
    rows = mb.main(["--scale", "tiny", "--device", "cpu", "--models", "llava-mlp", "--workloads", "synthetic-long",
                    "--batch-sizes", "2", "--variants", "baseline", "--isolate", "on", "--kv-blocks", "2",
                    "--output", str(tmp_path / "small.json")])
    assert "blocks" in rows[0]["error"]
