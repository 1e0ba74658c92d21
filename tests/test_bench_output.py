"""bench.py keeps standard output for its one JSON line (libraries that write to descriptor 1 go to stderr)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_only_the_result_line_reaches_stdout():
    code = ("import os, sys; sys.path.insert(0, %r); import bench; bench.claim_stdout(); "
            "os.write(1, b'NCCL version x.y\\n'); print('a python print'); bench.emit({'metric': 'm', 'value': 1})" % ROOT)
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, timeout=120)
    assert p.returncode == 0, p.stderr
    assert json.loads(p.stdout) == {"metric": "m", "value": 1} and p.stdout.count("\n") == 1
    assert "NCCL version" in p.stderr and "a python print" in p.stderr


def test_reference_arm_reports_unavailable_for_tensor_parallel_runs():
    env = dict(os.environ, WORLD_SIZE="2", RANK="0", LOCAL_RANK="0")
    p = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--gpus", "2"], capture_output=True,
                       text=True, cwd=ROOT, env=env, timeout=300)
    assert p.returncode == 0
    line = json.loads(p.stdout)
    assert line["impl"] == "reference" and "unavailable" in line


def test_check_mode_comparison_rule():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.compare_first_tokens([5, 6, 7, 8], [5, 6, 7, 8]) == (4, 4)
    assert bench.compare_first_tokens([5, 6, 7, 8], [5, 0, 7, 0]) == (2, 4)
    assert bench.compare_first_tokens([5, 6], [5, 6, 7]) == (2, 3)          # a missing request counts as a miss
