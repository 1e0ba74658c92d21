"""Descriptor exchange of the package's own symmetric-memory rendezvous (parallel/symm_native.py), on gloo ranks:
the part of the runtime that needs no GPU.  Every rank must end up with a descriptor of every rank's allocation
(here: an anonymous file that names its owner), and rank 0's multicast descriptor must reach every rank."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4])
def test_every_rank_receives_every_descriptor(tmp_path, world):
    out = str(tmp_path / "fds.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29680 + world), os.path.join(HERE, "symm_fd_worker.py"),
           out]
    r = subprocess.run(cmd, env=dict(os.environ, MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES=""),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert [e["rank"] for e in res] == list(range(world))
    for e in res:
        assert e["seen"] == [f"owner {r_}" for r_ in range(world)]
        assert e["root"] == "owner 0" and e["own_fd_kept"]
