"""Worker of tests/test_symm_fd_exchange.py: gloo ranks that pass file descriptors around the way the
symmetric-memory rendezvous does (each rank's descriptor to every rank; rank 0's descriptor to the others)."""
import json
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fastcache_b200.parallel import symm_native  # noqa: E402


def main():
    out = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # an anonymous file whose content names its owner
    fd = os.memfd_create(f"rank{rank}")
    os.write(fd, f"owner {rank}".encode())
    fds = symm_native._exchange_fds(fd, rank, world, dist.group.WORLD)
    seen = []
    for r_, f in enumerate(fds):
        seen.append(os.pread(f, 64, 0).decode())
        if r_ != rank:
            os.close(f)
    got = symm_native._exchange_fds_from_root(fd, rank, world, dist.group.WORLD)
    root = os.pread(got, 64, 0).decode() if got >= 0 else None
    everyone = [None] * world
    dist.all_gather_object(everyone, {"rank": rank, "seen": seen, "root": root, "own_fd_kept": fds[rank] == fd})
    if rank == 0:
        with open(out, "w") as fh:
            json.dump(everyone, fh)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
