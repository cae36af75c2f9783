"""Run by tests/test_multiproc_cpu.py under torchrun (CPU ranks): the benchmark's child-process section in its
plumbing-only mode.  Rank 0 writes what the children reported."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402

if __name__ == "__main__":
    rank = int(os.environ["RANK"])
    res = bench._run_fused_children(rank, 2, 1, dry_run=True, limit_s=120)
    if rank == 0:
        with open(sys.argv[1], "w") as f:
            json.dump(res, f)
