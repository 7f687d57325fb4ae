"""CPU tests of the multi-process side of bench.py: two gloo ranks compute the shards they
would own of every benchmark configuration (strong split) and the per-rank maxima the
benchmark reports; plus the reference arm's line under a two-rank launch.  No GPU involved."""
import json
import os
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys
sys.path.insert(0, {root!r})
import torch.distributed as dist
import bench
xc = bench.load_package()
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
shards = {{k: bench.strong_shard(xc, k, world, rank) for k in bench.CONFIGS}}
# every rank contributes "its" time; the benchmark reports the slowest rank
times = bench.max_over_ranks([10.0 + rank, 5.0 - rank], dist)
gathered = [None] * world
dist.all_gather_object(gathered, shards)
dist.barrier()
if rank == 0:
    print(json.dumps({{"times": times, "shards": gathered}}))
dist.destroy_process_group()
'''


def run_ranks(script_text, world):
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "worker.py")
        with open(path, "w") as f:
            f.write(script_text)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", "29671", path]
        return subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)


def test_two_gloo_ranks_split_every_configuration_without_gaps(xc):
    r = run_ranks(WORKER.format(root=ROOT), 2)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    data = json.loads(line)
    assert data["times"] == [11.0, 5.0]                      # max over ranks, element-wise
    import bench
    for k, (mode, rows, cols, nl, nr) in bench.CONFIGS.items():
        parts = [s[k] for s in data["shards"]]
        if mode == "one_to_one":                             # replicas only: not split
            assert parts[0] == [0, 1, 1, 1] and parts[1] == [0, 0, 0, 0]
            continue
        units = nr if mode == "one_to_many" else nl
        covered = []
        for first, count, a_nl, a_nr in parts:
            covered.extend(range(first, first + count))
            if mode == "one_to_many":
                assert (a_nl, a_nr) == (1, count)
            elif mode == "n_to_m":
                assert (a_nl, a_nr) == (count, nr)
            else:
                assert (a_nl, a_nr) == (count, count * (nr // nl))
        assert covered == list(range(units))                  # contiguous, complete, no overlap
        assert abs(parts[0][1] - parts[1][1]) <= 1


def test_reference_arm_prints_one_line_from_rank_zero():
    """`bench.py --impl reference` under a two-rank launch: rank 0 alone times the reference's
    CPU code and prints the line; the other rank exits without work."""
    with tempfile.TemporaryDirectory() as tmp:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", "29672", os.path.join(ROOT, "bench.py"),
               "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", "--cpu-seconds", "1.5"]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=tmp)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "xcorr_gflops" and d["unit"] == "GFLOP/s"
    assert d["value"] > 0 and d["n_gpus"] == 2 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
