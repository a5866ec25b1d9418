"""CPU: the multi-GPU host logic with world_size 2 on gloo, and the in-library batch split."""
import ctypes as C
import json
import os
import subprocess
import sys

from conftest import ROOT
import fastface_b200 as ff


def test_bench_rank_protocol_world2_gloo():
    """bench.py under torchrun with 2 ranks (gloo, no GPU): rank 0 prints one JSON line whose
    time is the max over ranks and whose value is the aggregate over both ranks."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29617", os.path.join(ROOT, "bench.py"),
           "--gpus", "2", "--steps", "4", "--warmup", "1", "--batch", "64", "--dry-run"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    d = json.loads(lines[0])
    assert d["n_gpus"] == 2 and d["steps"] == 4
    assert abs(d["ms_per_step"] - 20.0 / 4) < 1e-9                 # slowest rank: 10 * (1 + 1) ms
    assert abs(d["value"] - 2 * 4 * 64 / 0.020) < 1e-6             # both ranks' faces / max time


def test_reference_arm_other_ranks_exit_quietly():
    """--impl reference under torchrun: only rank 0 works and prints; rank 1 exits 0 silently."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_shard_plan(built_lib):
    lib = ff.load_library()
    lib.fastface_shard_plan.restype = C.c_int
    lib.fastface_shard_plan.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    starts, counts = (C.c_int * 16)(), (C.c_int * 16)()
    for n, nd in [(65536, 8), (65536, 2), (10, 4), (3, 8), (1, 1), (1025, 2)]:
        used = lib.fastface_shard_plan(n, nd, starts, counts)
        assert 1 <= used <= nd
        assert starts[0] == 0 and sum(counts[:used]) == n
        for d in range(1, used):
            assert starts[d] == starts[d - 1] + counts[d - 1]          # contiguous, in order
        assert max(counts[:used]) - min(counts[:used - 1] or [counts[0]]) <= max(counts[:used])
        assert max(counts[:used]) == -(-n // nd)
    assert lib.fastface_shard_plan(0, 4, starts, counts) == 0
