"""Host-side multi-rank logic on CPU: batch sharding and the reductions the benchmark uses, run as two
gloo ranks."""
import os
import socket
import subprocess
import sys

import pytest

from blackforge_b200.launch import shard_range

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_partitions_exactly():
    for total in (0, 1, 5, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            covered = [i for s, c in spans for i in range(s, s + c)]
            assert covered == list(range(total))
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["BFB_ROOT"])
from blackforge_b200 import launch
rank, world = launch.init_process_group("gloo")
assert world == 2
start, count = launch.shard_range(5, rank, world)
total = launch.sum_over_ranks(count)
slowest = launch.max_over_ranks(10.0 + rank)
ident = launch.broadcast_bytes(bytes(range(128)) if rank == 0 else b"", 128)
launch.barrier()
assert total == 5.0 and slowest == 11.0 and ident == bytes(range(128)), (total, slowest)
print("rank", rank, "ok", start, count)
"""


def test_two_gloo_ranks_reduce_and_broadcast(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), BFB_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "rank 0 ok 0 3" in outs[0] and "rank 1 ok 3 2" in outs[1]
