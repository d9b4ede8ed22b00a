"""Row-shard planning and the gathered LM head on CPU ranks (gloo, world size 2 and 3)."""
import os
import socket
import subprocess
import sys

import pytest

from brotensor_b200 import shard, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("n,world,align", [(128256, 8, 16), (128256, 1, 16), (70, 3, 1), (33, 2, 16), (5, 8, 1), (0, 2, 1)])
def test_row_ranges_partition(n, world, align):
    rs = [shard.row_range(n, world, r, align) for r in range(world)]
    assert rs[0][0] == 0 and rs[-1][1] == n
    for (b0, e0), (b1, e1) in zip(rs, rs[1:]):
        assert e0 == b1 and b0 <= e0
    for b, e in rs[:-1]:
        assert b % align == 0 and (e % align == 0 or e == n)
    lens = [e - b for b, e in rs]
    assert max(lens) - min(lens) <= 2 * align - 1  # one unit of imbalance plus the ragged tail


def test_lm_head_config_shards_are_equal_byte_ranges():
    fmt, N, K = synth.Q6_K, 128256, 4096
    for world in (1, 2, 4, 8):
        spans = [shard.byte_range(fmt, N, K, world, r, 16) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == synth.packed_bytes(fmt, N, K)
        assert len({e - b for b, e in spans}) == 1
        assert all(e0 == b1 for (_, e0), (b1, _) in zip(spans, spans[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_head_matches_unsharded_on_gloo_ranks(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env, cwd=ROOT)
    assert r.returncode == 0 and "DIST_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
