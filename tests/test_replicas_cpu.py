"""Multi-GPU means independent replicas (decode is single-request; the reference is one engine per GPU,
crates/tachyon/src/engine.rs:192): what the ranks share is a barrier and a max over their times.  Two gloo ranks on the CPU."""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_two_ranks_agree_on_the_slowest_replica():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29517",
           os.path.join(HERE, "ranks_helper.py")]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    got = json.loads(line)
    assert got["world"] == 2 and got["slowest"] == 11.0 and got["total"] == 300.0


def test_replicas_draw_disjoint_batches():
    sys.path.insert(0, os.path.dirname(HERE))
    import bench

    a, b = bench.encoder_batch(1000, 8, 5), bench.encoder_batch(1000, 8, 6)
    assert [len(q) for q in a] != [len(q) for q in b]
    assert all(16 <= len(q) <= 512 for q in a + b)
