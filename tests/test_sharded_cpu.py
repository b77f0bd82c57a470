"""Head sharding + output all-gather on CPU: two gloo ranks, the CPU oracle as the local engine."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_head_sharding_and_gather_with_gloo(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "sharded_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count(" ok") == world


@pytest.mark.parametrize("mode", ["leave", "vanish"])
def test_rank_that_leaves_is_detected_on_the_host(mode):
    # failure detection without any device fault: one rank stops between steps; the others learn of it from the
    # key-value store before they launch the next step and raise PeerLost instead of hanging in the gather
    world = 3
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "sharded_failure_worker.py"), mode]
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("detected:") == world - 1 and "NOT detected" not in r.stdout
    assert ("a rank left" in r.stdout) if mode == "leave" else ("within" in r.stdout)


def test_uneven_head_split_is_rejected():
    sys.path.insert(0, os.path.join(ROOT, "chunk-attention_b200"))
    from chunk_attn.sharded import HeadShardedAttention

    class Fake:
        def __init__(self, **kw):
            self.kw = kw

    a = HeadShardedAttention(6, 8, 4, attention_factory=Fake)   # no process group: world size 1
    assert a.h_local == 6 and a.local.kw["n_heads"] == 6
