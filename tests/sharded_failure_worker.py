"""Worker of tests/test_sharded_cpu.py::test_rank_that_leaves_is_detected_on_the_host: gloo ranks, the numpy
oracle as the local engine.  All ranks run two steps; then the last rank stops taking part — politely
(`leave()`, mode "leave") or by simply exiting between steps (mode "vanish") — and the others must get PeerLost
from the host-side check of their next forward() instead of hanging in the all-gather."""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "chunk-attention_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)

from chunk_attn.sharded import HeadShardedAttention, PeerLost  # noqa: E402
from sharded_worker import OracleBackedLocal  # noqa: E402


def main():
    mode = sys.argv[1]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    H, d, C = 6, 8, 4
    g = torch.Generator().manual_seed(99)
    sharded = HeadShardedAttention(H, d, C, attention_factory=OracleBackedLocal)
    sharded.enable_peer_check(timeout_s=3.0)
    for s in range(3):
        n = 5 + s
        sharded.add_seq([100 * s + j for j in range(n)], torch.randn(n, H, d, generator=g), torch.randn(n, H, d, generator=g))
    q = torch.randn(3, H, d, generator=g)
    for step in range(2):
        assert sharded.forward(q).shape == (3, H, d)
    if rank == world - 1:
        if mode == "leave":
            sharded.leave()
        print("rank %d gone" % rank, flush=True)
        os._exit(0)   # between steps, nothing of this rank in flight
    t0 = time.monotonic()
    try:
        sharded.forward(q)
    except PeerLost as exc:
        dt = time.monotonic() - t0
        assert dt < (1.0 if mode == "leave" else 6.0), dt
        print("rank %d detected: %s" % (rank, exc), flush=True)
        os._exit(0)   # no collective with the missing rank is attempted, not even a clean shutdown
    print("rank %d NOT detected" % rank, flush=True)
    os._exit(3)


if __name__ == "__main__":
    main()
