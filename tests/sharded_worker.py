"""Worker of tests/test_sharded_cpu.py: one rank of a gloo process group.  Each rank owns a head slice
through HeadShardedAttention (backed by the CPU oracle here, by the CUDA engine in production),
replays the same add / append / remove trace, and checks the all-gathered output against the
full-width oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "chunk-attention_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)

from chunk_attn.sharded import HeadShardedAttention  # noqa: E402
from chunk_attn_oracle import Attention as OracleAttention  # noqa: E402


class OracleBackedLocal:
    """The local-engine surface HeadShardedAttention needs, served by the numpy oracle."""

    def __init__(self, n_heads, d_head, chunk_size, **_):
        self.o = OracleAttention(n_heads, d_head, chunk_size)

    def add_seq(self, tokens, k, v):
        return self.o.add_seq(tokens, k.numpy(), v.numpy())

    def append_token(self, tokens, k, v, fused=True):
        self.o.append_token(tokens, k.numpy(), v.numpy())
        return []

    def remove_seq(self, i):
        self.o.remove_seq(i)

    def reserve(self):
        return self.o.reserve()

    def refresh_kernel_context(self, force=False):
        pass

    def forward(self, q, partition=0):
        return torch.from_numpy(self.o.forward(q.numpy(), partition))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    H, d, C = 8, 16, 4
    g = torch.Generator().manual_seed(1234)  # same stream on every rank: identical full-width inputs
    sharded = HeadShardedAttention(H, d, C, attention_factory=OracleBackedLocal)
    full = OracleAttention(H, d, C)
    assert sharded.h_local == H // world and sharded.head_slice == slice(rank * H // world, (rank + 1) * H // world)
    shared_k, shared_v = torch.randn(10, H, d, generator=g), torch.randn(10, H, d, generator=g)
    rows = []
    for s in range(5):
        n_u = 3 + s
        k = torch.cat([shared_k, torch.randn(n_u, H, d, generator=g)])
        v = torch.cat([shared_v, torch.randn(n_u, H, d, generator=g)])
        toks = list(range(10)) + [1000 * (s + 1) + j for j in range(n_u)]
        i1 = sharded.add_seq(toks, k, v)            # full-width tensors: sliced inside
        i2 = full.add_seq(toks, k.numpy(), v.numpy())
        assert i1 == i2
        rows.insert(i1, s)
    for step in range(3):
        n = len(rows)
        q, nk, nv = (torch.randn(n, H, d, generator=g) for _ in range(3))
        sharded.append_token([50 + step] * n, nk, nv)
        full.append_token([50 + step] * n, nk.numpy(), nv.numpy())
        out = sharded.forward(q)                    # all-gather over gloo
        assert out.shape == (n, H, d)
        ref = full.forward(q.numpy(), 0)
        assert np.abs(out.numpy() - ref).max() < 1e-5, "rank %d step %d" % (rank, step)
        # already-sliced inputs are accepted too
        out2 = sharded.forward(q[:, sharded.head_slice].contiguous())
        assert np.abs(out2.numpy() - ref).max() < 1e-5
        local = sharded.forward(q, gather=False)
        assert local.shape == (n, H // world, d)
        if step == 1:
            sharded.remove_seq(2)
            full.remove_seq(2)
            rows.pop(2)
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
