"""The CPU oracle against its pins: the golden vectors produced by the unmodified reference
(tests/golden), the reference build itself where present, and dense fp64 attention."""
import os

import numpy as np
import pytest

from chunk_attn_oracle import Attention as OracleAttention, dense_forward
from golden_replay import fixtures, replay
from ref_loader import load_reference
from tree_traces import kv_for, tails_shape


@pytest.mark.parametrize("path", fixtures(), ids=lambda p: os.path.basename(p)[:-4])
def test_oracle_reproduces_reference_golden_vectors(path):
    worst = replay(path, lambda H, d, C: OracleAttention(H, d, C), tol=2e-6,
                   tree_of=lambda e: e.shape(), tails_of=lambda e: tails_shape(e.tails))
    assert worst < 2e-6


def test_golden_set_is_complete():
    names = {os.path.basename(p)[:-4] for p in fixtures()}
    assert {"ref_forward_case", "ref_add_seq_case", "cfg1_scaled", "two_level_churn", "random_trace_0"} <= names


@pytest.mark.parametrize("C", [2, 5, 16])
def test_oracle_vs_dense_and_partitions_agree(C):
    rng = np.random.default_rng(C)
    H, d = 3, 8
    ora = OracleAttention(H, d, C)
    shared = list(range(3 * C))
    sk, sv = kv_for(len(shared), H, d, rng)
    for s in range(5):
        n_u = C + s
        uk, uv = kv_for(n_u, H, d, rng)
        ora.add_seq(shared + [1000 * (s + 1) + j for j in range(n_u)], np.concatenate([sk, uk]), np.concatenate([sv, uv]))
    q = rng.standard_normal((5, H, d)).astype(np.float32)
    dense = dense_forward(ora, q)
    for part in (0, 1, 2):
        assert np.abs(ora.forward(q, part) - dense).max() < 1e-5
    with pytest.raises(RuntimeError):
        ora.forward(q, 3)


def test_oracle_vs_reference_build_live():
    ref = load_reference("cpu")
    if ref is None:
        pytest.skip("oracle/_ref is not built here")
    import torch
    H, d, C = 8, 64, 32
    g = torch.Generator().manual_seed(0)
    ra = ref.Attention(n_heads=H, d_head=d, chunk_size=C, memory_mb=64, dtype=torch.float32, device=torch.device("cpu"))
    ora = OracleAttention(H, d, C)
    sk, sv = torch.randn(256, H, d, generator=g), torch.randn(256, H, d, generator=g)
    for s in range(4):
        uk, uv = torch.randn(32, H, d, generator=g), torch.randn(32, H, d, generator=g)
        toks = list(range(256)) + [1_000_000 * (s + 1) + j for j in range(32)]
        k, v = torch.cat([sk, uk]), torch.cat([sv, uv])
        assert ra.add_seq(tokens=toks, k=k, v=v) == ora.add_seq(toks, k.numpy(), v.numpy())
    q = torch.randn(4, H, d, generator=g)
    for part in (0, 2):
        assert np.abs(ra.forward(q, part).numpy() - ora.forward(q.numpy(), part)).max() < 1e-6
