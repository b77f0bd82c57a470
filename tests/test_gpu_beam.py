"""Beam-search surface on the GPU: `Attention.append_completion` (copy-on-write of the forked leaf +
single-row K/V writes), `duplicate`, `add_seq_async`, and the `ca_scatter_rows` entry point, against
the oracle on the same fp16-rounded values."""
import numpy as np
import pytest
import torch

from chunk_attn import Attention, cabi
from chunk_attn_oracle import Attention as OracleAttention
from gpu_helpers import CabiEngine, round_to

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def kv(g, n, H, d, scale=0.5):
    return torch.randn(n, H, d, generator=g) * scale, torch.randn(n, H, d, generator=g) * scale


def both(dtype, H, d, C):
    eng = Attention(n_heads=H, d_head=d, chunk_size=C, memory_mb=64, dtype=dtype, device=DEV)
    return eng, OracleAttention(H, d, C)


def compare(eng, ora, g, H, d, dtype, tol):
    n = len(ora.tails)
    assert len(eng.tails) == n
    q = torch.randn(n, H, d, generator=g)
    out = eng.forward(q=q.to(DEV, dtype)).float().cpu().numpy()
    want = ora.forward(round_to(q, dtype).numpy())
    assert np.isfinite(out).all()
    np.testing.assert_allclose(out, want, atol=tol, rtol=0)
    # the trees agree chunk for chunk
    assert [c.tokens for c in eng.tails] == [c.tokens for c in ora.tails]


@pytest.mark.parametrize("dtype,H,d,C,tol", [(torch.float16, 4, 128, 64, 1e-3), (torch.float32, 2, 64, 16, 1e-4),
                                             (torch.float16, 3, 32, 8, 1e-3)])
def test_beam_search_steps_match_oracle(dtype, H, d, C, tol):
    g = torch.Generator().manual_seed(7)
    eng, ora = both(dtype, H, d, C)
    shared = list(range(2 * C + 3))
    sk, sv = kv(g, len(shared), H, d)
    for s, extra in enumerate([5, C - 4, 0]):
        toks = shared + [1000 * (s + 1) + j for j in range(extra)]
        uk, uv = kv(g, extra, H, d)
        k, v = torch.cat([sk, uk]), torch.cat([sv, uv])
        i1 = eng.add_seq(tokens=toks, k=k.to(DEV, dtype), v=v.to(DEV, dtype))
        i2 = ora.add_seq(toks, round_to(k, dtype).numpy(), round_to(v, dtype).numpy())
        assert i1 == i2
    compare(eng, ora, g, H, d, dtype, tol)
    tok = 50000
    for step in range(2 * C // 3 + 6):  # long enough for every leaf to cross a chunk boundary
        n = len(ora.tails)
        if step % 3 == 2:
            # an ordinary decode step over all rows in between (the device-side token counters and the
            # forks have to compose)
            toks = [tok + i for i in range(n)]
            k, v = kv(g, n, H, d)
            eng.append_token(tokens=toks, k=k.to(DEV, dtype), v=v.to(DEV, dtype))
            ora.append_token(toks, round_to(k, dtype).numpy(), round_to(v, dtype).numpy())
            tok += n
        else:
            row = (step * 5) % n
            width = 1 + (step % 4 if n < 12 else 0)  # keep the batch bounded
            toks = [tok + i for i in range(width)]
            k, v = kv(g, width, H, d)
            assert eng.append_completion(seq_idx=row, tokens=toks, k=k.to(DEV, dtype), v=v.to(DEV, dtype)) == row
            ora.append_completion(row, toks, round_to(k, dtype).numpy(), round_to(v, dtype).numpy())
            tok += width
        if n >= 10:  # prune a beam, as a search does
            eng.remove_seq(n // 2)
            ora.remove_seq(n // 2)
        compare(eng, ora, g, H, d, dtype, tol)
    assert eng.device_status() == 0


def test_append_completion_rejects_bad_input_without_changing_anything():
    eng, _ = both(torch.float16, 4, 128, 64)
    g = torch.Generator().manual_seed(1)
    k, v = kv(g, 10, 4, 128)
    eng.add_seq(tokens=list(range(10)), k=k.to(DEV, torch.float16), v=v.to(DEV, torch.float16))
    k2, v2 = kv(g, 2, 4, 128)
    with pytest.raises(RuntimeError, match=r"\[n_tokens, n_heads, d_head\]"):
        eng.append_completion(seq_idx=0, tokens=[1, 2, 3], k=k2.to(DEV), v=v2.to(DEV))
    with pytest.raises(RuntimeError, match="out of range"):
        eng.append_completion(seq_idx=4, tokens=[1, 2], k=k2.to(DEV), v=v2.to(DEV))
    assert len(eng.tails) == 1 and eng.tails[0].tokens == list(range(10))


def test_scatter_rows_entry_point():
    H, d, C = 4, 128, 64
    eng = CabiEngine(H, d, C, torch.float16, max_chunks=8)
    g = torch.Generator().manual_seed(2)
    k, v = kv(g, 5, H, d)
    kd, vd = k.to(DEV, torch.float16), v.to(DEV, torch.float16)
    eng.ctx.scatter_rows(kd, vd, [3, 3, 5, 0, 7], [0, 63, 17, 1, 2])
    for tok, (cid, row) in enumerate([(3, 0), (3, 63), (5, 17), (0, 1), (7, 2)]):
        ko = torch.empty(H, row + 1, d, dtype=torch.float16, device=DEV)
        vo = torch.empty_like(ko)
        eng.ctx.read_chunk(cid, row + 1, ko, vo)
        assert torch.equal(ko[:, row], kd[tok]) and torch.equal(vo[:, row], vd[tok])
    # a strided source (every second head of a wider tensor)
    wide = torch.randn(2, 2 * H, d, generator=g).to(DEV, torch.float16)
    eng.ctx.scatter_rows(wide[:, ::2], wide[:, ::2], [1, 2], [4, 5])
    ko = torch.empty(H, 5, d, dtype=torch.float16, device=DEV)
    eng.ctx.read_chunk(1, 5, ko, torch.empty_like(ko))
    assert torch.equal(ko[:, 4], wide[0, ::2])
    with pytest.raises(cabi.CAError, match="row outside the chunk"):
        eng.ctx.scatter_rows(kd[:1], vd[:1], [0], [64])
    with pytest.raises(cabi.CAError, match="chunk id outside the pool"):
        eng.ctx.scatter_rows(kd[:1], vd[:1], [8], [0])


def test_add_seq_async_resolves_in_order_and_matches_add_seq():
    H, d, C, dtype = 4, 128, 64, torch.float16
    g = torch.Generator().manual_seed(3)
    a, _ = both(dtype, H, d, C)
    b, _ = both(dtype, H, d, C)
    shared = list(range(100))
    sk, sv = kv(g, 100, H, d)
    futures, want = [], []
    for s in range(6):
        toks = shared + [1000 * (s + 1) + j for j in range(10 + s)] if s % 2 == 0 else [7000 + 100 * s + j for j in range(30)]
        n_own = len(toks) - (100 if s % 2 == 0 else 0)
        uk, uv = kv(g, n_own, H, d)
        k = torch.cat([sk, uk]) if s % 2 == 0 else uk
        v = torch.cat([sv, uv]) if s % 2 == 0 else uv
        kd, vd = k.to(DEV, dtype), v.to(DEV, dtype)
        futures.append(a.add_seq_async(tokens=toks, k=kd, v=vd))
        del kd, vd  # the worker holds its own references
        want.append(b.add_seq(tokens=toks, k=k.to(DEV, dtype), v=v.to(DEV, dtype)))
    assert [f.get() for f in futures] == want
    q = torch.randn(6, H, d, generator=g).to(DEV, dtype)
    assert torch.equal(a.forward(q=q), b.forward(q=q))
    # a failing insertion surfaces at get(), and the worker keeps going
    bad = a.add_seq_async(tokens=[1, 2, 3], k=torch.zeros(2, H, d, device=DEV, dtype=dtype),
                          v=torch.zeros(2, H, d, device=DEV, dtype=dtype))
    with pytest.raises(RuntimeError, match="one K/V row per token"):
        bad.get()
    ok = a.add_seq_async(tokens=[5], k=torch.zeros(1, H, d, device=DEV, dtype=dtype),
                         v=torch.zeros(1, H, d, device=DEV, dtype=dtype))
    assert ok.get() == b.add_seq(tokens=[5], k=torch.zeros(1, H, d, device=DEV, dtype=dtype),
                                 v=torch.zeros(1, H, d, device=DEV, dtype=dtype))
