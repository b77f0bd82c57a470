"""Randomised multi-level prefix trees at sizes the numpy oracle is too slow for: the tensor-core / TMA path
against (a) a dense fp32 attention over each row's full K/V history computed with torch on the GPU and (b) the
independent any-geometry kernel (partition=2), through add / remove / append / fork operations."""
import random

import pytest
import torch

from chunk_attn import Attention, cabi

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
TOL = 1e-3


class Mirror:
    """Row-ordered list of (tokens, k, v) histories kept next to the engine."""

    def __init__(self, H, seed, memory_mb=1024, wide=None, finish=None):
        self.H, self.d = H, 128
        self.attn = Attention(n_heads=H, d_head=128, chunk_size=64, memory_mb=memory_mb, dtype=torch.float16, device=DEV)
        if wide is not None:   # 2: every shared run on the tcgen05 kernel, 0: none (default: the planner decides)
            self.attn.set_option(cabi.CA_OPT_WIDE_RUNS, wide)
        if finish is not None:  # 0: the short-tails kernel writes partial rows and the merge kernel always runs
            self.attn.set_option(cabi.CA_OPT_FINISH_IN_TAILS, finish)
        self.g = torch.Generator(device=DEV).manual_seed(seed)
        self.rows = []
        self.next_token = 1

    def rand(self, n):
        return (torch.randn(n, self.H, self.d, generator=self.g, device=DEV) * 0.5).half()

    def fresh_tokens(self, n):
        t = list(range(self.next_token, self.next_token + n))
        self.next_token += n
        return t

    def add(self, src_row, cut, n_new):
        """New sequence = first `cut` tokens of row src_row (None: nothing) + n_new fresh tokens."""
        if src_row is None:
            toks, k, v = [], self.rand(0), self.rand(0)
        else:
            st, sk, sv = self.rows[src_row]
            toks, k, v = st[:cut], sk[:cut], sv[:cut]
        toks = toks + self.fresh_tokens(n_new)
        k, v = torch.cat([k, self.rand(n_new)]), torch.cat([v, self.rand(n_new)])
        idx = self.attn.add_seq(tokens=toks, k=k, v=v)
        self.rows.insert(idx, (toks, k, v))
        return idx

    def remove(self, row):
        self.attn.remove_seq(row)
        self.rows.pop(row)

    def append_all(self):
        n = len(self.rows)
        toks, k, v = self.fresh_tokens(n), self.rand(n), self.rand(n)
        self.attn.append_token(tokens=toks, k=k, v=v)
        self.rows = [(t + [toks[i]], torch.cat([rk, k[i:i + 1]]), torch.cat([rv, v[i:i + 1]]))
                     for i, (t, rk, rv) in enumerate(self.rows)]

    def fork(self, row, width):
        toks, k, v = self.fresh_tokens(width), self.rand(width), self.rand(width)
        self.attn.append_completion(seq_idx=row, tokens=toks, k=k, v=v)
        t, rk, rv = self.rows[row]
        self.rows[row:row + 1] = [(t + [toks[i]], torch.cat([rk, k[i:i + 1]]), torch.cat([rv, v[i:i + 1]]))
                                  for i in range(width)]

    def check(self):
        n = len(self.rows)
        assert len(self.attn.tails) == n
        q = self.rand(n)
        out = self.attn.forward(q=q)
        gen = self.attn.forward(q=q, partition=2)
        assert torch.isfinite(out).all()
        worst = 0.0
        for i, (_, k, v) in enumerate(self.rows):
            s = torch.einsum("hd,thd->ht", q[i].float(), k.float()) / self.d ** 0.5
            want = torch.einsum("ht,thd->hd", s.softmax(-1), v.float())
            worst = max(worst, (out[i].float() - want).abs().max().item(), (gen[i].float() - want).abs().max().item())
        assert worst < TOL, worst
        assert self.attn.device_status() == 0
        return worst


@pytest.mark.parametrize("wide", [None, 2, 0])
@pytest.mark.parametrize("H,seed", [(1, 0), (3, 1), (8, 2), (40, 3)])
def test_random_trees(H, seed, wide):
    rnd = random.Random(seed)
    m = Mirror(H, seed, memory_mb=1536 if H == 40 else 768, wide=wide)
    # a few unrelated roots, then sequences branching off existing ones at chunk-aligned and ragged cuts
    for _ in range(3):
        m.add(None, 0, rnd.choice([1, 63, 64, 65, 200, 512]))
    for step in range(70):
        r = rnd.random()
        n = len(m.rows)
        if r < 0.5 and n < 96:
            src = rnd.randrange(n)
            length = len(m.rows[src][0])
            cut = rnd.choice([length, (length // 64) * 64, rnd.randint(0, length), max(0, (length // 64 - 1) * 64)])
            m.add(src, cut, rnd.choice([1, 2, 17, 64, 130]))
        elif r < 0.62 and n > 2:
            m.remove(rnd.randrange(n))
        elif r < 0.72 and n < 90:
            m.fork(rnd.randrange(n), rnd.randint(1, 4))
        else:
            m.append_all()
        if step % 7 == 6:
            m.check()
    m.check()
    st = m.attn.plan_stats()
    assert st["fast_path"] == 1 and st["n_shared_chunks"] > 0


@pytest.mark.parametrize("wide", [0, 2])
def test_wide_batch_over_one_long_prefix(wide):
    """300 rows over one 1024-token prefix (row blocks of 64 in the chunk-first phase of the persistent kernel, of
    100 on the tcgen05 kernel), ragged suffixes, and a decode loop long enough for every tail to cross a chunk boundary."""
    m = Mirror(4, 9, memory_mb=1024, wide=wide)
    rnd = random.Random(9)
    m.add(None, 0, 1024 + 5)
    for _ in range(299):
        m.add(0, 1024, rnd.randint(1, 70))
    m.check()
    for step in range(66):
        m.append_all()
        if step % 22 == 21:
            m.check()
    assert m.attn.plan_stats()["n_shared_chunks"] == 16


def test_one_very_long_sequence_and_short_neighbours():
    """A 20 000-token row next to one-token rows: item lists of very different lengths."""
    m = Mirror(2, 11, memory_mb=512)
    m.add(None, 0, 20_000)
    for _ in range(5):
        m.add(None, 0, 1)
    m.add(0, 19_968, 3)
    m.check()
    for _ in range(3):
        m.append_all()
    m.check()


@pytest.mark.parametrize("finish", [1, 0])
def test_many_short_tails_take_the_warp_per_item_kernel(finish):
    """400 rows whose private part is a fraction of one chunk: their items go to the half-warp-per-item kernel
    (plan_stats n_items_short), through appended tokens without a rebuild and across the chunk boundary; with
    finish = 1 that kernel also combines the rows' partials and stores the output whenever every row has such a tail."""
    m = Mirror(4, 13, memory_mb=512, finish=finish)
    rnd = random.Random(13)
    m.add(None, 0, 256 + 3)
    for _ in range(399):
        m.add(0, 256, rnd.randint(1, 60))
    m.check()
    st = m.attn.plan_stats()
    assert st["n_items_short"] >= 390 * 4
    assert st["kernels_per_step"] == (2 if finish and st["n_items_short"] == 400 * 4 else 3)
    for step in range(70):  # every tail fills up and gets a successor on the way
        m.append_all()
        if step % 10 == 9:
            m.check()
    # rows without any shared prefix, all short: the persistent kernel has nothing to do
    m2 = Mirror(4, 14, memory_mb=512, finish=finish)
    for _ in range(320):
        m2.add(None, 0, rnd.randint(1, 64))
    m2.check()
    assert m2.attn.plan_stats()["n_items_short"] >= 300 * 4  # (a row of exactly 64 tokens has a full chunk + an empty tail)


@pytest.mark.parametrize("wide,finish", [(0, 0), (2, 0), (0, 1), (2, 1)])
def test_large_batch_of_short_lists_takes_the_eight_lane_merge(wide, finish):
    """600 rows over one 256-token prefix, a few private tokens each: 2400 (row, head) pairs of two to four pieces,
    the shape the eight-lanes-per-pair merge kernel serves; appended tokens and a removed row on the way."""
    m = Mirror(4, 21, memory_mb=1024, wide=wide, finish=finish)
    rnd = random.Random(21)
    m.add(None, 0, 256 + 2)
    for _ in range(599):
        m.add(0, 256, rnd.randint(1, 30))
    m.check()
    for step in range(3):
        m.append_all()
    m.remove(17)
    m.check()
