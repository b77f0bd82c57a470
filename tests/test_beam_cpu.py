"""Beam-search surface on the host: PrefixTree.append_completion (tree shape, row order, capacity
check before mutation) and the oracle's restatement of it against dense attention."""
import numpy as np
import pytest

from chunk_attn import PrefixTree, cabi
from chunk_attn_oracle import Attention as OracleAttention, dense_attention


def rows_of(t):
    return {cid: (b, e) for cid, _, b, e in t.get_chunks()}


def test_fork_keeps_row_and_inserts_clones_after_it():
    t = PrefixTree(chunk_size=4, max_chunks=64)
    t.add_seq([1, 2, 3, 4, 5])      # row 0: [1234] -> [5]
    t.add_seq([1, 2, 3, 4, 6, 7])   # row 1: [1234] -> [6 7]
    t.add_seq([9])                  # row 2
    pairs, slots = t.append_completion(1, [70, 71, 72])
    assert len(pairs) == 2 and all(src == t.tails[1].id for src, _ in pairs)
    assert [dst for _, dst in pairs] == [t.tails[2].id, t.tails[3].id]
    assert [x.tokens for x in t.tails] == [[5], [6, 7, 70], [6, 7, 71], [6, 7, 72], [9]]
    assert slots == [(t.tails[1].id, 2), (t.tails[2].id, 2), (t.tails[3].id, 2)]
    assert t.get_trie().children[0].n_seqs == 4 and t.get_trie().n_seqs == 5
    r = rows_of(t)
    for i, tail in enumerate(t.tails):
        assert r[tail.id] == (i, i + 1)


def test_single_token_is_a_plain_append_to_one_row():
    t = PrefixTree(chunk_size=4, max_chunks=64)
    t.add_seq([1, 2])
    t.add_seq([3])
    pairs, slots = t.append_completion(0, [5])
    assert pairs == [] and slots == [(t.tails[0].id, 2)]
    assert [x.tokens for x in t.tails] == [[1, 2, 5], [3]]


def test_leaves_that_fill_up_get_successors():
    t = PrefixTree(chunk_size=4, max_chunks=64)
    t.add_seq([1, 2, 3])
    pairs, slots = t.append_completion(0, [4, 5])
    assert [x.tokens for x in t.tails] == [[], []]                       # fresh empty tails
    assert [x.tokens for x in t.get_trie().children] == [[1, 2, 3, 4], [1, 2, 3, 5]]
    assert all(len(c.children) == 1 for c in t.get_trie().children)
    # the K/V rows go to the (now full) forked leaves, not to the new tails
    assert slots == [(t.get_trie().children[0].id, 3), (t.get_trie().children[1].id, 3)]
    # forking an empty reserved tail works as well
    pairs, slots = t.append_completion(1, [8, 9])
    assert [x.tokens for x in t.tails] == [[], [8], [9]]
    assert t.get_trie().children[1].n_seqs == 2


def test_capacity_is_checked_before_anything_changes():
    t = PrefixTree(chunk_size=2, max_chunks=4)
    t.add_seq([1, 2, 3])            # [1 2] -> [3]: 2 chunks
    before = [(cid, n, b, e) for cid, n, b, e in t.get_chunks()]
    with pytest.raises(RuntimeError, match="capacity reached"):
        t.append_completion(0, [7, 8])   # 1 clone + 2 successors = 3 more chunks, only 2 left
    assert t.get_chunks() == before and len(t.tails) == 1 and t.tails[0].tokens == [3]
    with pytest.raises(RuntimeError, match="out of range"):
        t.append_completion(3, [1])
    with pytest.raises(RuntimeError, match="at least one token"):
        t.append_completion(0, [])


def test_work_list_of_a_forked_tree_is_accepted_by_the_planner():
    t = PrefixTree(chunk_size=64, max_chunks=256)
    base = list(range(200))
    t.add_seq(base)
    for step in range(3):
        for row in reversed(range(len(t.tails))):
            t.append_completion(row, [1000 + step, 2000 + step])
    assert len(t.tails) == 8
    plan = cabi.Plan(t.get_chunks(), len(t.tails), 4)
    st = plan.stats()
    assert st["n_shared_chunks"] == 3  # the three full chunks of the common history


def test_oracle_beam_step_matches_dense():
    rng = np.random.default_rng(0)
    H, d, C = 2, 8, 4
    ora = OracleAttention(H, d, C)
    hist = {}

    def kv(n):
        return rng.standard_normal((n, H, d)).astype(np.float32), rng.standard_normal((n, H, d)).astype(np.float32)

    for s, toks in enumerate([[1, 2, 3, 4, 5, 6], [1, 2, 3, 4, 7], [8, 9]]):
        k, v = kv(len(toks))
        if s == 1:  # shared prefix rows must carry the same values
            k[:4], v[:4] = hist[0][0][:4], hist[0][1][:4]
        idx = ora.add_seq(toks, k, v)
        hist = {(r + 1 if r >= idx else r): kvp for r, kvp in hist.items()}
        hist[idx] = (k, v)
    for step in range(6):  # fork every row in turn; crosses chunk boundaries
        row = step % len(ora.tails)
        n_new = 1 + step % 3
        k, v = kv(n_new)
        ora.append_completion(row, [100 + step * 10 + i for i in range(n_new)], k, v)
        old = hist
        hist = {}
        for r, (hk, hv) in old.items():
            if r < row:
                hist[r] = (hk, hv)
            elif r > row:
                hist[r + n_new - 1] = (hk, hv)
            else:
                for i in range(n_new):
                    hist[row + i] = (np.concatenate([hk, k[i:i + 1]]), np.concatenate([hv, v[i:i + 1]]))
        q = rng.standard_normal((len(ora.tails), H, d)).astype(np.float32)
        out = ora.forward(q)
        for r in range(len(ora.tails)):
            hk, hv = hist[r]
            want = dense_attention(q[r], hk.transpose(1, 0, 2), hv.transpose(1, 0, 2))
            np.testing.assert_allclose(out[r], want, rtol=1e-5, atol=1e-6)
