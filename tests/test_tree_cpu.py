"""Host prefix tree: the reference's own tree-shape assertions, and differential runs against the
oracle (and against the unmodified reference build when it is present) on random traces."""
import numpy as np
import pytest

from chunk_attn import PrefixTree
from chunk_attn_oracle import Attention as OracleAttention
from ref_loader import load_reference
from tree_traces import kv_for, random_trace, tails_shape, tree_shape


def node(n):
    return (n.n_seqs, n.n_tokens, n.tokens)


def test_add_seq_shapes():
    # the sequence of inserts and every assertion of the reference's test_add_seq
    # (tests/test_chunk_attn_cpu.py:24-175)
    t = PrefixTree(chunk_size=2, max_chunks=64)
    assert t.add_seq([1, 2, 3, 4, 5]) == 0
    trie = t.get_trie()
    assert node(trie) == (1, 0, [])
    n1 = trie.children[0]
    n2 = n1.children[0]
    n3 = n2.children[0]
    assert node(n1) == (1, 2, [1, 2]) and node(n2) == (1, 2, [3, 4]) and node(n3) == (1, 1, [5])
    assert t.tails == [n3]

    assert t.add_seq([1, 2, 3, 4, 6]) == 1
    assert node(trie) == (2, 0, []) and node(n1) == (2, 2, [1, 2]) and node(n2) == (2, 2, [3, 4])
    n4 = n2.children[1]
    assert node(n3) == (1, 1, [5]) and node(n4) == (1, 1, [6])
    assert t.tails == [n3, n4]

    assert t.add_seq([1, 2, 3, 4]) == 2          # exact prefix: gets an empty private tail
    n5 = n2.children[2]
    assert node(trie) == (3, 0, []) and node(n2) == (3, 2, [3, 4]) and node(n5) == (1, 0, [])
    assert t.tails == [n3, n4, n5]

    assert t.add_seq([1, 7]) == 3                # [1, 7] != [1, 2]: new branch under the root
    n6 = trie.children[1]
    n7 = n6.children[0]
    assert node(trie) == (4, 0, []) and node(n1) == (3, 2, [1, 2])
    assert node(n6) == (1, 2, [1, 7]) and node(n7) == (1, 0, [])
    assert t.tails == [n3, n4, n5, n7]

    assert t.add_seq([1, 2]) == 3                # lands after n2's three sequences
    n8 = n1.children[1]
    assert node(trie) == (5, 0, []) and node(n1) == (4, 2, [1, 2]) and node(n2) == (3, 2, [3, 4])
    assert node(n8) == (1, 0, [])
    assert t.tails == [n3, n4, n5, n8, n7]

    assert t.add_seq([1, 2, 3, 4, 5]) == 3       # never shares the leaf [5]
    n9 = n2.children[3]
    assert node(trie) == (6, 0, []) and node(n1) == (5, 2, [1, 2]) and node(n2) == (4, 2, [3, 4])
    assert node(n3) == (1, 1, [5]) and node(n9) == (1, 1, [5])
    assert t.tails == [n3, n4, n5, n9, n8, n7]
    assert all(c.capacity == 2 for c in t.tails)


def test_append_token_shapes():
    # tests/test_chunk_attn_cpu.py:177-215
    t = PrefixTree(chunk_size=2, max_chunks=64)
    t.add_seq([1, 2, 3, 4, 5])
    t.add_seq([1, 2, 3, 4, 6, 7])
    t.append_token([8, 9])
    trie = t.get_trie()
    n1 = trie.children[0]
    n2 = n1.children[0]
    n3, n4 = n2.children
    n5 = n4.children[0]
    assert node(trie) == (2, 0, []) and node(n1) == (2, 2, [1, 2]) and node(n2) == (2, 2, [3, 4])
    assert node(n3) == (1, 2, [5, 8]) and node(n4) == (1, 2, [6, 7]) and node(n5) == (1, 1, [9])
    assert t.tails == [n3, n5]
    with pytest.raises(RuntimeError, match="num of seqs is not equal to num of tokens"):
        t.append_token([1])


def test_remove_shapes():
    # tests/test_chunk_attn_cpu.py:267-303
    t = PrefixTree(chunk_size=2, max_chunks=64)
    t.add_seq([1, 2, 3, 4, 5])
    t.add_seq([1, 2, 3, 4, 6])
    t.remove_seq(0)
    trie = t.get_trie()
    n1 = trie.children[0]
    n2 = n1.children[0]
    n3 = n2.children[0]
    assert node(trie) == (1, 0, []) and node(n1) == (1, 2, [1, 2]) and node(n2) == (1, 2, [3, 4])
    assert node(n3) == (1, 1, [6]) and len(n2.children) == 1
    assert t.chunks_in_use() == 3
    t.remove_seq(0)
    assert t.chunks_in_use() == 0 and t.tails == [] and node(trie) == (0, 0, [])
    with pytest.raises(RuntimeError):
        t.remove_seq(0)


def test_pool_exhaustion_leaves_tree_intact():
    t = PrefixTree(chunk_size=2, max_chunks=3)
    t.add_seq([1, 2, 3])                      # 2 chunks
    before = tree_shape(t.get_trie())
    with pytest.raises(RuntimeError, match="capacity reached"):
        t.add_seq([9, 9, 9, 9])               # needs 2 + an empty tail
    assert tree_shape(t.get_trie()) == before and len(t.tails) == 1
    t.add_seq([1, 2, 4])                      # shares [1, 2]: needs only one more
    assert t.chunks_in_use() == 3
    t.append_token([5, 6])                    # fills both tails
    with pytest.raises(RuntimeError, match="capacity reached"):
        t.reserve()


def test_clear_and_reuse():
    t = PrefixTree(chunk_size=4, max_chunks=32)
    for i in range(5):
        t.add_seq([1, 2, 3, 4, 10 + i])
    t.clear()
    assert t.chunks_in_use() == 0 and t.tails == []
    assert t.add_seq([1, 2, 3]) == 0


def test_duplicate_rows_follow_source():
    t = PrefixTree(chunk_size=2, max_chunks=32)
    t.add_seq([1, 2, 3])
    t.add_seq([1, 2, 4])
    pairs = t.duplicate(0, 2)
    assert len(pairs) == 2 and all(src == t.tails[0].id for src, _ in pairs)
    assert [x.tokens for x in t.tails] == [[3], [3], [3], [4]]
    assert t.get_trie().n_seqs == 4 and t.get_trie().children[0].n_seqs == 4
    # the depth-first work list agrees with the row order
    rows = {cid: (b, e) for cid, _, b, e in t.get_chunks()}
    for i, tail in enumerate(t.tails):
        assert rows[tail.id] == (i, i + 1)


def run_trace(ops, chunk_size, drivers):
    """Apply ops to every driver; return list of per-step (tree shape, tails shape, returned idx)."""
    rng = np.random.default_rng(0)
    H, d = 1, 2
    out = [[] for _ in drivers]
    for op, arg in ops:
        if op == "add":
            k, v = kv_for(arg, H, d, rng)
        elif op == "append":
            k, v = kv_for(len(arg), H, d, rng)
        for i, drv in enumerate(drivers):
            ret = drv(op, arg, k if op != "remove" else None, v if op != "remove" else None)
            out[i].append(ret)
    return out


@pytest.mark.parametrize("seed", range(12))
def test_differential_vs_oracle(seed):
    chunk_size = [2, 3, 4][seed % 3]
    ops = random_trace(seed, chunk_size=chunk_size)
    eng = PrefixTree(chunk_size=chunk_size, max_chunks=4096)
    ora = OracleAttention(1, 2, chunk_size)

    def drive_engine(op, arg, k, v):
        r = None
        if op == "add":
            r = eng.add_seq(arg)
        elif op == "remove":
            eng.remove_seq(arg)
        else:
            eng.append_token(arg)
        return (r, tree_shape(eng.get_trie()), tails_shape(eng.tails),
                [(nt, b, e) for _, nt, b, e in eng.get_chunks()])

    def drive_oracle(op, arg, k, v):
        r = None
        if op == "add":
            r = ora.add_seq(arg, k, v)
        elif op == "remove":
            ora.remove_seq(arg)
        else:
            ora.append_token(arg, k, v)
        return (r, ora.shape(), tails_shape(ora.tails), [(c.n_tokens, b, e) for c, b, e in ora.get_chunks()])

    a, b = run_trace(ops, chunk_size, [drive_engine, drive_oracle])
    assert a == b


@pytest.mark.parametrize("seed", range(6))
def test_differential_vs_reference_build(seed):
    ref = load_reference("cpu")
    if ref is None:
        pytest.skip("oracle/_ref is not built here")
    import torch
    chunk_size = [2, 3, 4][seed % 3]
    ops = random_trace(100 + seed, chunk_size=chunk_size)
    eng = PrefixTree(chunk_size=chunk_size, max_chunks=4096)
    ra = ref.Attention(n_heads=1, d_head=2, chunk_size=chunk_size, memory_mb=1, dtype=torch.float32,
                       device=torch.device("cpu"))
    for op, arg in ops:
        if op == "add":
            k = torch.zeros(len(arg), 1, 2)
            assert eng.add_seq(arg) == ra.add_seq(tokens=arg, k=k, v=k)
        elif op == "remove":
            eng.remove_seq(arg)
            ra.remove_seq(arg)
        else:
            k = torch.zeros(len(arg), 1, 2)
            eng.append_token(arg)
            ra.append_token(tokens=arg, k=k, v=k, fused=False)
        assert tree_shape(eng.get_trie()) == tree_shape(ra.get_trie())
        assert tails_shape(eng.tails) == tails_shape(ra.tails)
