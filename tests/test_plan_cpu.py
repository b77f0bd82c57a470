"""Work-list builder (planner): emulate, in numpy, what the kernels do with a plan and compare the
result with dense attention.  Runs without a GPU."""
import numpy as np
import pytest

from chunk_attn import cabi
from chunk_attn_oracle import Attention as OracleAttention, dense_forward
from plan_emulator import emulate
from tree_traces import kv_for, random_trace

C = 64  # the fast path's chunk size; the planner is only used for that geometry


def build_tree(spec, H=2, d=8, seed=0, chunk_size=C):
    """spec: list of token lists.  Returns the oracle tree (which owns K/V per chunk)."""
    rng = np.random.default_rng(seed)
    shared_kv = {}
    ora = OracleAttention(H, d, chunk_size)
    for toks in spec:
        # K/V are a function of (position, token id) so that shared prefixes carry equal values
        k = np.zeros((len(toks), H, d), np.float32)
        v = np.zeros((len(toks), H, d), np.float32)
        for i, t in enumerate(toks):
            key = (i, t)
            if key not in shared_kv:
                shared_kv[key] = (rng.standard_normal((H, d)).astype(np.float32),
                                  rng.standard_normal((H, d)).astype(np.float32))
            k[i], v[i] = shared_kv[key]
        ora.add_seq(toks, k, v)
    return ora


def plan_of(ora, n_heads, **kw):
    infos = [(c.id, c.n_tokens, b, e) for c, b, e in ora.get_chunks()]
    return cabi.Plan(infos, len(ora.tails), n_heads, chunk_size=ora.chunk_size, **kw), infos


def kv_map(ora):
    return {c.id: (c.k, c.v) for c, _, _ in ora.get_chunks()}


def check(ora, H, d, atol=1e-9, **kw):
    plan, _ = plan_of(ora, H, **kw)
    rng = np.random.default_rng(7)
    q = rng.standard_normal((len(ora.tails), H, d)).astype(np.float32)
    sched = "split" if kw.get("split_phases") else "fused"
    out, loads = emulate(plan, kv_map(ora), q, ora.chunk_size, schedule=sched)
    ref = dense_forward(ora, q)
    assert np.abs(out - ref).max() < atol
    return plan, loads


def shared_spec(n_seqs, shared, unique, base=0):
    return [list(range(base, base + shared)) + [1_000_000 * (s + 1) + j for j in range(unique)] for s in range(n_seqs)]


@pytest.mark.parametrize("n_ctas", [1, 3, 16, 148])
@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("tensor_tails", [True, False])
def test_single_level_prefix(n_ctas, split, tensor_tails):
    ora = build_tree(shared_spec(6, 5 * C, 2 * C + 17))
    plan, loads = check(ora, 2, 8, n_ctas=n_ctas, split_phases=split, seq_first_tensor=tensor_tails)
    assert sorted(set(int(f) >> 8 for f in plan.items()[:, 5])) == ([4] if tensor_tails else [0, 4])
    st = plan.stats()
    assert st["n_shared_chunks"] == 5 and st["n_runs"] == 1
    assert st["n_chunks"] == 5 + 6 * 3


def test_partial_tails_and_empty_tails():
    for unique in (0, 1, 17, 63, 64, 65):
        ora = build_tree(shared_spec(5, 2 * C, unique))
        check(ora, 2, 8, n_ctas=7)


def test_two_level_tree_and_row_blocks():
    # 3 groups under a root prefix; group sizes 2, 20 and 70 exercise the 4-, 2- and 1-split items
    spec = []
    root = list(range(2 * C))
    for g, n in enumerate((2, 20, 70)):
        gp = [10_000 * (g + 1) + j for j in range(C)]
        for s in range(n):
            spec.append(root + gp + [1_000_000 * (len(spec) + 1) + j for j in range(9)])
    ora = build_tree(spec, H=1, d=4)
    plan, _ = check(ora, 1, 4, n_ctas=20)
    items = plan.items()
    splits = sorted(set(int(f) >> 8 for f in items[:, 5]))
    assert splits == [1, 2, 4]  # 92 and 70 rows -> blocks of <= 64 rows, 1 split; 20 -> 2; 2 rows and tails -> 4
    assert plan.stats()["n_runs"] == 4


def test_more_than_128_sharers_splits_rows():
    ora = build_tree(shared_spec(150, C, 3), H=1, d=4)
    plan, _ = check(ora, 1, 4, n_ctas=8)
    rows = [int(r) for r in plan.items()[:, 3] if r > 1]
    assert max(rows) <= 64


def test_no_sharing_and_full_sharing():
    ora = build_tree(shared_spec(4, 0, 3 * C + 5))
    plan, _ = check(ora, 2, 8, n_ctas=5)
    assert plan.stats()["n_shared_chunks"] == 0
    ora = build_tree([list(range(2 * C))] * 5)
    plan, _ = check(ora, 2, 8, n_ctas=5)
    assert plan.stats()["n_shared_chunks"] == 2


def test_tpp_threshold_moves_chunks_to_the_private_walk():
    ora = build_tree(shared_spec(3, 2 * C, 10))
    plan, _ = check(ora, 2, 8, n_ctas=4, tpp_threshold=3)
    assert plan.stats()["n_shared_chunks"] == 0
    plan, _ = check(ora, 2, 8, n_ctas=4, tpp_threshold=2)
    assert plan.stats()["n_shared_chunks"] == 2


def test_delta_tokens_are_applied_to_tails_only():
    ora = build_tree(shared_spec(4, C, 20))
    plan, _ = plan_of(ora, 2, n_ctas=6)
    # append 3 tokens to every sequence without rebuilding the plan
    rng = np.random.default_rng(3)
    for step in range(3):
        k, v = kv_for(4, 2, 8, rng)
        ora.append_token([5000 + step] * 4, k, v)
    q = rng.standard_normal((4, 2, 8)).astype(np.float32)
    out, _ = emulate(plan, kv_map(ora), q, C, delta=3)
    assert np.abs(out - dense_forward(ora, q)).max() < 1e-9


@pytest.mark.parametrize("seed", range(8))
def test_random_traces(seed):
    ops = random_trace(seed, n_ops=40, chunk_size=8, vocab=2, max_len=50, max_live=12)
    rng = np.random.default_rng(seed)
    ora = OracleAttention(2, 4, 8)
    pos_kv = {}
    for op, arg in ops:
        if op == "add":
            k = np.zeros((len(arg), 2, 4), np.float32)
            v = np.zeros((len(arg), 2, 4), np.float32)
            for i, t in enumerate(arg):
                if (i, t) not in pos_kv:
                    pos_kv[(i, t)] = kv_for(1, 2, 4, rng)
                k[i], v[i] = pos_kv[(i, t)][0][0], pos_kv[(i, t)][1][0]
            ora.add_seq(arg, k, v)
        elif op == "remove":
            ora.remove_seq(arg)
        else:
            k, v = kv_for(len(arg), 2, 4, rng)
            ora.append_token(arg, k, v)
        if not ora.tails:
            continue
        # the planner is geometry-agnostic: exercise it with chunk_size 8 (4 splits of 2 tokens)
        check(ora, 2, 4, n_ctas=1 + seed, split_phases=bool(seed & 1))


def test_items_of_config2_shape():
    # 32 sequences, 2048 shared + 512 unique tokens, 32 heads: full-size items first, single tiles last
    infos = []
    cid = 0
    for _ in range(32):
        infos.append((cid, C, 0, 32)); cid += 1
    for s in range(32):
        for _ in range(8):
            infos.append((cid, C, s, s + 1)); cid += 1
        infos.append((cid, 0, s, s + 1)); cid += 1
    plan = cabi.Plan(infos, 32, 32, n_ctas=296)
    items = np.repeat(plan.items(), 32, axis=0)   # every item stands for one piece of work per head
    sizes = items[:, 0]
    full = sizes - (items[:, 5] & 1)          # the tails are empty here
    assert sizes.max() == 9 and full.max() == 8 and full[0] == 8 and full.min() >= 1
    # guided self-scheduling: full-size items while much work remains, single tiles at the end
    assert (full[:296] == 8).all() and (full[-296:] == 1).all()
    means = [full[i:i + 200].mean() for i in range(0, len(full) - 200, 200)]
    assert all(a >= b - 0.5 for a, b in zip(means, means[1:]))
    st = plan.stats()
    assert st["unique_kv_bytes"] == 301_989_888 and st["n_runs"] == 1 and st["n_ctas"] == 296
    assert int((sizes - (items[:, 5] & 1)).sum()) == 32 * 32 + 32 * 32 * 8  # every full tile exactly once


def test_rejects_bad_work_lists():
    with pytest.raises(cabi.CAError, match="outside the pool"):
        cabi.Plan([(5, 1, 0, 1)], 1, 1, max_chunks=5)
    with pytest.raises(cabi.CAError, match="served by no chunk"):
        cabi.Plan([(0, 1, 0, 1)], 2, 1)
    with pytest.raises(cabi.CAError, match="needs its own tail"):
        cabi.Plan([(0, C, 0, 2)], 2, 1)
    with pytest.raises(cabi.CAError, match="empty or outside"):
        cabi.Plan([(0, 1, 1, 1)], 2, 1)
    with pytest.raises(cabi.CAError, match="n_tokens"):
        cabi.Plan([(0, C + 1, 0, 1)], 1, 1)


def test_short_tails_go_to_the_end_of_the_list_when_there_are_many():
    """Private parts of a single chunk become single-tile items after the persistent kernel's items as soon as
    there are more of them than four per CTA; the merge lists do not care who writes a slot."""
    H, d = 2, 8
    spec = shared_spec(6, 2 * C, 5) + shared_spec(2, 2 * C, 3 * C + 7, base=0)  # 6 short tails, 2 long private parts
    ora = build_tree(spec, H, d)
    plan, _ = check(ora, H, d, n_ctas=2)          # 12 short items > 4 x 2 CTAs: routed
    st = plan.stats()
    items = plan.items()
    assert st["n_items_short"] == 6 * H and st["kernels_per_step"] == 3
    tail = items[-st["n_items_short"] // H:]      # the list holds every item once for all heads
    assert all(int(r[0]) == 1 and int(r[3]) == 1 and int(r[5]) & 1 for r in tail)      # one tile, one row, a tail
    assert sorted(int(r[2]) for r in tail) == list(range(6))
    main = items[:-st["n_items_short"] // H]
    assert not any(int(r[3]) == 1 and int(r[2]) < 6 for r in main)                     # none of them is walked twice
    plan2, _ = check(ora, H, d, n_ctas=64)        # 12 short items <= 4 x 64 CTAs: they stay in the main list
    assert plan2.stats()["n_items_short"] == 0 and plan2.stats()["kernels_per_step"] == 2
    plan3, _ = check(ora, H, d, n_ctas=2, seq_first_tensor=False)   # the CUDA-core option keeps its own walk
    assert plan3.stats()["n_items_short"] == 0


# ---- wide shared runs: the items of the tcgen05 kernel -----------------------------------------------------------
@pytest.mark.parametrize("n_seqs,n_ctas", [(2, 8), (70, 8), (130, 296), (300, 16)])
def test_wide_runs_forced(n_seqs, n_ctas):
    # wide_runs = 2 sends every shared run to the wide kernel: row blocks of up to 128 rows, pieces of up to 32 chunks
    ora = build_tree(shared_spec(n_seqs, 5 * C, C + 9), H=2, d=8)
    plan, loads = check(ora, 2, 8, n_ctas=n_ctas, wide_runs=2)
    st = plan.stats()
    items = plan.items()
    wide = items[len(items) - st["n_items_wide"] // 2:]
    assert st["n_items_wide"] > 0 and st["n_items_cf"] == 0
    assert all(int(r[3]) > 1 for r in wide) and max(int(r[3]) for r in wide) <= 128
    blocks = (n_seqs + 127) // 128
    assert sum(int(r[0]) for r in wide) == 5 * blocks                # every chunk once per row block (and per head)
    assert st["kernels_per_step"] == 3                                # wide + persistent (the private tails) + merge


def test_wide_routing_by_cost():
    # automatic routing: a long prefix under many rows and next to nothing else is bound by the contraction ...
    ora = build_tree(shared_spec(100, 20 * C, 3), H=2, d=8)
    plan, _ = check(ora, 2, 8, n_ctas=32, wide_runs=1)
    assert plan.stats()["n_items_wide"] > 0
    # ... the same prefix under long private tails is bound by memory and stays with the persistent kernel,
    ora = build_tree(shared_spec(40, 2 * C, 20 * C), H=2, d=8)
    plan, _ = check(ora, 2, 8, n_ctas=32, wide_runs=1)
    assert plan.stats()["n_items_wide"] == 0
    # and so do runs of few rows, however long
    ora = build_tree(shared_spec(32, 30 * C, 3), H=2, d=8)
    plan, _ = check(ora, 2, 8, n_ctas=32, wide_runs=1)
    assert plan.stats()["n_items_wide"] == 0
    # wide_runs = 0 never routes
    ora = build_tree(shared_spec(100, 20 * C, 3), H=2, d=8)
    plan, _ = check(ora, 2, 8, n_ctas=32, wide_runs=0)
    assert plan.stats()["n_items_wide"] == 0


def test_wide_two_level_tree_and_long_runs():
    # a root run of 70 chunks (pieces of at most 32) over 150 rows (two row blocks), groups below it
    spec = []
    root = list(range(70 * C))
    for g, n in enumerate((100, 50)):
        gp = [10_000_000 * (g + 1) + j for j in range(2 * C)]
        for s in range(n):
            spec.append(root + gp + [100_000_000 * (len(spec) + 1) + j for j in range(5)])
    ora = build_tree(spec, H=1, d=4)
    plan, loads = check(ora, 1, 4, n_ctas=4, wide_runs=2, atol=1e-8)
    wide = plan.items()[len(plan.items()) - plan.stats()["n_items_wide"]:]   # one head
    assert max(int(r[0]) for r in wide) <= 32 and min(int(r[0]) for r in wide) >= 2
