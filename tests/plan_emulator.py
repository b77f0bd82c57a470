"""numpy emulation of what the kernels do with a work list (plan): every item, expanded over the
heads as the kernels expand it (piece v = item v // H for head v % H, partial row ts of head h in slot
ts * H + h), produces partial (max, sum, O) rows exactly as the kernels' warps would, and the per-row
merge lists combine them.  It lets the planner be checked end to end against dense attention on a machine without a
GPU: any tile that is dropped, duplicated, mis-assigned to a row or mis-merged shows up as a
numerical mismatch."""
import math

import numpy as np

from chunk_attn import cabi


def emulate(plan, kv_of_chunk, q, chunk_size, delta=0, schedule="fused"):
    """plan: cabi.Plan; kv_of_chunk: chunk_id -> (K [H, C, d], V [H, C, d]) float arrays;
    q: [n_seqs, H, d].  Returns out [n_seqs, H, d] float64 and the list of (cta, item) visits."""
    items = plan.items()
    st = plan.stats()
    n_seqs, H, d = q.shape
    scale = 1.0 / math.sqrt(d)
    part_o = np.full((st["n_slots"], d), np.nan)
    part_m = np.full(st["n_slots"], np.nan)
    part_l = np.full(st["n_slots"], np.nan)
    # items are self-scheduled: any CTA may take any item, each exactly once
    loads = [int(r[0]) for r in items]
    wide_chunks = plan.array(cabi.PLAN_WIDE_CHUNKS)
    assert st["n_items"] == len(items) * H and st["n_slots"] % H == 0
    n_wide = st["n_items_wide"] // H
    is_wide = [bool(int(r[5]) & 2) for r in items]
    assert sum(is_wide) == n_wide and all(is_wide[len(items) - n_wide:]), "wide items come last"
    assert all(1 <= n <= (32 if w else 9) for n, w in zip(loads, is_wide))
    if schedule == "split":
        kinds = [int(r[3]) > 1 for r in items[:len(items) - n_wide]]
        assert kinds == sorted(kinds, reverse=True), "chunk-first items must come first"
        assert sum(kinds) * H == st["n_items_cf"]

    for row, head in ((row, head) for row in items for head in range(H)):
        n_tiles, _, row_begin, n_rows, slot_base, flags, last_tokens = (int(x) for x in row[:7])
        tiles = row[7:]
        tile_begin = 0
        splits = flags >> 8
        tail = flags & 1
        if flags & 2:   # a piece of a wide run for the tcgen05 kernel: up to 128 rows, chunk list held aside
            assert 2 <= n_rows <= 128 and splits == 1 and not tail and last_tokens == chunk_size
            tiles = wide_chunks[int(row[7]):int(row[7]) + n_tiles]
        else:
            assert n_rows <= 64
        ks, vs = [], []
        for j in range(n_tiles):
            nt = chunk_size
            if j == n_tiles - 1:
                nt = min(chunk_size, last_tokens + (delta if tail else 0))
            K, V = kv_of_chunk[int(tiles[tile_begin + j])]
            ks.append((K[head], nt))
            vs.append(V[head])
        if n_rows == 1:
            assert splits in (0, 4)
            groups = [(slot_base, [(0, chunk_size)])]  # warps combined on chip: one slot, all tokens
        else:
            tw = chunk_size // splits
            groups = [(slot_base + sp * n_rows, [(sp * tw, (sp + 1) * tw)]) for sp in range(splits)]
        qr = q[row_begin:row_begin + n_rows, head, :].astype(np.float64)
        for slot0, ranges in groups:
            lo, hi = ranges[0]
            kk = [k[lo:min(hi, nt)] for (k, nt) in ks]
            vv = [v[lo:min(hi, nt)] for v, (k, nt) in zip(vs, ks)]
            Kc = np.concatenate(kk, axis=0).astype(np.float64) if kk else np.zeros((0, d))
            Vc = np.concatenate(vv, axis=0).astype(np.float64) if vv else np.zeros((0, d))
            sl = (slot0 + np.arange(n_rows)) * H + head   # this head's copies of the item's partial rows
            if Kc.shape[0] == 0:
                part_m[sl] = -1e30
                part_l[sl] = 0
                part_o[sl] = 0
                continue
            s = qr @ Kc.T * scale
            m = s.max(axis=1)
            p = np.exp(s - m[:, None])
            part_m[sl] = m
            part_l[sl] = p.sum(axis=1)
            part_o[sl] = p @ Vc

    merge_off = plan.array(cabi.PLAN_MERGE_OFF)
    merge_slots = plan.array(cabi.PLAN_MERGE_SLOTS)
    used = np.zeros(st["n_slots"], np.int32)
    out = np.zeros((n_seqs, H, d))
    for s_ in range(n_seqs):
        for h in range(H):
            sl = merge_slots[merge_off[s_]:merge_off[s_ + 1]] * H + h
            used[sl] += 1
            m = part_m[sl]
            assert not np.isnan(m).any(), "merge list names a slot nobody wrote"
            M = m.max()
            w = np.exp(m - M)
            L = (w * part_l[sl]).sum()
            out[s_, h] = (w[:, None] * part_o[sl]).sum(axis=0) / L if L > 0 else 0.0
    assert (used == 1).all(), "every partial slot must be merged exactly once"
    return out, loads
