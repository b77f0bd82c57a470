"""numpy emulation of what the kernels do with a work list (plan): every item produces partial
(max, sum, O) rows exactly as the persistent kernel's warps would, and the merge lists combine
them.  It lets the planner be checked end to end against dense attention on a machine without a
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
    assert all(1 <= n <= 9 for n in loads)
    if schedule == "split":
        kinds = [int(r[3]) > 1 for r in items]
        assert kinds == sorted(kinds, reverse=True), "chunk-first items must come first"
        assert sum(kinds) == st["n_items_cf"]

    for row in items:
        n_tiles, head, row_begin, n_rows, slot_base, flags, last_tokens = (int(x) for x in row[:7])
        tiles = row[7:]
        tile_begin = 0
        splits = flags >> 8
        tail = flags & 1
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
            if Kc.shape[0] == 0:
                part_m[slot0:slot0 + n_rows] = -1e30
                part_l[slot0:slot0 + n_rows] = 0
                part_o[slot0:slot0 + n_rows] = 0
                continue
            s = qr @ Kc.T * scale
            m = s.max(axis=1)
            p = np.exp(s - m[:, None])
            part_m[slot0:slot0 + n_rows] = m
            part_l[slot0:slot0 + n_rows] = p.sum(axis=1)
            part_o[slot0:slot0 + n_rows] = p @ Vc

    merge_off = plan.array(cabi.PLAN_MERGE_OFF)
    merge_slots = plan.array(cabi.PLAN_MERGE_SLOTS)
    used = np.zeros(st["n_slots"], np.int32)
    out = np.zeros((n_seqs, H, d))
    for s_ in range(n_seqs):
        for h in range(H):
            sl = merge_slots[merge_off[s_ * H + h]:merge_off[s_ * H + h + 1]]
            used[sl] += 1
            m = part_m[sl]
            assert not np.isnan(m).any(), "merge list names a slot nobody wrote"
            M = m.max()
            w = np.exp(m - M)
            L = (w * part_l[sl]).sum()
            out[s_, h] = (w[:, None] * part_o[sl]).sum(axis=0) / L if L > 0 else 0.0
    assert (used == 1).all(), "every partial slot must be merged exactly once"
    return out, loads
