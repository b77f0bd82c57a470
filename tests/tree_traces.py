"""Small helpers shared by the tests: random tree traces and tree-shape extraction."""
import random

import numpy as np


def tree_shape(root):
    """Nested (n_seqs, tokens, [children]) of a Chunk tree (oracle, engine or reference object)."""
    return (root.n_seqs, list(root.tokens), [tree_shape(c) for c in root.children])


def tails_shape(tails):
    return [(t.n_seqs, list(t.tokens)) for t in tails]


def random_trace(seed, n_ops=60, chunk_size=4, vocab=3, max_len=14, max_live=9):
    """A reproducible list of tree operations: ('add', tokens) | ('remove', idx) | ('append', tokens).
    A tiny vocabulary and short sequences make prefix collisions, exact-prefix inserts, full-chunk
    tails and removals of shared branches all frequent."""
    rng = random.Random(seed)
    ops, live = [], 0
    for _ in range(n_ops):
        r = rng.random()
        if live == 0 or (r < 0.45 and live < max_live):
            n = rng.randint(1, max_len)
            ops.append(("add", [rng.randrange(vocab) for _ in range(n)]))
            live += 1
        elif r < 0.65:
            ops.append(("remove", rng.randrange(live)))
            live -= 1
        else:
            ops.append(("append", [rng.randrange(vocab) + 10 for _ in range(live)]))
    return ops


def kv_for(tokens_or_n, n_heads, d_head, rng):
    n = tokens_or_n if isinstance(tokens_or_n, int) else len(tokens_or_n)
    k = rng.standard_normal((n, n_heads, d_head)).astype(np.float32)
    v = rng.standard_normal((n, n_heads, d_head)).astype(np.float32)
    return k, v
