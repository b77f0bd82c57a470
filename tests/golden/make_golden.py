"""Generate the golden vectors of tests/golden/ from the UNMODIFIED reference (its MKL CPU build in
oracle/_ref/cpu, made by oracle/build_ref.py).  Run where the reference tree and that build exist:

    python tests/golden/make_golden.py

Each fixture is a small .npz holding seeded inputs in the exact form they were fed to the reference,
the row index every add_seq returned, the tree shape and the `tails` order after each operation,
and the reference's forward() outputs for partition 0 (chunk-first) and 2 (sequence-first).
The fixtures pin oracle/chunk_attn_oracle.py on machines where the reference cannot be built.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))
from ref_loader import load_reference  # noqa: E402
from tree_traces import random_trace, tails_shape, tree_shape  # noqa: E402


def run_case(ref, name, H, d, C, ops, seed):
    """ops: list of ('add', tokens) | ('remove', idx) | ('append', tokens) | ('forward',)."""
    g = torch.Generator().manual_seed(seed)
    attn = ref.Attention(n_heads=H, d_head=d, chunk_size=C, memory_mb=64, dtype=torch.float32,
                         device=torch.device("cpu"))
    arrays, log = {}, []
    pos_kv = {}
    for i, op in enumerate(ops):
        rec = {"op": op[0]}
        if op[0] == "add":
            toks = op[1]
            # K/V are a function of (position, token id): sequences that share a prefix carry equal values
            k = torch.zeros(len(toks), H, d)
            v = torch.zeros(len(toks), H, d)
            for j, t in enumerate(toks):
                if (j, t) not in pos_kv:
                    pos_kv[(j, t)] = (torch.randn(H, d, generator=g), torch.randn(H, d, generator=g))
                k[j], v[j] = pos_kv[(j, t)]
            rec["tokens"] = toks
            rec["row"] = int(attn.add_seq(tokens=toks, k=k, v=v))
            arrays["k%d" % i], arrays["v%d" % i] = k.numpy(), v.numpy()
        elif op[0] == "remove":
            rec["row"] = op[1]
            attn.remove_seq(op[1])
        elif op[0] == "append":
            toks = op[1]
            k, v = torch.randn(len(toks), H, d, generator=g), torch.randn(len(toks), H, d, generator=g)
            rec["tokens"] = toks
            attn.append_token(tokens=toks, k=k, v=v, fused=False)
            arrays["k%d" % i], arrays["v%d" % i] = k.numpy(), v.numpy()
        elif op[0] == "forward":
            n = len(attn.tails)
            q = torch.randn(n, H, d, generator=g)
            arrays["q%d" % i] = q.numpy()
            arrays["out0_%d" % i] = attn.forward(q, 0).numpy()
            arrays["out2_%d" % i] = attn.forward(q, 2).numpy()
        rec["tree"] = tree_shape(attn.get_trie())
        rec["tails"] = tails_shape(attn.tails)
        log.append(rec)
    meta = {"name": name, "n_heads": H, "d_head": d, "chunk_size": C, "seed": seed, "log": log}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), meta=json.dumps(meta), **arrays)
    print("wrote", name, "%d ops" % len(ops))


def main():
    ref = load_reference("cpu")
    if ref is None:
        raise SystemExit("oracle/_ref/cpu is not built: run `python oracle/build_ref.py` first")
    # 1. the reference's own forward test shape: two sequences sharing four tokens, chunk_size 2
    run_case(ref, "ref_forward_case", 2, 4, 2,
             [("add", [1, 2, 3, 4, 5]), ("add", [1, 2, 3, 4, 6, 7]), ("forward",)], seed=10)
    # 2. the insert sequence of the reference's test_add_seq, with a forward after every insert
    ops = []
    for toks in ([1, 2, 3, 4, 5], [1, 2, 3, 4, 6], [1, 2, 3, 4], [1, 7], [1, 2], [1, 2, 3, 4, 5]):
        ops += [("add", toks), ("forward",)]
    run_case(ref, "ref_add_seq_case", 2, 4, 2, ops, seed=11)
    # 3. configuration 1 scaled to fixture size: H4 d16 c8, 4 sequences = 32 shared + 8 unique
    shared = list(range(32))
    ops = [("add", shared + [1000 * (s + 1) + j for j in range(8)]) for s in range(4)] + [("forward",)]
    run_case(ref, "cfg1_scaled", 4, 16, 8, ops, seed=12)
    # 4. two-level tree with appended tokens and churn (configuration 4, scaled)
    root, groups = list(range(16)), [[100 * (g + 1) + j for j in range(8)] for g in range(3)]
    ops = [("add", root + groups[g] + [10000 * (3 * g + s + 1) + j for j in range(5)]) for g in range(3) for s in range(3)]
    ops.append(("forward",))
    for step in range(6):
        live = 9
        ops.append(("append", [500 + step] * live))
        ops.append(("forward",))
    ops += [("remove", 4), ("remove", 0), ("add", root + groups[1] + [777, 778]), ("forward",)]
    ops += [("append", [900] * 8), ("forward",)]
    run_case(ref, "two_level_churn", 2, 8, 4, ops, seed=13)
    # 5. random traces: prefix collisions, exact-prefix inserts, full-chunk tails, removals
    for seed in (0, 1, 2):
        trace = random_trace(seed, n_ops=30, chunk_size=3, vocab=3, max_len=12, max_live=7)
        ops, live = [], 0
        for op, arg in trace:
            ops.append((op, arg))
            live += 1 if op == "add" else (-1 if op == "remove" else 0)
            if live > 0:
                ops.append(("forward",))
        run_case(ref, "random_trace_%d" % seed, 2, 4, 3, ops, seed=20 + seed)


if __name__ == "__main__":
    main()
