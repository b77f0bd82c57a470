"""Replay a golden fixture (tests/golden/*.npz, produced from the unmodified reference by
tests/golden/make_golden.py) on any engine with the add_seq / remove_seq / append_token / forward
surface, checking rows, tree shape, `tails` order and forward outputs step by step."""
import glob
import json
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def fixtures():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def listify(x):
    """JSON turns tuples into lists: compare tree shapes in list form."""
    if isinstance(x, (list, tuple)):
        return [listify(y) for y in x]
    return x


def replay(path, make_engine, tol, tree_of=None, tails_of=None, to_input=lambda a: a, to_numpy=np.asarray,
           partitions=(0, 2)):
    """make_engine(n_heads, d_head, chunk_size) -> engine.  Returns the worst forward error seen."""
    data = np.load(path)
    meta = json.loads(str(data["meta"]))
    eng = make_engine(meta["n_heads"], meta["d_head"], meta["chunk_size"])
    worst = 0.0
    for i, rec in enumerate(meta["log"]):
        op = rec["op"]
        if op == "add":
            row = eng.add_seq(rec["tokens"], to_input(data["k%d" % i]), to_input(data["v%d" % i]))
            assert row == rec["row"], (path, i, row, rec["row"])
        elif op == "remove":
            eng.remove_seq(rec["row"])
        elif op == "append":
            eng.append_token(rec["tokens"], to_input(data["k%d" % i]), to_input(data["v%d" % i]))
        elif op == "forward":
            for part in partitions:
                out = to_numpy(eng.forward(to_input(data["q%d" % i]), part))
                err = float(np.abs(out.astype(np.float64) - data["out%d_%d" % (part, i)]).max())
                assert err < tol, (path, i, part, err)
                worst = max(worst, err)
        if tree_of is not None:
            assert listify(tree_of(eng)) == rec["tree"], (path, i)
        if tails_of is not None:
            assert listify(tails_of(eng)) == rec["tails"], (path, i)
    return worst
