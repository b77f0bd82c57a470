"""Where the cycles of the tcgen05 kernel for wide shared runs go (diagnostics, run on a B200):
    python tests/wide_cycle_accounting.py
sets CA_OPT_TRACE = 2, runs a few decode steps of three shapes whose shared runs the planner routes to that kernel,
and prints, per K/V tile, the SM cycles of the CTA's two serial roles: the thread that issues the MMAs (issuing,
waiting for P, waiting for the K tile) and a softmax thread (waiting for a score tile, from scores to P)."""
import sys, os
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "chunk-attention_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)
import numpy as np, torch
from chunk_attn import cabi
import synthetic_workloads as W
from gpu_helpers import CabiEngine

def build(name, n_seqs, shared, unique):
    w = W.single_level(name, 32, 128, 64, torch.float16, n_seqs, shared, unique, 2, 0.5, "cuda")
    eng = CabiEngine(32, 128, 64, torch.float16, max_chunks=shared // 64 + 2 * n_seqs + 8)
    rows = W.populate(eng, w)
    q = w.q[rows].to("cuda", torch.float16).contiguous()
    return eng, q


def traced(eng, q, mode):
    eng.ctx.set_option(cabi.CA_OPT_TRACE, mode)
    for _ in range(5):
        eng.forward(q)
    torch.cuda.synchronize()
    return eng.ctx.read_trace().astype(np.int64)


def run(name, n_seqs, shared, unique):
    eng, q = build(name, n_seqs, shared, unique)
    # timeline of a CTA (CA_OPT_TRACE = 1): ns since the first CTA of the launch entered
    tr = traced(eng, q, 1)
    rel = (tr[:, :7] - tr[:, 0].min()) / 1e3
    st = eng.ctx.stats()
    tiles = st["n_items_wide"] and (shared // 64) * ((n_seqs + 127) // 128) * 32 / len(tr)
    print(name, "ctas", len(tr), "tiles/cta %.1f" % tiles, "kernels per step", st["kernels_per_step"])
    print("  timeline, median us (slowest CTA): " + ", ".join(
        "%s %.2f (%.2f)" % (n, np.median(rel[:, i]), rel[:, i].max())
        for i, n in enumerate(["entry", "set-up done", "first S", "last P", "O complete", "rows stored", "exit"])))
    # cycles of the two serial roles (CA_OPT_TRACE = 2)
    tr = traced(eng, q, 2)
    sm = tr[:, 7] >> 48
    tr[:, 7] &= (1 << 48) - 1
    # a CTA had the SM to itself if no other CTA of the launch ran there (one wave: lifetimes overlap)
    alone = np.array([np.sum(sm == x) == 1 for x in sm])
    print("  ctas alone on their SM:", int(alone.sum()))
    for nm, col in (("mma issue QK (8+2)", 2), ("mma issue PV (4+2)", 1), ("mma wait P(+V)", 3), ("mma wait K", 7),
                    ("softmax wait S", 4), ("softmax chain", 5)):
        c = tr[:, col] / tiles
        line = "  %-19s cycles per tile: min %6.0f median %6.0f max %6.0f" % (nm, c.min(), np.median(c), c.max())
        if alone.any() and not alone.all():
            line += "   | alone on the SM: median %6.0f, sharing it: median %6.0f" % (np.median(c[alone]), np.median(c[~alone]))
        print(line)


run("cfg3_s4096", 64, 4096, 0)
run("sys1024", 1024, 2048, 8)
run("sys128", 128, 2048, 8)
