"""The tcgen05 / TMEM kernel for wide shared runs (tensor memory accumulators, MMAs fed by shared-memory
descriptors straight from the staged K/V tiles) against the CPU oracle, dense fp64 and the independent
sequence-first kernel, with the routing forced on (every shared run) and left to the planner."""
import math

import pytest
import torch

from chunk_attn import Attention, cabi
import synthetic_workloads as W
from gpu_helpers import CabiEngine, max_abs, oracle_for, round_to

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3


def wide_engine(H, max_chunks, mode=2, **kw):
    eng = CabiEngine(H, 128, 64, torch.float16, max_chunks=max_chunks, **kw)
    eng.ctx.set_option(cabi.CA_OPT_WIDE_RUNS, mode)
    return eng


def check_vs_oracle(w, eng, tol=TOL_F16):
    ora, orows = oracle_for(w)
    rows = W.populate(eng, w)
    assert rows == orows
    q = round_to(w.q[rows], w.dtype)
    ref = ora.forward(q.numpy(), 0)
    out = eng.forward(q).float().cpu().numpy()
    assert torch.isfinite(torch.from_numpy(out)).all()
    assert max_abs(out, ref) < tol
    assert eng.ctx.status() == 0
    return eng.ctx.stats()


@pytest.mark.parametrize("n_seqs", [2, 3, 16, 17, 33, 64, 70, 128, 130, 260])
def test_wide_sharer_counts(n_seqs):
    # every shared run forced onto the wide kernel: one row block up to 128 rows, several above
    w = W.single_level("wn%d" % n_seqs, 2, 128, 64, torch.float16, n_seqs, 3 * 64, 64 + 9, 300 + n_seqs, 0.5)
    st = check_vs_oracle(w, wide_engine(2, 3 + n_seqs * 3))
    assert st["n_items_wide"] > 0 and st["n_items_cf"] == 0


@pytest.mark.parametrize("n_ctas", [1, 296])
def test_wide_long_run_rising_scores(n_ctas):
    # 40 shared chunks: pieces of up to 32 tiles (one CTA) or about a wave of short pieces; the keys grow along the
    # prefix and the queries are large, so row maxima keep rising from tile to tile and the accumulator in tensor
    # memory is rescaled on the way
    H, n_seqs, shared = 2, 20, 40 * 64
    w = W.single_level("rise", H, 128, 64, torch.float16, n_seqs, shared, 7, 411, 0.5)
    ramp = torch.linspace(0.2, 2.0, shared).view(-1, 1, 1)
    w.seqs[0][0].k.mul_(ramp)          # the shared segment is one object referenced by every sequence
    w.q = w.q * 6
    eng = wide_engine(H, 40 + n_seqs * 2 + 4)
    eng.ctx.set_option(cabi.CA_OPT_NUM_CTAS, n_ctas)
    st = check_vs_oracle(w, eng)
    assert st["n_items_wide"] == (2 * H if n_ctas == 1 else st["n_items_wide"]) and st["n_items_wide"] >= 2 * H


def test_wide_two_level_tree_with_decode():
    # root prefix over 150 rows (two row blocks), two groups below it, private tails; tokens appended without a rebuild
    cfg = W.Config4(n_heads=2, n_groups=2, per_group=75, root_len=6 * 64, group_len=2 * 64, unique_len=30, steps=6,
                    churn_every=3, churn=5)
    from chunk_attn_oracle import Attention as OracleAttention
    eng = wide_engine(2, 700)
    ora = OracleAttention(2, 128, 64)
    seqs = []

    def add(segs):
        tokens, k, v = W.cat_segments(segs)
        i1 = eng.add_seq(tokens, k, v)
        assert i1 == ora.add_seq(tokens, round_to(k, torch.float16).numpy(), round_to(v, torch.float16).numpy())
        seqs.insert(i1, segs)

    for segs in cfg.initial():
        add(segs)
    worst = 0.0
    for step in range(cfg.steps):
        if step and step % cfg.churn_every == 0:
            for _ in range(cfg.churn):
                i = cfg.rng.randrange(len(seqs))
                eng.remove_seq(i)
                ora.remove_seq(i)
                seqs.pop(i)
            for _ in range(cfg.churn):
                add(cfg.new_sequence(cfg.rng.randrange(cfg.n_groups)))
        q, nk, nv = cfg.step_inputs(len(seqs))
        toks = [7_000_000 + step] * len(seqs)
        eng.append_token(toks, nk, nv)
        ora.append_token(toks, round_to(nk, torch.float16).numpy(), round_to(nv, torch.float16).numpy())
        qr = round_to(q, torch.float16)
        worst = max(worst, max_abs(eng.forward(qr).float().cpu().numpy(), ora.forward(qr.numpy(), 0)))
    assert worst < TOL_F16
    assert eng.ctx.stats()["n_items_wide"] > 0 and eng.ctx.status() == 0


def dense_rows(w, rows, out, q, pairs):
    worst = 0.0
    for r, h in pairs:
        _, k, v = W.cat_segments(w.seqs[rows[r]], head_slice=slice(h, h + 1))
        k, v = k.half().double()[:, 0], v.half().double()[:, 0]
        s = (k @ q[r, h].double()) / math.sqrt(128)
        worst = max(worst, (out[r, h].double() - torch.softmax(s, 0) @ v).abs().max().item())
    return worst


def test_fully_shared_batch_is_routed_by_the_planner():
    # configuration 3 at s = 4096 (64 identical contexts, K/V resident in L2): the step is bound by the contraction,
    # so the planner itself sends the run to the tensor-memory kernel
    w = W.config3(4096, gen_device="cuda")
    dev = torch.device("cuda:0")
    attn = Attention(n_heads=32, d_head=128, chunk_size=64, memory_mb=200, dtype=torch.float16, device=dev)
    rows = W.populate(attn, w, device=dev, dtype=torch.float16)
    q = w.q[rows].to(dev, torch.float16)
    out = attn.forward(q=q)
    st = attn.plan_stats()
    assert st["n_items_wide"] > 0 and st["n_items_cf"] == 0
    gen = attn.forward(q=q, partition=2)
    assert (out.float() - gen.float()).abs().max().item() < TOL_F16
    g = torch.Generator().manual_seed(3)
    pairs = [(int(torch.randint(0, 64, (1,), generator=g)), int(torch.randint(0, 32, (1,), generator=g))) for _ in range(8)]
    assert dense_rows(w, rows, out, q, pairs) < TOL_F16
    attn.set_option(cabi.CA_OPT_WIDE_RUNS, 0)       # the mma.sync walk of the same work
    out0 = attn.forward(q=q)
    assert attn.plan_stats()["n_items_wide"] == 0
    assert (out.float() - out0.float()).abs().max().item() < TOL_F16
    assert attn.device_status() == 0


def test_many_requests_over_one_system_prompt():
    # 1024 requests over a 2048-token prompt with 8-token suffixes (H8 to keep the test small): eight row blocks per head
    # on the wide kernel, the suffixes on the warp-per-item kernel, nothing left for the persistent kernel
    dev = torch.device("cuda:0")
    w = W.single_level("sys", 8, 128, 64, torch.float16, 1024, 2048, 8, 77, 0.5, gen_device="cuda")
    attn = Attention(n_heads=8, d_head=128, chunk_size=64, memory_mb=400, dtype=torch.float16, device=dev)
    rows = W.populate(attn, w, device=dev, dtype=torch.float16)
    q = w.q[rows].to(dev, torch.float16)
    out = attn.forward(q=q)
    st = attn.plan_stats()
    # 8 row blocks x 8 heads, each cut into as many pieces as fill one wave of CTAs
    assert st["n_items_wide"] > 0 and st["n_items_wide"] % 64 == 0 and st["n_items_cf"] == 0
    # ... and the short-tails kernel, last in the step, stores the output rows itself: no merge launch
    assert st["n_items_short"] == 1024 * 8 and st["kernels_per_step"] == 2
    gen = attn.forward(q=q, partition=2)
    assert (out.float() - gen.float()).abs().max().item() < TOL_F16
    g = torch.Generator().manual_seed(4)
    pairs = [(int(torch.randint(0, 1024, (1,), generator=g)), int(torch.randint(0, 8, (1,), generator=g))) for _ in range(8)]
    assert dense_rows(w, rows, out, q, pairs) < TOL_F16
    attn.set_option(cabi.CA_OPT_FINISH_IN_TAILS, 0)      # the same step with partial rows for the tails and the merge kernel
    out3 = attn.forward(q=q)
    assert attn.plan_stats()["kernels_per_step"] == 3
    assert (out.float() - out3.float()).abs().max().item() < 5e-4
    assert attn.device_status() == 0


def test_cycle_accounting_trace_mode_computes_the_same_rows():
    # CA_OPT_TRACE = 2 runs the instantiation of the wide kernel that accounts for the cycles of its serial roles;
    # the rows it computes are the same, and every CTA reports time spent issuing MMAs and in the softmax chain
    # (100 identical contexts and few CTAs: the whole step is one shared run and the empty private tails are short
    # items that cost no launch, so the trace read back is the wide kernel's)
    w = W.single_level("acct", 4, 128, 64, torch.float16, 100, 16 * 64, 0, 21, 0.5, gen_device="cuda")
    eng = CabiEngine(4, 128, 64, torch.float16, max_chunks=16 + 2 * 100 + 8)
    rows = W.populate(eng, w)
    q = w.q[rows].to("cuda", torch.float16).contiguous()
    eng.ctx.set_option(cabi.CA_OPT_WIDE_RUNS, 2)
    eng.ctx.set_option(cabi.CA_OPT_NUM_CTAS, 8)
    plain = eng.forward(q).clone()
    eng.ctx.set_option(cabi.CA_OPT_TRACE, 2)
    traced = eng.forward(q)
    assert torch.equal(plain, traced)
    tr = eng.ctx.read_trace().astype("int64")
    st = eng.ctx.stats()
    assert st["n_items_wide"] > 0 and st["n_items_wide"] + st["n_items_short"] == st["n_items"]
    assert len(tr) == st["n_items_wide"]
    assert len(tr) > 0 and (tr[:, 2] > 0).all() and (tr[:, 5] > 0).all() and (tr[:, 6] > tr[:, 0]).all()
    with pytest.raises(RuntimeError):
        eng.ctx.set_option(cabi.CA_OPT_TRACE, 3)
    eng.ctx.set_option(cabi.CA_OPT_TRACE, 0)
    assert eng.ctx.status() == 0
