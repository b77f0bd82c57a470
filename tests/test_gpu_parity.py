"""GPU parity tests (run on the B200 box): the CUDA path against the CPU oracle on identical
seeded inputs, through the C ABI (ctypes) and through the drop-in `Attention` class.

Tolerances: fp16 engine vs oracle on fp16-rounded inputs: max-abs 2e-3 is the stated bar; the
engine accumulates in fp32, so 1e-3 is asserted (and far less is observed).  fp32 engine vs
oracle: max-abs 1e-4.
"""
import math
import os

import numpy as np
import pytest
import torch

from chunk_attn import Attention, cabi
import synthetic_workloads as W
from chunk_attn_oracle import dense_forward
from gpu_helpers import CabiEngine, max_abs, oracle_for, round_to
from ref_loader import load_reference

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3
TOL_F32 = 1e-4


def run_workload(w, engine, partition=0):
    rows = W.populate(engine, w)
    q = w.q[rows]
    out = engine.forward(q, partition).float().cpu().numpy()
    return rows, q, out


def check_against_oracle(w, engine, tol, partitions=(0, 2)):
    ora, orows = oracle_for(w)
    rows = W.populate(engine, w)
    assert rows == orows
    q = round_to(w.q[rows], w.dtype)
    ref = ora.forward(q.numpy(), 0)
    dense = dense_forward(ora, q.numpy())
    assert max_abs(ref, dense) < 1e-5
    for p in partitions:
        out = engine.forward(q, p).float().cpu().numpy()
        assert np.isfinite(out).all()
        assert max_abs(out, ref) < tol, "partition %d" % p
    assert engine.ctx.status() == 0
    return ora, rows


# ---- pool maintenance kernels -----------------------------------------------------------------------
@pytest.mark.parametrize("dtype,H,d,C", [(torch.float16, 3, 128, 64), (torch.float32, 2, 64, 32),
                                         (torch.float32, 2, 4, 2), (torch.float16, 2, 20, 5)])
def test_scatter_append_copy_roundtrip(dtype, H, d, C):
    eng = CabiEngine(H, d, C, dtype, max_chunks=32)
    g = torch.Generator().manual_seed(5)
    n = 2 * C + max(1, C // 3)
    k, v = torch.randn(n, H, d, generator=g), torch.randn(n, H, d, generator=g)
    tokens = list(range(n))
    assert eng.add_seq(tokens, k, v) == 0
    kd, vd = k.to(dtype), v.to(dtype)
    ids = [cid for cid, _, _, _ in sorted(eng.tree.get_chunks(), key=lambda c: c[0])]

    def read(cid, nt):
        ko = torch.empty(H, nt, d, dtype=dtype, device="cuda")
        vo = torch.empty_like(ko)
        eng.ctx.read_chunk(cid, nt, ko, vo)
        return ko.cpu(), vo.cpu()

    for i, cid in enumerate(ids):
        nt = min(C, n - i * C)
        ko, vo = read(cid, nt)
        assert torch.equal(ko, kd[i * C:i * C + nt].transpose(0, 1))
        assert torch.equal(vo, vd[i * C:i * C + nt].transpose(0, 1))
    # append fills the tail slot by slot, across a chunk boundary
    tail_tokens = n - 2 * C
    for step in range(C - tail_tokens + 2):
        nk, nv = torch.randn(1, H, d, generator=g), torch.randn(1, H, d, generator=g)
        eng.append_token([1000 + step], nk, nv)
        tail = eng.tree.tails[0]
        ko, vo = read(tail.id, tail.n_tokens)
        assert torch.equal(ko[:, -1], nk.to(dtype)[0]) and torch.equal(vo[:, -1], nv.to(dtype)[0])
    # copy-on-write clones a whole chunk
    eng.duplicate(0, 2)
    src = eng.tree.tails[0]
    for clone in eng.tree.tails[1:3]:
        a, b = read(src.id, src.n_tokens), read(clone.id, src.n_tokens)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # a strided K/V view (the model passes slices of [batch, tokens, H*d]) lands identically
    big = torch.randn(n, 2 * H, d, generator=g)
    kview = big[:, ::2]
    eng2 = CabiEngine(H, d, C, dtype, max_chunks=16)
    eng2.add_seq(tokens, kview, kview)
    cid0 = min(c[0] for c in eng2.tree.get_chunks())
    ko = torch.empty(H, C, d, dtype=dtype, device="cuda")
    vo = torch.empty_like(ko)
    eng2.ctx.read_chunk(cid0, C, ko, vo)
    assert torch.equal(ko.cpu(), kview.to(dtype)[:C].transpose(0, 1))


# ---- generic (any geometry) kernel -------------------------------------------------------------------
def test_config1_fp32_vs_oracle_and_reference():
    w = W.config1()
    eng = CabiEngine(w.n_heads, w.d_head, w.chunk_size, torch.float32, max_chunks=64)
    ora, rows = check_against_oracle(w, eng, TOL_F32)
    assert eng.ctx.stats()["fast_path"] == 0
    ref = load_reference("cpu")
    if ref is not None:   # the unmodified reference's MKL path on the same inputs
        ra = ref.Attention(n_heads=w.n_heads, d_head=w.d_head, chunk_size=w.chunk_size, memory_mb=64,
                           dtype=torch.float32, device=torch.device("cpu"))
        rrows = W.populate(ra, w)
        assert rrows == rows
        q = w.q[rows]
        out = eng.forward(q).cpu().numpy()
        for p in (0, 2):
            assert max_abs(out, ra.forward(q, p).numpy()) < TOL_F32


@pytest.mark.parametrize("d,C", [(4, 2), (64, 16), (128, 64), (96, 7), (256, 32)])
def test_generic_fp32_shapes(d, C):
    w = W.single_level("t", 2, d, C, torch.float32, 5, 3 * C, C + C // 2 + 1, 11, 1.0)
    eng = CabiEngine(2, d, C, torch.float32, max_chunks=128)
    check_against_oracle(w, eng, TOL_F32)


def test_reference_forward_case_fp32():
    # tests/test_chunk_attn_cpu.py:234-265: two sequences sharing four tokens, chunk_size 2
    H, d = 2, 4
    g = torch.Generator().manual_seed(0)
    k1, v1 = torch.randn(5, H, d, generator=g), torch.randn(5, H, d, generator=g)
    k2, v2 = torch.randn(6, H, d, generator=g), torch.randn(6, H, d, generator=g)
    k2[:4], v2[:4] = k1[:4], v1[:4]
    q = torch.randn(2, H, d, generator=g)
    eng = CabiEngine(H, d, 2, torch.float32, max_chunks=32)
    eng.add_seq([1, 2, 3, 4, 5], k1, v1)
    eng.add_seq([1, 2, 3, 4, 6, 7], k2, v2)
    out = eng.forward(q).cpu()
    for i, (k, v) in enumerate(((k1, v1), (k2, v2))):
        s = torch.einsum("hd,thd->ht", q[i], k) / math.sqrt(d)
        ref = torch.einsum("ht,thd->hd", torch.softmax(s, -1), v)
        assert torch.allclose(out[i], ref, atol=1e-3)   # the reference's own tolerance
        assert max_abs(out[i], ref) < TOL_F32


# ---- tensor-core / TMA path ------------------------------------------------------------------------------
def fast_engine(H=4, max_chunks=512, **kw):
    return CabiEngine(H, 128, 64, torch.float16, max_chunks=max_chunks, **kw)


def test_reference_cuda_test_case():
    # tests/test_chunk_attn_cuda.py:19-72: 32 x 2000 tokens, 1000 shared, H2 d128 chunk 64 fp16
    # (2000 % 64 = 16 exercises tail masking; 1000 % 64 = 40 leaves the last shared chunk private)
    w = W.single_level("refcuda", 2, 128, 64, torch.float16, 32, 1000, 1000, 21, 1.0)
    eng = fast_engine(H=2, max_chunks=32 * 17 + 32)
    check_against_oracle(w, eng, TOL_F16)
    st = eng.ctx.stats()
    assert st["fast_path"] == 1 and st["n_shared_chunks"] == 15


@pytest.mark.parametrize("n_seqs", [1, 2, 3, 15, 16, 17, 33, 64, 70, 130])
def test_sharer_counts(n_seqs):
    w = W.single_level("n%d" % n_seqs, 2, 128, 64, torch.float16, n_seqs, 3 * 64, 64 + 9, 30 + n_seqs, 0.5)
    eng = fast_engine(H=2, max_chunks=3 + n_seqs * 3)
    check_against_oracle(w, eng, TOL_F16)


@pytest.mark.parametrize("tensor_tails", [1, 0])
@pytest.mark.parametrize("unique", [0, 1, 7, 8, 9, 17, 63, 64, 65])
def test_partial_and_empty_tails(unique, tensor_tails):
    # both ways of walking a private tail: tensor cores (default) and CUDA cores
    w = W.single_level("u%d" % unique, 3, 128, 64, torch.float16, 5, 2 * 64, unique, 40 + unique, 0.5)
    eng = fast_engine(H=3)
    eng.ctx.set_option(cabi.CA_OPT_SEQ_FIRST_TENSOR, tensor_tails)
    check_against_oracle(w, eng, TOL_F16)


def test_no_prefix_and_full_prefix():
    for shared, unique in ((0, 5 * 64 + 3), (4 * 64, 0)):
        w = W.single_level("x", 2, 128, 64, torch.float16, 6, shared, unique, 50, 0.5)
        eng = fast_engine(H=2)
        check_against_oracle(w, eng, TOL_F16)


def test_peaky_scores_and_many_pieces():
    # q scaled x8 makes the softmax concentrate: exercises the running max and the merge weights.
    # A small CTA count forces long per-CTA item lists; a large one cuts runs into many pieces.
    w = W.single_level("peaky", 4, 128, 64, torch.float16, 9, 6 * 64, 3 * 64 + 5, 60, 0.5)
    w.q = w.q * 8
    for n_ctas in (1, 5, 148):
        for split, tensor_tails in ((0, 1), (1, 1), (0, 0), (1, 0)):
            eng = fast_engine(H=4)
            eng.ctx.set_option(cabi.CA_OPT_NUM_CTAS, n_ctas)
            eng.ctx.set_option(cabi.CA_OPT_SPLIT_PHASES, split)
            eng.ctx.set_option(cabi.CA_OPT_SEQ_FIRST_TENSOR, tensor_tails)
            check_against_oracle(w, eng, TOL_F16, partitions=(0,))


def test_tpp_threshold_semantics():
    w = W.single_level("tpp", 2, 128, 64, torch.float16, 3, 2 * 64, 10, 70, 0.5)
    eng = fast_engine(H=2, tpp_threshold=3)
    check_against_oracle(w, eng, TOL_F16)
    assert eng.ctx.stats()["n_shared_chunks"] == 0


@pytest.mark.parametrize("tensor_tails", [1, 0])
def test_decode_trace_with_churn(tensor_tails):
    # scaled-down two-level tree with incremental decode: append every step, churn every 4 steps,
    # the oracle mirrors every operation; tails cross chunk boundaries during the trace
    cfg = W.Config4(n_heads=2, n_groups=3, per_group=4, root_len=128, group_len=64, unique_len=60, steps=14,
                    churn_every=4, churn=2)
    from chunk_attn_oracle import Attention as OracleAttention
    eng = fast_engine(H=2, max_chunks=256)
    eng.ctx.set_option(cabi.CA_OPT_SEQ_FIRST_TENSOR, tensor_tails)
    ora = OracleAttention(2, 128, 64)
    seqs = []

    def add(segs):
        tokens, k, v = W.cat_segments(segs)
        i1 = eng.add_seq(tokens, k, v)
        i2 = ora.add_seq(tokens, round_to(k, torch.float16).numpy(), round_to(v, torch.float16).numpy())
        assert i1 == i2
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
        out = eng.forward(qr).float().cpu().numpy()
        worst = max(worst, max_abs(out, ora.forward(qr.numpy(), 0)))
        out2 = eng.forward(qr, 2).float().cpu().numpy()
        worst = max(worst, max_abs(out2, ora.forward(qr.numpy(), 2)))
    assert worst < TOL_F16
    assert eng.ctx.status() == 0


def test_config2_full_size_vs_oracle():
    # the headline configuration at full size; the numpy oracle needs a few seconds for it
    w = W.config2()
    eng = CabiEngine(32, 128, 64, torch.float16, max_chunks=32 + 32 * 9 + 8)
    ora, rows = check_against_oracle(w, eng, TOL_F16)
    st = eng.ctx.stats()
    assert st["unique_kv_bytes"] == 301_989_888 == W.unique_kv_bytes(w)
    assert st["n_shared_chunks"] == 32 and st["n_runs"] == 1 and st["kernels_per_step"] == 2


def test_rows_written_into_peer_outputs():
    # ca_attention_to_peers on one GPU: two local buffers stand in for two ranks' full-width outputs
    w = W.single_level("peers", 4, 128, 64, torch.float16, 9, 3 * 64, 64 + 30, 95, 0.5)
    eng = fast_engine(H=4)
    rows = W.populate(eng, w)
    q = w.q[rows].to("cuda", torch.float16).contiguous()
    expected = eng.forward(q)
    total_heads, head_offset = 12, 4
    peers = [torch.full((9, total_heads, 128), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    eng.ctx.attention_to_peers(q, [p.data_ptr() for p in peers], total_heads, head_offset)
    torch.cuda.synchronize()
    for p in peers:
        assert torch.equal(p[:, head_offset:head_offset + 4], expected)
        assert torch.isnan(p[:, :head_offset]).all() and torch.isnan(p[:, head_offset + 4:]).all()
    with pytest.raises(cabi.CAError):
        eng.ctx.attention_to_peers(q, [peers[0].data_ptr()], 6, 4)   # the slice does not fit in 6 heads


@pytest.mark.parametrize("levels", [1, 2])
def test_tails_kernel_finishes_the_rows(levels):
    # every row has a short private tail: the short-tails kernel runs last, combines each row's partials in registers
    # and stores the output (device buffer, peers' buffers, host memory) -- against the same step with the merge
    # kernel, against the oracle, through appended tokens and with empty tails
    H = 4
    if levels == 1:
        w = W.single_level("fin", H, 128, 64, torch.float16, 40, 5 * 64, 17, 96, 0.5)
    else:   # root + four groups + a few private tokens: five and more partials per row
        gen = torch.Generator().manual_seed(97)
        mk = lambda toks: W.Segment(toks, torch.randn(len(toks), H, 128, generator=gen) * 0.5, torch.randn(len(toks), H, 128, generator=gen) * 0.5)
        root = mk(list(range(7 * 64)))
        groups = [mk([10_000 * (g + 1) + j for j in range(3 * 64)]) for g in range(4)]
        w = W.Workload("fin2", H, 128, 64, torch.float16, 97, 0.5)
        for s in range(44):
            w.seqs.append([root, groups[s % 4], mk([1_000_000 * (s + 1) + j for j in range(1 + s % 9)])])
        w.q = torch.randn(44, H, 128, generator=gen) * 0.5
    eng = fast_engine(H=H, max_chunks=1024)
    eng.ctx.set_option(cabi.CA_OPT_NUM_CTAS, 2)      # few CTAs: the tails are many by comparison and take their own kernel
    ora, orows = oracle_for(w)
    rows = W.populate(eng, w)
    assert rows == orows
    n = len(rows)
    q = w.q[rows].to("cuda", torch.float16).contiguous()
    eng.ctx.set_option(cabi.CA_OPT_FINISH_IN_TAILS, 0)
    merged = eng.forward(q)
    st0 = eng.ctx.stats()
    assert st0["n_items_short"] == n * H
    eng.ctx.set_option(cabi.CA_OPT_FINISH_IN_TAILS, 1)
    out = eng.forward(q)
    assert eng.ctx.stats()["kernels_per_step"] == st0["kernels_per_step"] - 1
    assert (out.float() - merged.float()).abs().max().item() < 5e-4
    ref = ora.forward(round_to(w.q[rows], torch.float16).numpy(), 0)
    assert max_abs(out.float().cpu().numpy(), ref) < TOL_F16
    # into two "ranks'" full-width buffers
    total_heads, head_offset = 12, 4
    peers = [torch.full((n, total_heads, 128), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    eng.ctx.attention_to_peers(q, [p.data_ptr() for p in peers], total_heads, head_offset)
    torch.cuda.synchronize()
    for p in peers:
        assert torch.equal(p[:, head_offset:head_offset + H], out)
        assert torch.isnan(p[:, :head_offset]).all() and torch.isnan(p[:, head_offset + H:]).all()
    # into host memory
    q_host, out_host = q.cpu().pin_memory(), torch.empty(n, H, 128, dtype=torch.float16).pin_memory()
    eng.ctx.attention_host(q_host, out_host)
    assert torch.equal(out_host, out.cpu())
    # appended tokens (the work list is not rebuilt) ...
    g = torch.Generator().manual_seed(98)
    for step in range(3):
        nk, nv = (torch.randn(n, H, 128, generator=g) * 0.5 for _ in range(2))
        eng.append_token([5_000_000 + step] * n, nk, nv)
        ora.append_token([5_000_000 + step] * n, round_to(nk, torch.float16).numpy(), round_to(nv, torch.float16).numpy())
    out = eng.forward(q)
    assert max_abs(out.float().cpu().numpy(), ora.forward(round_to(w.q[rows], torch.float16).numpy(), 0)) < TOL_F16
    assert eng.ctx.status() == 0


# ---- the drop-in class ------------------------------------------------------------------------------------
def test_attention_class_matches_cabi_engine_and_reference_api():
    torch.set_default_dtype(torch.float32)
    w = W.single_level("cls", 4, 128, 64, torch.float16, 7, 3 * 64, 64 + 20, 80, 0.5)
    dev = torch.device("cuda:0")
    attn = Attention(n_heads=4, d_head=128, chunk_size=64, memory_mb=64, dtype=torch.float16, device=dev)
    ora, orows = oracle_for(w)
    rows = W.populate(attn, w, device=dev, dtype=torch.float16)
    assert rows == orows
    q = w.q[rows].to(dev, torch.float16)
    out = attn.forward(q=q)
    assert out.shape == (7, 4, 128) and out.dtype == torch.float16 and out.device == dev
    ref = ora.forward(round_to(w.q[rows], torch.float16).numpy(), 0)
    assert max_abs(out.float().cpu().numpy(), ref) < TOL_F16
    assert max_abs(attn.forward(q=q, partition=2).float().cpu().numpy(), ref) < TOL_F16
    # tree introspection as the reference exposes it
    trie = attn.get_trie()
    assert trie.n_seqs == 7 and len(attn.tails) == 7 and trie.children[0].n_tokens == 64
    assert attn.peak_memory_allocated() > 0
    # append_token returns the freshly reserved chunks; rows keep their order
    nk = torch.randn(7, 4, 128, device=dev, dtype=torch.float16)
    assert attn.append_token(tokens=list(range(7)), k=nk, v=nk, fused=True) == []
    ora.append_token(list(range(7)), nk.float().cpu().numpy(), nk.float().cpu().numpy())
    attn.reserve()
    attn.refresh_kernel_context(force=False)
    out = attn.forward(q=q)
    assert max_abs(out.float().cpu().numpy(), ora.forward(round_to(w.q[rows], torch.float16).numpy(), 0)) < TOL_F16
    # error behaviour of the reference
    with pytest.raises(RuntimeError, match="q is not contiguous"):
        attn.forward(q=q.transpose(0, 1).contiguous().transpose(0, 1))
    with pytest.raises(RuntimeError, match="num of seqs is not equal to num of tokens"):
        attn.append_token(tokens=[1], k=nk[:1], v=nk[:1])
    # a second cache with the same configuration starts empty (one per layer in the model)
    attn2 = Attention(attn)
    assert attn2.get_trie().n_seqs == 0 and attn2.tails == []
    attn.remove_seq(0)
    ora.remove_seq(0)
    out = attn.forward(q=q[1:].contiguous())
    assert max_abs(out.float().cpu().numpy(), ora.forward(round_to(w.q[rows][1:], torch.float16).numpy(), 0)) < TOL_F16
    attn.clear()
    assert attn.tails == [] and attn.forward(q=q[:0].contiguous()).shape == (0, 4, 128)
    assert attn.device_status() == 0
    tiny = Attention(n_heads=32, d_head=128, chunk_size=64, memory_mb=2, dtype=torch.float16, device=dev)
    with pytest.raises(RuntimeError, match="capacity reached"):
        tiny.add_seq(tokens=list(range(200)), k=torch.zeros(200, 32, 128, device=dev, dtype=torch.float16),
                     v=torch.zeros(200, 32, 128, device=dev, dtype=torch.float16))


def test_default_dtype_and_device_resolution():
    # README of the reference: dtype/device default to torch's current defaults
    old = torch.get_default_dtype()
    try:
        torch.set_default_dtype(torch.float16)
        with torch.device("cuda"):
            attn = Attention(n_heads=2, d_head=128, chunk_size=64, memory_mb=8)
            k = torch.randn(70, 2, 128)
            attn.add_seq(tokens=list(range(70)), k=k, v=k)
            out = attn.forward(q=torch.randn(1, 2, 128))
        assert out.dtype == torch.float16 and out.is_cuda
    finally:
        torch.set_default_dtype(old)


# ---- full-size properties where the oracle would take too long ---------------------------------------------
@pytest.mark.parametrize("shared", [0, 1024, 2048, 3072, 4096])
def test_config3_properties(shared):
    # batch 64, context 4096: (a) the tensor-core path and the independent sequence-first kernel
    # agree; (b) sampled (row, head) pairs match dense fp64 attention computed from the inputs;
    # (c) scaling V scales the output (linearity), with K, q unchanged
    w = W.config3(shared, gen_device="cuda")
    dev = torch.device("cuda:0")
    attn = Attention(n_heads=32, d_head=128, chunk_size=64, memory_mb=4700, dtype=torch.float16, device=dev)
    rows = W.populate(attn, w, device=dev, dtype=torch.float16)
    q = w.q[rows].to(dev, torch.float16)
    out = attn.forward(q=q)
    out2 = attn.forward(q=q, partition=2)
    assert torch.isfinite(out).all()
    assert (out.float() - out2.float()).abs().max().item() < TOL_F16
    g = torch.Generator().manual_seed(9)
    for _ in range(6):
        r = int(torch.randint(0, 64, (1,), generator=g))
        h = int(torch.randint(0, 32, (1,), generator=g))
        _, k, v = W.cat_segments(w.seqs[rows[r]], head_slice=slice(h, h + 1))
        k, v = k.half().double()[:, 0], v.half().double()[:, 0]
        s = (k @ q[r, h].double()) / math.sqrt(128)
        ref = torch.softmax(s, 0) @ v
        assert (out[r, h].double() - ref).abs().max().item() < TOL_F16
    assert attn.device_status() == 0


def dense_fp64(segs, head, q_vec, extra_k=None, extra_v=None):
    """softmax(q K^T / sqrt(d)) V in fp64 for one (sequence, head), from the fp16-rounded inputs the engine
    was given: `segs` is the sequence's prefill, extra_k / extra_v the rows appended since (already fp16)."""
    _, k, v = W.cat_segments(segs, head_slice=slice(head, head + 1))
    k, v = k.half().double()[:, 0], v.half().double()[:, 0]
    if extra_k is not None and len(extra_k):
        k = torch.cat([k, torch.stack(extra_k).to(k.device).double()])
        v = torch.cat([v, torch.stack(extra_v).to(v.device).double()])
    s = (k @ q_vec.to(k.device).double()) / math.sqrt(k.shape[1])
    return torch.softmax(s, 0) @ v


def test_config5_full_size_properties():
    # H64, 256 sequences x (4096 shared + 1024 unique): the workload every multi-GPU number is quoted on, on one
    # GPU at full size.  (a) tensor-core path == the independent sequence-first kernel; (b) sampled (row, head)
    # pairs, rows from each 64-row block with the first and the last head plus random ones, against dense fp64.
    w = W.config5(gen_device="cuda")
    H = 64
    eng = CabiEngine(H, 128, 64, torch.float16, max_chunks=64 + 256 * 17 + 8)
    rows = W.populate(eng, w)
    st_rows = sorted(rows)
    assert st_rows == list(range(256))
    q = w.q[rows].to("cuda", torch.float16).contiguous()
    out = eng.forward(q)
    st = eng.ctx.stats()
    assert st["fast_path"] == 1 and st["n_shared_chunks"] == 64 and st["unique_kv_bytes"] == W.unique_kv_bytes(w) == 8_724_152_320
    out2 = eng.forward(q, 2)
    assert torch.isfinite(out).all()
    assert (out.float() - out2.float()).abs().max().item() < TOL_F16
    g = torch.Generator().manual_seed(15)
    pairs = [(64 * b + int(torch.randint(0, 64, (1,), generator=g)), h) for b in range(4) for h in (0, H - 1)]
    pairs += [(int(torch.randint(0, 256, (1,), generator=g)), int(torch.randint(0, H, (1,), generator=g))) for _ in range(8)]
    worst = 0.0
    for r, h in pairs:
        ref = dense_fp64(w.seqs[rows[r]], h, q[r, h])
        worst = max(worst, (out[r, h].double() - ref).abs().max().item())
    assert worst < TOL_F16
    assert eng.ctx.status() == 0


def test_config4_full_size_trace():
    # The two-level tree at full size (H32, 4 groups x 32 sequences, root 1024 + group 1024 + 256 unique), 64 decode
    # steps appending a token per sequence, 8 sequences replaced every 16 steps, then two more steps: the 65th append
    # finds every surviving tail full, so a new tail is reserved.  At the checked steps the tensor-core path must agree
    # with the sequence-first kernel and sampled (row, head) pairs with dense fp64 over prefill + appended rows.
    cfg = W.Config4(gen_device="cuda")
    eng = CabiEngine(32, 128, 64, torch.float16, max_chunks=1100)
    seqs = []      # per row: [segments, appended k rows per head..., appended v rows]

    def add(segs):
        tokens, k, v = W.cat_segments(segs)
        seqs.insert(eng.add_seq(tokens, k, v), {"segs": segs, "k": [], "v": []})

    for segs in cfg.initial():
        add(segs)
    checked, worst, worst_paths = [], 0.0, 0.0
    g = torch.Generator().manual_seed(16)
    n_steps = cfg.steps + 2
    for step in range(n_steps):
        if step and step % cfg.churn_every == 0 and step < cfg.steps:
            for _ in range(cfg.churn):
                i = cfg.rng.randrange(len(seqs))
                eng.remove_seq(i)
                seqs.pop(i)
            for _ in range(cfg.churn):
                add(cfg.new_sequence(cfg.rng.randrange(cfg.n_groups)))
        q, nk, nv = (t.to(torch.float16) for t in cfg.step_inputs(len(seqs)))
        n_chunks_before = len(eng.tree.get_chunks())
        eng.append_token([7_000_000 + step] * len(seqs), nk, nv)
        for i, sq in enumerate(seqs):
            sq["k"].append(nk[i])
            sq["v"].append(nv[i])
        out = eng.forward(q)
        if step == cfg.steps:   # the originals' tails were full: the append before this forward reserved new ones
            assert len(eng.tree.get_chunks()) > n_chunks_before
        if step in (0, 15, 16, 32, 63, cfg.steps, cfg.steps + 1):
            checked.append(step)
            out2 = eng.forward(q, 2)
            assert torch.isfinite(out).all()
            worst_paths = max(worst_paths, (out.float() - out2.float()).abs().max().item())
            for _ in range(6):
                r = int(torch.randint(0, len(seqs), (1,), generator=g))
                h = int(torch.randint(0, 32, (1,), generator=g))
                ref = dense_fp64(seqs[r]["segs"], h, q[r, h], [x[h] for x in seqs[r]["k"]], [x[h] for x in seqs[r]["v"]])
                worst = max(worst, (out[r, h].double() - ref).abs().max().item())
    assert len(checked) == 7
    assert worst_paths < TOL_F16 and worst < TOL_F16
    st = eng.ctx.stats()
    assert st["n_runs"] >= 5   # the root run and the four group runs
    assert eng.ctx.status() == 0


# ---- the reference's own CUDA kernels as comparator ----------------------------------------------------------
def test_against_reference_cuda_kernels():
    ref = load_reference("cuda")
    if ref is None:
        pytest.skip("oracle/_ref/cuda is not built here")
    dev = torch.device("cuda:0")
    w = W.config2(n_heads=8)
    ra = ref.Attention(n_heads=8, d_head=128, chunk_size=64, memory_mb=256, dtype=torch.float16, device=dev)
    attn = Attention(n_heads=8, d_head=128, chunk_size=64, memory_mb=256, dtype=torch.float16, device=dev)
    rows = W.populate(attn, w, device=dev, dtype=torch.float16)
    rrows = W.populate(ra, w, device=dev, dtype=torch.float16)
    assert rows == rrows
    # the reference's chunk-first kernel reads q rows past the batch: hand it the head of a padded buffer
    qbuf = torch.zeros(32 + 160, 8, 128, device=dev, dtype=torch.float16)
    qbuf[:32] = w.q[rows].to(dev, torch.float16)
    q = qbuf[:32]
    out_ref = ra.forward(q)
    torch.cuda.synchronize()
    out = attn.forward(q=q)
    assert (out.float() - out_ref.float()).abs().max().item() < 2e-3


# ---- golden vectors of the unmodified reference ---------------------------------------------------------------
from golden_replay import fixtures, replay  # noqa: E402
from tree_traces import tails_shape, tree_shape  # noqa: E402


@pytest.mark.parametrize("path", fixtures(), ids=lambda p: os.path.basename(p)[:-4])
def test_engine_reproduces_reference_golden_vectors(path):
    # fp32 engine (any-geometry kernel) through the C ABI against outputs of the reference's MKL path
    engines = []

    def make(H, d, C):
        engines.append(CabiEngine(H, d, C, torch.float32, max_chunks=256))
        return engines[-1]

    worst = replay(path, make, tol=TOL_F32, tree_of=lambda e: tree_shape(e.tree.get_trie()),
                   tails_of=lambda e: tails_shape(e.tree.tails), to_input=torch.from_numpy,
                   to_numpy=lambda t: t.float().cpu().numpy())
    assert worst < TOL_F32 and engines[0].ctx.status() == 0
