"""The Llama decode loop over chunk attention (prefill -> add_seq, decode -> append_token + forward,
per layer) against a dense fp32 recomputation of the same weights, and the continuous-batching host
on the real engine."""
import random

import pytest
import torch

from chunk_attn.models.llama_hf import LlamaConfig, LlamaForCausalLM
from chunk_attn.models.model_host import ModelHost
from chunk_attn.models.sequence import Sequence
from llama_dense import dense_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LOGIT_TOL = 2e-2  # fp16 activations and weights against fp32; logits have a spread of about 0.5


def make_model(hidden=512, heads=4, layers=2, inter=1024, vocab=512, seed=0):
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                      num_attention_heads=heads, max_position_embeddings=1024, chunk_attn_kvcache_gb=0.25,
                      torch_dtype=torch.float16, torch_device=DEV)
    model = LlamaForCausalLM(cfg, seed=seed).to(device=DEV, dtype=torch.float16).eval()
    return model, model.create_kv_caches()


def prompts_with_shared_prefix(rnd, vocab, shared, uniques):
    sys_p = [rnd.randrange(1, vocab) for _ in range(shared)]
    return [sys_p + [rnd.randrange(1, vocab) for _ in range(u)] for u in uniques]


def rows_in_cache_order(seqs):
    """Each prefill returned the row it was inserted at, at that moment: replaying the insertions gives
    the caches' row order (what ModelHost does with its running list)."""
    order = []
    for s in seqs:
        order.insert(s.index, s)
    return order


def check_against_dense(model, seq, step_logits, first_pos):
    """step_logits[j] are the engine's scores at position first_pos + j of seq.tokens."""
    ref = dense_logits(model, seq.tokens, model.model.cos_sin_cache)
    for j, got in enumerate(step_logits):
        want = ref[first_pos + j]
        err = (got.float() - want).abs().max().item()
        assert err < LOGIT_TOL, "position %d: max logit error %g" % (first_pos + j, err)


@pytest.mark.parametrize("hidden,heads", [(512, 4), (256, 4)])  # d_head 128: TMA/tensor-core path; 64: generic kernel
def test_decode_loop_matches_dense(hidden, heads):
    model, caches = make_model(hidden=hidden, heads=heads)
    rnd = random.Random(1)
    # shared 130 tokens (2 full chunks + 2), tails of different fill; one unrelated prompt of exactly one chunk
    prompts = prompts_with_shared_prefix(rnd, 512, 130, [5, 70, 1]) + [[rnd.randrange(1, 512) for _ in range(64)]]
    seqs = [Sequence(p, max_tokens=80) for p in prompts]
    logs = {s.id: [] for s in seqs}
    lg = model.logits(seqs, caches, prefill=True)
    # rows come back in cache (DFS) order from now on
    for s, row in zip(seqs, lg):
        logs[s.id].append(row.clone())
        s.append(int(row.argmax()))
    running = rows_in_cache_order(seqs)
    for _ in range(70):  # crosses a chunk boundary for every sequence
        lg = model.logits(running, caches, prefill=False)
        for s, row in zip(running, lg):
            logs[s.id].append(row.clone())
            s.append(int(row.argmax()))
    for s in seqs:
        check_against_dense(model, s, logs[s.id], len(s.prompt_tokens) - 1)
    first = caches[0].get_trie().children[0]
    assert first.n_seqs == 3 and first.n_tokens == 64  # the 130-token prefix really is shared
    assert all(c.device_status() == 0 for c in caches)


def test_prefix_sharing_does_not_change_the_scores():
    """The same prompts through a sharing cache and through share_prefix=False caches."""
    import chunk_attn
    model, caches = make_model()
    cfg = model.config
    plain = [chunk_attn.Attention(n_heads=4, d_head=128, chunk_size=64, memory_mb=64, share_prefix=False,
                                  dtype=torch.float16, device=torch.device(DEV)) for _ in range(cfg.num_hidden_layers)]
    rnd = random.Random(2)
    prompts = prompts_with_shared_prefix(rnd, 512, 192, [3, 40])
    outs = []
    for kv in (caches, plain):
        seqs = [Sequence(p) for p in prompts]
        toks = model(seqs, kv, prefill=True)
        for s, t in zip(seqs, toks):
            s.append(t)
        run = rows_in_cache_order(seqs)
        rows = []
        for _ in range(5):
            lg = model.logits(run, kv, prefill=False)
            rows.append(torch.stack([lg[run.index(s)] for s in seqs]))
            for s, row in zip(run, lg):
                s.append(int(row.argmax()))
        outs.append(torch.stack(rows))
    assert caches[0].plan_stats()["n_shared_chunks"] == 3 and plain[0].plan_stats()["n_shared_chunks"] == 0
    torch.testing.assert_close(outs[0], outs[1], atol=5e-3, rtol=0)


def test_model_host_on_the_engine():
    model, caches = make_model()
    rnd = random.Random(3)
    prompts = prompts_with_shared_prefix(rnd, 512, 100, [4, 30, 64, 9, 1, 17]) + \
        [[rnd.randrange(1, 512) for _ in range(20)]]
    lens = [12, 40, 7, 70, 25, 1, 33]
    host = ModelHost(model, caches, max_batch_size=4)
    host.cycle_time = 0.05
    with host:
        pending = [host.predict_async(p, n) for p, n in zip(prompts[:4], lens[:4])]
        pending[2].get_result(timeout=120)
        pending += [host.predict_async(p, n) for p, n in zip(prompts[4:], lens[4:])]
        results = [s.get_result(timeout=120) for s in pending]
    assert host.peak_batch_size <= 4 and host.peak_batch_size >= 2
    for p, n, toks in zip(prompts, lens, results):
        assert toks[:len(p)] == p and len(toks) == len(p) + n
        ref = dense_logits(model, toks, model.model.cos_sin_cache)
        for t in range(len(p) - 1, len(toks) - 1):
            # greedy: the token chosen must be the dense argmax up to the engine's fp16 error
            assert ref[t, toks[t + 1]] >= ref[t].max() - 2 * LOGIT_TOL
    assert all(len(c.get_trie().children) == 0 for c in caches)  # everything was retired
    assert all(c.device_status() == 0 for c in caches)


def test_ragged_prefill_ignores_padding():
    """A short prompt prefilled next to a long one gets the scores it gets alone."""
    model, caches = make_model(layers=1)
    rnd = random.Random(5)
    short = [rnd.randrange(1, 512) for _ in range(7)]
    long = [rnd.randrange(1, 512) for _ in range(150)]
    both = model.logits([Sequence(short), Sequence(long)], None, prefill=True)
    alone = model.logits([Sequence(short)], None, prefill=True)
    torch.testing.assert_close(both[0], alone[0], atol=2e-3, rtol=0)
    ref = dense_logits(model, short, model.model.cos_sin_cache)[-1]
    assert (both[0].float() - ref).abs().max().item() < LOGIT_TOL


def test_layers_share_their_work_lists():
    """Caches made with Attention(other) plan once per tree change: the first layer to refresh builds the
    work list, the others find their chunk lists identical and only upload it."""
    import chunk_attn
    first = chunk_attn.Attention(n_heads=4, d_head=128, chunk_size=64, memory_mb=32, dtype=torch.float16,
                                 device=torch.device(DEV))
    layers = [first] + [chunk_attn.Attention(first) for _ in range(3)]
    alone = chunk_attn.Attention(n_heads=4, d_head=128, chunk_size=64, memory_mb=32, dtype=torch.float16,
                                 device=torch.device(DEV))
    g = torch.Generator().manual_seed(0)
    shared = list(range(130))
    ks = [torch.randn(140, 4, 128, generator=g).half().to(DEV) for _ in range(5)]  # one K/V set per cache
    for s in range(3):
        toks = shared + [1000 * (s + 1) + j for j in range(10)]
        for c, k in zip(layers + [alone], ks):
            c.add_seq(tokens=toks, k=k, v=k)
    q = torch.randn(3, 4, 128, generator=g).half().to(DEV)
    outs = [c.forward(q=q) for c in layers]
    assert first.plan_sharing() == (1, 3)          # built once, reused by the three other layers
    assert alone.plan_sharing() == (0, 0) and alone.forward(q=q) is not None and alone.plan_sharing() == (1, 0)
    # every layer computed with its own K/V: same values as a cache that planned for itself
    for c, k, o in zip(layers, ks, outs):
        solo = chunk_attn.Attention(n_heads=4, d_head=128, chunk_size=64, memory_mb=32, dtype=torch.float16,
                                    device=torch.device(DEV))
        for s in range(3):
            solo.add_seq(tokens=shared + [1000 * (s + 1) + j for j in range(10)], k=k, v=k)
        assert torch.equal(solo.forward(q=q), o)
    # a decode step does not touch the tree shape: no new plan; filling the tails (64 steps later) makes one
    nk = torch.randn(3, 4, 128, generator=g).half().to(DEV)
    for c in layers:
        c.append_token(tokens=[7, 8, 9], k=nk, v=nk)
        c.forward(q=q)
    assert first.plan_sharing() == (1, 3)
    # a cache whose options change plans for itself from then on
    layers[2].set_option(chunk_attn.cabi.CA_OPT_SEQ_FIRST_TENSOR, 0)
    for c in layers:
        c.remove_seq(0)
        c.forward(q=q[1:].contiguous())
    assert layers[2].plan_sharing() == (1, 0)
    assert first.plan_sharing() == (2, 5)
