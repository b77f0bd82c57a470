"""The reference's OWN model layer -- LlamaChunkAttention / LlamaForCausalLM of llama_hf/modeling_llama.py and
ModelHost of model_host.py, the unmodified files -- driving THIS repository's `chunk_attn.Attention` and
`chunk_attn.ops`: prefill through add_seq per row, decode through append_token(fused=True) + forward(q=q),
reserve() + refresh_kernel_context(False) after every layer, remove_seq when a request finishes.  Results are
checked against a dense fp32 recomputation of the same weights.  (The files are installed into oracle/_ref/py by
oracle/build_ref.py; xformers, which they import for the prefill attention, is stood in for by torch's
scaled_dot_product_attention in tests/reference_models.py.)"""
import random

import pytest
import torch

import reference_models as R
from llama_dense import dense_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LOGIT_TOL = 1e-2  # fp16 weights and activations against fp32; observed about 2e-3 on logits of spread 0.3


@pytest.fixture(scope="module")
def ref():
    if not R.available():
        pytest.skip("the reference's model files are not installed under oracle/_ref/py (oracle/build_ref.py installs them)")
    pkg = R.load()   # an import that cannot be satisfied raises here, naming the symbol
    yield pkg
    R.unload()


def make_model(ref, hidden=256, heads=2, layers=2, vocab=512, seed=0):
    from chunk_attn.models.llama_hf import LlamaConfig, LlamaForCausalLM   # the reference's classes
    assert LlamaForCausalLM.__module__ == "chunk_attn.models.llama_hf.modeling_llama"
    assert R.MODELS_DIR in __import__("sys").modules[LlamaForCausalLM.__module__].__file__
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=layers,
                      num_attention_heads=heads, max_position_embeddings=2048, torch_dtype=torch.float16,
                      torch_device=DEV, chunk_attn_kvcache_gb=0.25, pad_token_id=0)
    cfg.rope_scaling = None   # newer transformers fill in a default dict; the reference supports none
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg).to(device=DEV, dtype=torch.float16).eval()
    with torch.no_grad():     # a spread of weights that makes next-token scores distinguishable
        for p in model.parameters():
            if p.dim() == 2:
                p.normal_(0.0, 0.05)
    caches = model.create_kv_caches()
    import chunk_attn
    assert all(type(c) is chunk_attn.Attention and hasattr(c, "plan_stats") for c in caches)   # the B200 engine
    return model, caches


@torch.inference_mode()
def logits_of(model, seqs, caches, prefill):
    hidden = model.model(seqs, caches, prefill)       # what LlamaForCausalLM.forward does, keeping the scores
    return model.lm_head(hidden)[:, -1].float()


def table_of(model):
    return model.model.layers[0].self_attn.rotary_emb.cos_sin_cache


def test_reference_llama_layer_on_this_attention(ref):
    model, caches = make_model(ref)
    Sequence = ref.Sequence
    rnd = random.Random(5)
    shared = [rnd.randrange(1, 512) for _ in range(130)]          # two full chunks and two tokens are common
    # prompts of one prefill batch have the same length (the reference pads a batch to its longest prompt)
    batches = [[shared + [rnd.randrange(1, 512) for _ in range(20)] for _ in range(3)],
               [shared + [rnd.randrange(1, 512) for _ in range(61)] for _ in range(2)]]
    running, logs = [], {}
    for prompts in batches:
        seqs = [Sequence(prompt_tokens=p, max_tokens=100) for p in prompts]
        lg = logits_of(model, seqs, caches, prefill=True)
        for s, row in zip(seqs, lg):
            logs[s.id] = [row.clone()]
            s.append(int(row.argmax()))
        for s in seqs:
            running.insert(s.index, s)                            # add_seq returned the row: the caller inserts there
    for _ in range(70):                                           # every tail crosses a chunk boundary
        lg = logits_of(model, running, caches, prefill=False)
        for s, row in zip(running, lg):
            logs[s.id].append(row.clone())
            s.append(int(row.argmax()))
    worst = 0.0
    for s in running:
        want = dense_logits(model, s.tokens, table_of(model))
        first = len(s.prompt_tokens) - 1
        for j, got in enumerate(logs[s.id]):
            worst = max(worst, (got - want[first + j]).abs().max().item())
    assert worst < LOGIT_TOL, worst
    first_chunk = caches[0].get_trie().children[0]
    assert first_chunk.n_seqs == 5 and first_chunk.n_tokens == 64   # the prefix really is shared by all five
    assert all(c.device_status() == 0 for c in caches)
    assert caches[1].plan_sharing()[1] > 0                          # the layers shared their work lists


def test_reference_model_host_on_this_attention(ref):
    # continuous batching by the reference's ModelHost: requests arrive while others decode, finished ones are
    # removed (remove_seq on every layer's cache), every result must be the greedy continuation of its prompt
    model, caches = make_model(ref, seed=1)
    rnd = random.Random(6)
    shared = [rnd.randrange(1, 512) for _ in range(70)]
    # prompts of equal length: the reference pads a prefill batch to its longest prompt and reads the first new token
    # at the last (padded) position, so it is only right for batches of equal length -- as in its own benchmark
    prompts = [shared + [rnd.randrange(1, 512) for _ in range(20)] for _ in range(8)]
    budgets = [12, 30, 8, 20, 70, 3, 25, 16]
    host = ref.ModelHost(model, caches, max_batch_size=4)
    host.cycle_time = 0.05
    with host:
        handles = [host.predict_async(p, max_tokens=b) for p, b in zip(prompts, budgets)]
        results = [h.get_result() for h in handles]
    assert host.peak_batch_size <= 4
    for p, b, toks in zip(prompts, budgets, results):
        assert toks[:len(p)] == p and len(toks) == len(p) + b
        want = dense_logits(model, toks, table_of(model))
        for pos in range(len(p) - 1, len(toks) - 1):
            # the token the host produced must be the dense model's choice, or tie with it within the tolerance
            top = want[pos].max().item()
            assert want[pos][toks[pos + 1]].item() > top - 2 * LOGIT_TOL, (pos, toks[pos + 1])
    assert all(c.device_status() == 0 for c in caches)
