"""Llama decoder over one `chunk_attn.Attention` per layer.

Call protocol of the reference's decoder (src/chunk_attn/models/llama_hf/modeling_llama.py:184-298):
`model(seqs, kv_caches, prefill) -> [next token per sequence]`, `model.create_kv_caches()`.  Prefill
runs causal attention over the padded prompts and hands each prompt's K/V to `add_seq`, which
returns the row the sequence got; a decode step feeds every running sequence's last token, in row
order, through `append_token` + `forward` of each layer and then `reserve` +
`refresh_kernel_context`, exactly the calls the reference's attention layer makes (lines 78-106).

The decode step is laid out for the GPU rather than as a module-per-op graph: the residual stream
is threaded through `ops.fused_add_rms_norm` (one kernel for add + norm, in place), the rotation
is applied in place by `ops.rotary_embedding`, and projections are plain library GEMMs.  Parameter
names match Hugging Face Llama checkpoints (`model.layers.N.self_attn.q_proj.weight`, ...), so a
state dict of that family loads with `load_state_dict`.
"""
import torch
from torch import nn

import chunk_attn
from chunk_attn import ops

from .configuration_llama import LlamaConfig


def make_cos_sin_cache(rot_dim, max_position, base, dtype, device):
    """[max_position, rot_dim] = [cos | sin] of position * base^(-2i / rot_dim), the table
    `ops.rotary_embedding` reads."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    freqs = torch.outer(torch.arange(max_position, dtype=torch.float32), inv_freq)
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1).to(dtype=dtype, device=device)


class RMSNormWeight(nn.Module):
    """Holds the weight; the normalisation itself is `ops.rms_norm` / `ops.fused_add_rms_norm`."""

    def __init__(self, hidden_size, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x, residual=None):
        """Returns (normalised, residual stream).  With a residual, x += residual happens inside the
        kernel and both tensors are updated in place."""
        if residual is None:
            out = torch.empty_like(x)
            ops.rms_norm(out, x, self.weight.data, self.variance_epsilon)
            return out, x
        ops.fused_add_rms_norm(x, residual, self.weight.data, self.variance_epsilon)
        return x, residual


class LlamaChunkAttention(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.q_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False)
        self.k_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False)
        self.v_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False)
        self.o_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False)

    def qkv(self, hidden_states, positions, cos_sin_cache):
        """hidden_states [..., hidden], positions [...] -> rotated q, k and v as [..., H, d]."""
        q = self.q_proj(hidden_states)
        k = self.k_proj(hidden_states)
        v = self.v_proj(hidden_states)
        ops.rotary_embedding(positions, q, k, self.head_dim, cos_sin_cache, True)
        shape = hidden_states.shape[:-1] + (self.num_heads, self.head_dim)
        return q.view(shape), k.view(shape), v.view(shape)

    def prefill(self, hidden_states, seqs, positions, cos_sin_cache, kv_cache):
        """hidden_states [batch, n_tokens, hidden] (right-padded).  Causal attention inside each
        prompt; then each prompt's own K/V rows go to the cache, which stores only the part no
        earlier sequence has brought."""
        batch, n_tokens, _ = hidden_states.shape
        q, k, v = self.qkv(hidden_states, positions, cos_sin_cache)
        out = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=0.0, is_causal=True)
        out = out.transpose(1, 2).reshape(batch, n_tokens, self.hidden_size)
        if kv_cache is not None:
            for i, seq in enumerate(seqs):
                n = len(seq.tokens)
                seq.index = kv_cache.add_seq(tokens=seq.tokens, k=k[i, :n], v=v[i, :n])
        return self.o_proj(out)

    def decode(self, hidden_states, seqs, positions, cos_sin_cache, kv_cache):
        """hidden_states [n_seqs, hidden], one row per running sequence in cache row order."""
        q, k, v = self.qkv(hidden_states, positions, cos_sin_cache)
        kv_cache.append_token(tokens=[seq[-1] for seq in seqs], k=k, v=v, fused=True)
        out = kv_cache.forward(q=q)  # [n_seqs, H, d]
        return self.o_proj(out.view(-1, self.hidden_size))


class LlamaMLP(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.self_attn = LlamaChunkAttention(config)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = RMSNormWeight(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNormWeight(config.hidden_size, config.rms_norm_eps)

    def forward(self, hidden_states, residual, seqs, positions, cos_sin_cache, kv_cache, prefill):
        hidden_states, residual = self.input_layernorm(hidden_states, residual)
        attn = self.self_attn.prefill if prefill else self.self_attn.decode
        hidden_states = attn(hidden_states, seqs, positions, cos_sin_cache, kv_cache)
        hidden_states, residual = self.post_attention_layernorm(hidden_states, residual)
        hidden_states = self.mlp(hidden_states)
        if kv_cache is not None:
            # a tail that just filled gets its successor now, and the work list follows, so the next
            # layer's (and next step's) append finds room (reference modeling_llama.py:101-106)
            kv_cache.reserve()
            kv_cache.refresh_kernel_context(force=False)
        return hidden_states, residual


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.padding_idx = config.pad_token_id
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNormWeight(config.hidden_size, config.rms_norm_eps)
        self.cos_sin_cache = None

    def _rope_table(self):
        w = self.norm.weight
        if self.cos_sin_cache is None or self.cos_sin_cache.device != w.device or self.cos_sin_cache.dtype != w.dtype:
            head_dim = self.config.hidden_size // self.config.num_attention_heads
            self.cos_sin_cache = make_cos_sin_cache(head_dim, self.config.max_position_embeddings,
                                                    self.config.rope_theta, w.dtype, w.device)
        return self.cos_sin_cache

    def forward(self, seqs, kv_caches, prefill):
        """Returns the final hidden state of each sequence's last real token, [n_seqs, hidden]."""
        device = self.norm.weight.device
        table = self._rope_table()
        if prefill:
            lens = [len(seq) for seq in seqs]
            width = max(lens)
            if width > table.shape[0]:
                raise ValueError("prompt of %d tokens exceeds max_position_embeddings=%d" % (width, table.shape[0]))
            ids = [seq.tokens + [self.padding_idx] * (width - n) for seq, n in zip(seqs, lens)]
            pos = [list(range(n)) + [0] * (width - n) for n in lens]
        else:
            ids = [seq[-1] for seq in seqs]
            pos = [len(seq) - 1 for seq in seqs]
            if max(pos) >= table.shape[0]:
                raise ValueError("sequence exceeds max_position_embeddings=%d" % table.shape[0])
        input_ids = torch.tensor(ids, dtype=torch.long, device=device)
        positions = torch.tensor(pos, dtype=torch.int64, device=device)
        hidden_states = self.embed_tokens(input_ids)
        residual = None
        for i, layer in enumerate(self.layers):
            hidden_states, residual = layer(hidden_states, residual, seqs, positions, table,
                                            kv_caches[i] if kv_caches else None, prefill)
        hidden_states, _ = self.norm(hidden_states, residual)
        if prefill:
            last = torch.tensor([n - 1 for n in lens], dtype=torch.long, device=device)
            hidden_states = hidden_states[torch.arange(len(seqs), device=device), last]
        return hidden_states

    def detect_free_memory(self):
        """MB available for all layers' pools (reference modeling_llama.py:234-247)."""
        if self.config.chunk_attn_kvcache_gb > 0:
            free_mem = self.config.chunk_attn_kvcache_gb * 1024
        else:
            free_b, _total = torch.cuda.mem_get_info(torch.device(self.config.torch_device))
            free_mem = free_b / 1024 / 1024
        return 0.8 * free_mem

    def create_kv_caches(self):
        per_layer = self.detect_free_memory() / len(self.layers)
        first = chunk_attn.Attention(
            n_heads=self.config.num_attention_heads,
            d_head=self.config.hidden_size // self.config.num_attention_heads,
            chunk_size=self.config.chunk_size,
            memory_mb=int(per_layer),
            share_prefix=True,
            tpp_threshold=1,
            dtype=self.config.torch_dtype,
            device=torch.device(self.config.torch_device))
        return [first] + [chunk_attn.Attention(first) for _ in self.layers[1:]]


class LlamaForCausalLM(nn.Module):
    def __init__(self, config: LlamaConfig, seed=None):
        """Weights are left at torch's defaults unless `seed` is given: then every matrix is drawn
        N(0, 0.02²) from a CPU generator (the same values on every machine), norms stay at one."""
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if seed is not None:
            g = torch.Generator(device="cpu").manual_seed(seed)
            with torch.no_grad():
                for name, p in self.named_parameters():
                    if p.dim() >= 2:
                        p.copy_(torch.randn(p.shape, generator=g) * 0.02)
                self.model.embed_tokens.weight[config.pad_token_id].zero_()

    @torch.inference_mode()
    def logits(self, seqs, kv_caches, prefill):
        """[n_seqs, vocab] scores of each sequence's next token."""
        return self.lm_head(self.model(seqs, kv_caches, prefill))

    @torch.inference_mode()
    def forward(self, seqs, kv_caches, prefill):
        return torch.argmax(self.logits(seqs, kv_caches, prefill), dim=-1).tolist()

    def create_kv_caches(self):
        return self.model.create_kv_caches()
