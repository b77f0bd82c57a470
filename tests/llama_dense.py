"""Dense fp32 restatement of the Llama decoder, for checking the chunk-attention decode loop: the
whole sequence is recomputed with full causal attention, no KV cache, plain torch on the CPU or GPU.
Test infrastructure only."""
import torch


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, head_dim, base):
    # x: [T, H, d]; NeoX pairing (i, i + d/2)
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=x.device) / head_dim))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :head_dim // 2], x[..., head_dim // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


@torch.no_grad()
def dense_logits(model, tokens, table=None):
    """[len(tokens), vocab] next-token scores at every position, fp32, from the model's own weights.
    `table`: the model's fp16 cos/sin table; when given, the rotation uses its (rounded) entries so
    that only arithmetic, not the table's rounding, separates the two implementations."""
    cfg = model.config
    sd = {k: v.float() for k, v in model.state_dict().items()}
    dev = sd["lm_head.weight"].device
    H = cfg.num_attention_heads
    d = cfg.hidden_size // H
    ids = torch.tensor(tokens, dtype=torch.long, device=dev)
    pos = torch.arange(len(tokens), device=dev)
    x = sd["model.embed_tokens.weight"][ids]
    T = len(tokens)
    mask = torch.full((T, T), float("-inf"), device=dev).triu(1)
    for i in range(cfg.num_hidden_layers):
        p = "model.layers.%d." % i
        h = _rms(x, sd[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        q = (h @ sd[p + "self_attn.q_proj.weight"].T).view(T, H, d)
        k = (h @ sd[p + "self_attn.k_proj.weight"].T).view(T, H, d)
        v = (h @ sd[p + "self_attn.v_proj.weight"].T).view(T, H, d)
        if table is not None:
            cs = table.float()[pos]
            cos, sin = cs[:, None, :d // 2], cs[:, None, d // 2:]

            def rot(t):
                a, b = t[..., :d // 2], t[..., d // 2:]
                return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
            q, k = rot(q), rot(k)
        else:
            q, k = _rope(q, pos, d, cfg.rope_theta), _rope(k, pos, d, cfg.rope_theta)
        s = torch.einsum("thd,shd->hts", q, k) / d ** 0.5 + mask
        a = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H * d)
        x = x + a @ sd[p + "self_attn.o_proj.weight"].T
        h = _rms(x, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        g = torch.nn.functional.silu(h @ sd[p + "mlp.gate_proj.weight"].T) * (h @ sd[p + "mlp.up_proj.weight"].T)
        x = x + g @ sd[p + "mlp.down_proj.weight"].T
    x = _rms(x, sd["model.norm.weight"], cfg.rms_norm_eps)
    return x @ sd["lm_head.weight"].T
