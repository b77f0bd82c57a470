"""Configuration of the Llama decoder (field names of the reference's
src/chunk_attn/models/llama_hf/configuration_llama.py:100-191 that the decoder reads)."""
import dataclasses
import json

import torch


@dataclasses.dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = None
    hidden_act: str = "silu"
    max_position_embeddings: int = 10240
    rms_norm_eps: float = 1e-6
    pad_token_id: int = 0
    rope_theta: float = 10000.0
    rope_scaling: dict = None
    # engine side
    use_chunk_attn: bool = True
    chunk_size: int = 64
    chunk_attn_kvcache_gb: float = 0.0  # 0: size the pool from the device's free memory
    torch_dtype: torch.dtype = torch.float16
    torch_device: str = "cuda:0"

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_heads (got `hidden_size`: %d and `num_heads`: %d)."
                             % (self.hidden_size, self.num_attention_heads))
        if self.num_key_value_heads != self.num_attention_heads:
            # the KV chunks are indexed by query head, as in the reference (one K/V head per query head)
            raise NotImplementedError("grouped-query attention is not supported: num_key_value_heads must equal num_attention_heads")
        if self.rope_scaling is not None:
            raise NotImplementedError("rope_scaling is not supported")
        if self.hidden_act != "silu":
            raise NotImplementedError("hidden_act must be silu")

    @classmethod
    def from_dict(cls, d):
        names = {f.name for f in dataclasses.fields(cls)}
        d = {k: v for k, v in d.items() if k in names}
        if isinstance(d.get("torch_dtype"), str):
            d["torch_dtype"] = getattr(torch, d["torch_dtype"])
        return cls(**d)

    @classmethod
    def from_json_file(cls, path):
        with open(path) as f:
            return cls.from_dict(json.load(f))
