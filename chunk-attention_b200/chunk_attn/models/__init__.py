"""Serving-side callers of the attention engine: `Sequence`, `ModelHost` (continuous batching) and a
Llama decoder that keeps one `chunk_attn.Attention` per layer.  Same module paths and call protocol
as the reference's `chunk_attn.models` (src/chunk_attn/models/model_host.py, sequence.py, llama_hf/)."""
