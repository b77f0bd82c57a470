"""Profiler range markers for callers of the engine (`nvtx.range_push(name)` / `nvtx.range_pop()`), the module
the reference's model code imports as `chunk_attn.nvtx` (src/chunk_attn/nvtx.py:3-11).  No-ops without CUDA."""
import torch


def _noop(*_args, **_kwargs):
    return None


if torch.cuda.is_available():
    range_push = torch.cuda.nvtx.range_push
    range_pop = torch.cuda.nvtx.range_pop
else:
    range_push = _noop
    range_pop = _noop
