"""Helpers of the GPU parity tests: an engine driven purely through the C ABI (ctypes), and the
oracle / dense checkers fed with the same fp16-rounded inputs."""
import numpy as np
import torch

from chunk_attn import PrefixTree, cabi
from chunk_attn_oracle import Attention as OracleAttention, dense_forward

DT = {torch.float16: cabi.CA_DTYPE_F16, torch.float32: cabi.CA_DTYPE_F32}


class CabiEngine:
    """Prefix tree on the host (the compiled PrefixTree) + every device operation through the C ABI:
    ca_scatter_prefill, ca_refresh_kernel_context, ca_append_kv, ca_attention, ca_copy_chunks."""

    def __init__(self, n_heads, d_head, chunk_size, dtype, max_chunks=256, tpp_threshold=1, device=0):
        self.H, self.d, self.C, self.dtype = n_heads, d_head, chunk_size, dtype
        self.device = torch.device("cuda", device)
        nbytes = cabi.lib.ca_chunk_bytes(n_heads, d_head, chunk_size, DT[dtype])
        # fill the pool with NaN patterns: any read of a slot that was never written shows up
        self.pool = torch.full((max_chunks * nbytes,), 0xFF, dtype=torch.uint8, device=self.device)
        self.tree = PrefixTree(chunk_size, max_chunks)
        self.ctx = cabi.Context(n_heads, d_head, chunk_size, DT[dtype], self.pool, max_chunks, tpp_threshold, device)
        self.valid = False

    def add_seq(self, tokens, k, v):
        idx, created = self.tree.add_seq_detailed(list(tokens))
        if created:
            k = k.to(self.device, self.dtype)
            v = v.to(self.device, self.dtype)
            ids = [c[0] for c in created]
            self.ctx.scatter_prefill(k, v, created[0][1], sum(c[2] for c in created), ids)
        self.valid = False
        return idx

    def remove_seq(self, idx):
        self.tree.remove_seq(idx)
        self.valid = False

    def refresh(self, force=False):
        if force or not self.valid:
            self.ctx.refresh(self.tree.get_chunks(), len(self.tree.tails))
            self.valid = True

    def append_token(self, tokens, k, v):
        if self.tree.reserve():
            self.valid = False
        self.refresh()
        self.ctx.append_kv(k.to(self.device, self.dtype).contiguous(), v.to(self.device, self.dtype).contiguous())
        # host token ids (reserve already done: this only records the ids)
        self.tree.append_token(list(tokens))

    def duplicate(self, idx, copies):
        pairs = self.tree.duplicate(idx, copies)
        if pairs:
            self.ctx.copy_chunks([p[0] for p in pairs], [p[1] for p in pairs])
        self.valid = False

    def forward(self, q, partition=0):
        self.refresh()
        q = q.to(self.device, self.dtype).contiguous()
        out = torch.empty_like(q)
        self.ctx.attention(q, out, partition)
        return out


def round_to(x, dtype):
    """fp32 tensor carrying exactly the values the engine sees after the cast to its dtype."""
    return x.to(dtype).to(torch.float32)


def oracle_for(workload, dtype=None):
    """Oracle populated with the workload's values rounded to the engine's dtype."""
    import synthetic_workloads as W
    dtype = dtype or workload.dtype
    ora = OracleAttention(workload.n_heads, workload.d_head, workload.chunk_size)
    rows = []
    for si, segs in enumerate(workload.seqs):
        tokens, k, v = W.cat_segments(segs)
        idx = ora.add_seq(tokens, round_to(k, dtype).cpu().numpy(), round_to(v, dtype).cpu().numpy())
        rows.insert(idx, si)
    return ora, rows


def max_abs(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max())
