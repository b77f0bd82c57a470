"""Head-sharded decode attention across the GPUs of one node.

Attention heads are independent, so rank r of G owns heads [r*H/G, (r+1)*H/G) of q, k, v, of every
chunk and of the output.  Every rank replays the identical add / append / remove trace on its own
`Attention(n_heads=H/G)`: the prefix tree is replicated and deterministic, so row indices agree
everywhere without any metadata exchange.  The only collective is the optional all-gather of the
[n_seqs, H/G, d] output slices (NCCL over NVLink), followed by the permute to [n_seqs, H, d].
The reference itself is single-device (no torch.distributed anywhere in it).
"""
import torch
import torch.distributed as dist


class HeadShardedAttention:
    def __init__(self, n_heads, d_head, chunk_size, memory_mb=1024, share_prefix=True, tpp_threshold=1,
                 dtype=None, device=None, group=None, attention_factory=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_heads % self.world != 0:
            raise ValueError("n_heads (%d) must divide evenly over %d ranks" % (n_heads, self.world))
        self.n_heads, self.d_head = n_heads, d_head
        self.h_local = n_heads // self.world
        self.head_slice = slice(self.rank * self.h_local, (self.rank + 1) * self.h_local)
        if attention_factory is None:
            from .lib.chunk_attn_c import Attention
            attention_factory = Attention
        self.local = attention_factory(n_heads=self.h_local, d_head=d_head, chunk_size=chunk_size,
                                       memory_mb=memory_mb, share_prefix=share_prefix,
                                       tpp_threshold=tpp_threshold, dtype=dtype, device=device)
        self._gather_buf = None

    def _mine(self, t):
        """Accept full-width [*, H, d] tensors (sliced here) or already-local [*, H/G, d] ones."""
        if t.shape[1] == self.n_heads and self.world > 1:
            return t[:, self.head_slice]
        return t

    def add_seq(self, tokens, k, v):
        return self.local.add_seq(tokens=tokens, k=self._mine(k), v=self._mine(v))

    def append_token(self, tokens, k, v, fused=True):
        return self.local.append_token(tokens=tokens, k=self._mine(k).contiguous(), v=self._mine(v).contiguous(),
                                       fused=fused)

    def remove_seq(self, seq_idx):
        self.local.remove_seq(seq_idx)

    def reserve(self):
        return self.local.reserve()

    def refresh_kernel_context(self, force=False):
        self.local.refresh_kernel_context(force)

    def forward_local(self, q, partition=0):
        return self.local.forward(q=self._mine(q).contiguous(), partition=partition)

    def gather(self, out_local):
        """[n_seqs, H/G, d] on every rank -> [n_seqs, H, d] on every rank."""
        if self.world == 1:
            return out_local
        n = out_local.shape[0]
        shape = (self.world * n, self.h_local, self.d_head)  # rank-major concatenation along dim 0
        if self._gather_buf is None or self._gather_buf.shape != shape or self._gather_buf.dtype != out_local.dtype:
            self._gather_buf = torch.empty(shape, dtype=out_local.dtype, device=out_local.device)
        dist.all_gather_into_tensor(self._gather_buf, out_local.contiguous(), group=self.group)
        return self._gather_buf.view(self.world, n, self.h_local, self.d_head).permute(1, 0, 2, 3).reshape(
            n, self.n_heads, self.d_head)

    def forward(self, q, partition=0, gather=True):
        out = self.forward_local(q, partition)
        return self.gather(out) if gather else out
