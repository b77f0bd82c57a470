"""Head-sharded decode attention across the GPUs of one node.

Attention heads are independent, so rank r of G owns heads [r*H/G, (r+1)*H/G) of q, k, v, of every
chunk and of the output.  Every rank replays the identical add / append / remove trace on its own
`Attention(n_heads=H/G)`: the prefix tree is replicated and deterministic, so row indices agree
everywhere without any metadata exchange.  The only exchange is the optional gather of the [n_seqs, H/G, d] output slices into [n_seqs, H, d]
on every rank, in one of two ways:
  gather="nccl"  all_gather_into_tensor (NCCL over NVLink) followed by a permute;
  gather="p2p"   the merge kernel itself stores every output row into each rank's full-width buffer
                 (symmetric memory; one multimem.st per row segment that the NVSwitch replicates when a multicast
                 mapping exists, else plain peer stores over NVLink), followed by one barrier on the stream:
                 compute and gather in a single kernel, no collective call and no permute.  The barrier is this
                 library's own kernel (ca_peer_barrier): a release store of the step number into every peer's flag
                 array and a wait on one's own, BOUNDED -- a peer that never arrives costs the time limit and a
                 status code (`barrier_status()`), never a hung GPU.
The reference itself is single-device (no torch.distributed anywhere in it).
"""
import time

import torch
import torch.distributed as dist


class PeerLost(RuntimeError):
    """A rank of the group left, or did not reach the step within the time allowed.  Raised on the HOST, before
    anything of the step is launched, so no kernel or collective is left waiting for the missing rank."""


class HeadShardedAttention:
    def __init__(self, n_heads, d_head, chunk_size, memory_mb=1024, share_prefix=True, tpp_threshold=1,
                 dtype=None, device=None, group=None, attention_factory=None, gather="nccl", barrier="own",
                 multicast=True, barrier_timeout_s=2.0):
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
        if gather not in ("nccl", "p2p"):
            raise ValueError("gather must be 'nccl' or 'p2p'")
        self.gather_mode = gather if self.world > 1 else "nccl"
        self._symm = None      # (tensor [rows, H, d], handle, peer pointers)
        if barrier not in ("own", "torch"):
            raise ValueError("barrier must be 'own' (bounded, this library's kernel) or 'torch' (symmetric-memory barrier)")
        self.barrier_kind = barrier
        self.use_multicast = multicast
        self.barrier_timeout_ns = int(barrier_timeout_s * 1e9)
        self._flags = None     # (flag tensor, handle, peer pointers) of the own barrier
        self._epoch = 0
        self._status = None
        # host-side liveness check (off unless check_peers / peer_timeout_s is used)
        self.peer_timeout_s = None
        self._hb_store = None
        self._hb_step = 0
        self._hb_prefix = "ca_hb"

    # ---- failure detection: on the host, between steps -----------------------------------------------------
    def enable_peer_check(self, timeout_s, store=None, prefix="ca_hb"):
        """From now on every forward() first makes sure, through the process group's key-value store, that all
        ranks have reached the same step and that none has left; a missing rank raises PeerLost after
        `timeout_s` instead of leaving this rank's kernels (or its next collective) waiting on the device.
        Costs one store round trip per step, so it is meant for serving loops where a step is milliseconds."""
        if self.world == 1:
            return
        self._hb_store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.peer_timeout_s = float(timeout_s)
        self._hb_prefix = prefix
        self._hb_step = 0

    def check_peers(self):
        """One liveness round (called by forward() when enabled): announce this rank's arrival at the step, then
        wait until every rank has arrived.  Raises PeerLost when a rank has announced its departure with leave()
        or when the wait runs out."""
        if self._hb_store is None:
            return
        st, step = self._hb_store, self._hb_step
        self._hb_step += 1
        key = "%s/step/%d" % (self._hb_prefix, step)
        st.add(key, 1)
        deadline = time.monotonic() + self.peer_timeout_s
        while True:
            if st.add("%s/left" % self._hb_prefix, 0) > 0:
                raise PeerLost("a rank left the group before step %d" % step)
            arrived = st.add(key, 0)
            if arrived >= self.world:
                return
            if time.monotonic() > deadline:
                raise PeerLost("only %d of %d ranks reached step %d within %.1f s" %
                               (arrived, self.world, step, self.peer_timeout_s))
            time.sleep(0.0005)

    def leave(self):
        """Announce that this rank stops taking part.  Call it between steps, with none of this rank's kernels or
        collectives in flight; the other ranks learn of it at their next check_peers()."""
        if self._hb_store is not None:
            self._hb_store.add("%s/left" % self._hb_prefix, 1)

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

    def _symm_buffers(self, n_rows, dtype, device):
        """Two full-width output buffers in symmetric memory, used alternately, grown to the largest
        batch seen (a collective: every rank reaches this at the same step because the trees are
        replicated)."""
        if self._symm is None or self._symm[0][0].shape[0] < n_rows:
            import torch.distributed._symmetric_memory as symm_mem
            rows = max(n_rows, 64)
            group = self.group if self.group is not None else dist.group.WORLD
            bufs = []
            for _ in range(2):
                buf = symm_mem.empty((rows, self.n_heads, self.d_head), dtype=dtype, device=device)
                hdl = symm_mem.rendezvous(buf, group)
                mc = 0
                if self.use_multicast:
                    try:
                        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
                    except Exception:
                        mc = 0
                bufs.append((buf, hdl, [int(p) for p in hdl.buffer_ptrs], mc))
            self._symm = bufs
            self._step = 0
            if self._flags is None:
                flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
                flags.zero_()
                fh = symm_mem.rendezvous(flags, group)
                self._flags = (flags, fh, [int(p) for p in fh.buffer_ptrs])
                self._status = torch.zeros(1, dtype=torch.int32, device=device)
                torch.cuda.synchronize(device)
                fh.barrier(channel=0)   # once, at set-up: nobody signals before every array is zero
                torch.cuda.synchronize(device)
        return self._symm

    def multicast_in_use(self):
        return bool(self._symm and self._symm[0][3])

    def _barrier(self, hdl):
        if self.barrier_kind == "torch":
            hdl.barrier(channel=0)
            return
        from . import cabi
        self._epoch += 1
        cabi.peer_barrier(self._flags[2], self.rank, self._epoch, self.barrier_timeout_ns, self._status.data_ptr())

    def barrier_status(self):
        """0, or 6 when a barrier of this object gave up waiting for a peer (synchronises)."""
        return int(self._status.item()) if self._status is not None else 0

    def forward(self, q, partition=0, gather=True):
        """Attention of this rank's head slice; with gather=True the full-width [n_seqs, H, d] result on every rank.
        The gathered tensor is a view of a buffer this object reuses: with gather="nccl" it is overwritten by the
        next forward(), with gather="p2p" by the next-but-one (two buffers alternate and peers store into them),
        and it is only ordered against work on the stream forward() was called on.  Clone it to keep it."""
        if gather:
            self.check_peers()
        if gather and self.gather_mode == "p2p" and partition != 2:
            ql = self._mine(q).contiguous()
            # Buffer k & 1 for step k.  When a rank passes the barrier of step k + 1, every rank's stream
            # has passed its reads of step k's buffer, so step k + 2 may overwrite it without a barrier
            # of its own: one barrier per step.
            buf, hdl, ptrs, mc = self._symm_buffers(ql.shape[0], ql.dtype, ql.device)[self._step & 1]
            self._step += 1
            self.local.forward_to_peers(q=ql, peer_out_ptrs=ptrs, total_heads=self.n_heads,
                                        head_offset=self.rank * self.h_local, multicast_ptr=mc)
            self._barrier(hdl)       # every rank's rows have landed everywhere
            return buf[:ql.shape[0]]
        out = self.forward_local(q, partition)
        return self.gather(out) if gather else out
