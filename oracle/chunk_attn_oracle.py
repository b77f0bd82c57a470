"""CPU oracle for the ChunkAttention decode path: TEST INFRASTRUCTURE ONLY.

This module restates, in numpy float32, the algorithm of the reference's host prefix tree and
of its CPU (MKL) attention kernels.  It exists so that the CUDA engine can be checked against
an independent implementation; only the tests, the smoke check and the benchmark's CPU-baseline
leg may import it.  The shipped engine never does, and has no CPU fallback.

Parity status: PINNED.  The restatement is checked against (a) the unmodified reference built
from its own sources into oracle/_ref (oracle/build_ref.py) wherever that build is present, and
(b) golden vectors produced by that build and committed under tests/golden/ (generator:
tests/golden/make_golden.py), plus the exact tree-shape assertions of the reference's own unit
tests (tests/test_chunk_attn_cpu.py:24-215,267-303).

Every function cites the reference source it follows as  path:line  within the reference tree.
"""
import heapq
import math

import numpy as np

F32_LOWEST = np.float32(np.finfo(np.float32).min)  # std::numeric_limits<float>::lowest()


class Chunk:
    """Prefix-tree node holding up to `capacity` tokens (cpp/chunk_attn/chunk.h:9-65).

    K and V are stored head-major, [n_heads, capacity, d_head], as the reference's chunk views
    are (cpp/chunk_attn/chunk_allocator.cpp:46-50).
    """

    def __init__(self, capacity, n_heads, d_head, id=-1):
        self.capacity = capacity
        self.id = id                          # pool slot (the reference names chunks by address)
        self.tokens = []
        self.children = []
        self.parent = None
        self.n_seqs = 1                       # chunk.cpp:21
        self.k = np.zeros((n_heads, capacity, d_head), np.float32)
        self.v = np.zeros((n_heads, capacity, d_head), np.float32)

    @property
    def n_tokens(self):
        return len(self.tokens)

    def full(self):                           # chunk.h:26
        return len(self.tokens) == self.capacity

    def equal(self, ids, start, end):         # chunk.cpp:51-62
        n = end - start
        if self.n_tokens != n or end > len(ids):
            return False
        return self.tokens == list(ids[start:end])

    def append_tokens(self, ids, k, v, start, end):
        """k, v: [n_heads, n_tokens_total, d_head]; copies rows start:end (chunk.cpp:63-81)."""
        n = end - start
        if n > self.capacity - self.n_tokens:
            raise RuntimeError("no enough space in Chunk")
        t0 = self.n_tokens
        self.k[:, t0:t0 + n, :] = k[:, start:end, :]
        self.v[:, t0:t0 + n, :] = v[:, start:end, :]
        self.tokens.extend(int(t) for t in ids[start:end])

    def add_child(self, child):               # chunk.cpp:109-113
        self.children.append(child)
        child.parent = self
        return child

    def insert_child(self, idx, child):       # chunk.cpp:115-120
        self.children.insert(idx, child)
        child.parent = self
        return child


class Attention:
    """numpy restatement of GPT::Attention (cpp/chunk_attn/attention.h:16-75), fp32 only."""

    def __init__(self, n_heads, d_head, chunk_size, share_prefix=True):
        self.n_heads, self.d_head, self.chunk_size = n_heads, d_head, chunk_size
        self.share_prefix = share_prefix
        self.root = Chunk(0, n_heads, d_head)  # attention.cpp:28-29: capacity 0, n_seqs 0
        self.root.n_seqs = 0
        self.tails = []
        self._free_ids = []                    # recycled slots, lowest first
        self._next_id = 0

    def _new_chunk(self):
        """Lowest free slot first, as the reference's ordered free set hands chunks out
        (cpp/chunk_attn/chunk_allocator.cpp:57-68)."""
        if self._free_ids:
            cid = heapq.heappop(self._free_ids)
        else:
            cid = self._next_id
            self._next_id += 1
        return Chunk(self.chunk_size, self.n_heads, self.d_head, cid)

    # ---- tree maintenance -------------------------------------------------------------------
    def add_seq(self, tokens, k, v):
        """Insert a sequence; k, v are [n_tokens, n_heads, d_head].  Returns its row index.

        Follows cpp/chunk_attn/attention.cpp:141-193: whole chunks of token ids are matched
        against NON-LEAF children only; the row index is the number of sequences that precede
        the new one in depth-first order; a sequence whose last chunk is full gets an empty
        leaf so that every sequence owns a distinct tail.
        """
        k = np.ascontiguousarray(np.asarray(k, np.float32).transpose(1, 0, 2))
        v = np.ascontiguousarray(np.asarray(v, np.float32).transpose(1, 0, 2))
        tokens = [int(t) for t in tokens]
        total = len(tokens)
        seq_idx, start, prev = 0, 0, self.root
        if self.share_prefix:
            while start < total:
                prev.n_seqs += 1
                start += prev.n_tokens
                found = False
                for child in prev.children:
                    if child.children and child.equal(tokens, start, start + child.n_tokens):
                        prev, found = child, True
                        break
                    seq_idx += child.n_seqs
                if not found:
                    break
        else:
            prev.n_seqs += 1
        while start < total:
            end = min(start + self.chunk_size, total)
            child = self._new_chunk()
            child.append_tokens(tokens, k, v, start, end)
            prev = prev.add_child(child)
            start += self.chunk_size
        if prev.full():
            prev = prev.add_child(self._new_chunk())
        self.tails.insert(seq_idx, prev)
        return seq_idx

    def remove_seq(self, seq_idx):
        """cpp/chunk_attn/attention.cpp:263-278."""
        node = self.tails[seq_idx]
        while node is not None:
            node.n_seqs -= 1
            parent = node.parent
            if node.n_seqs <= 0 and parent is not None:
                parent.children = [c for c in parent.children if c is not node]
                heapq.heappush(self._free_ids, node.id)
            node = parent
        del self.tails[seq_idx]

    def reserve(self):
        """Give every full tail an empty child (cpp/chunk_attn/attention.cpp:116-131)."""
        new_chunks = []
        for i, tail in enumerate(self.tails):
            if tail.full():
                child = self._new_chunk()
                new_chunks.append(child)
                self.tails[i] = tail.add_child(child)
        return new_chunks

    def append_token(self, tokens, k, v):
        """One new token per live sequence; k, v are [n_seqs, n_heads, d_head]
        (cpp/chunk_attn/attention.cpp:80-114, the non-fused branch)."""
        if len(self.tails) != len(tokens):
            raise RuntimeError("num of seqs is not equal to num of tokens")
        new_chunks = self.reserve()
        k = np.asarray(k, np.float32).transpose(1, 0, 2)
        v = np.asarray(v, np.float32).transpose(1, 0, 2)
        for i, tail in enumerate(self.tails):
            tail.append_tokens(tokens, k, v, i, i + 1)
        return new_chunks

    def duplicate(self, seq_idx, copies):
        """Clone the leaf of sequence `seq_idx` `copies` times as its next siblings
        (cpp/chunk_attn/attention.cpp:287-313, Chunk::deep_copy chunk.cpp:93-107).

        The reference leaves its `tails_` list untouched here, which makes the clones
        unreachable as rows; this restatement inserts them after the source row, which is
        where a depth-first walk of the resulting tree places them.
        """
        if copies < 1:
            return
        node, start = self.root, 0
        while node.children:
            node.n_seqs += copies
            for child in node.children:
                end = start + child.n_seqs
                if start <= seq_idx < end:
                    node = child
                    break
                start = end
        pos = node.parent.children.index(node) + 1
        for c in range(copies):
            clone = self._new_chunk()
            clone.tokens = list(node.tokens)
            clone.k[...] = node.k
            clone.v[...] = node.v
            node.parent.insert_child(pos + c, clone)
            self.tails.insert(seq_idx + 1 + c, clone)

    def append_completion(self, seq_idx, tokens, k, v):
        """One beam-search step: row `seq_idx` forks into len(tokens) rows, row seq_idx + i continuing
        with tokens[i] and K/V k[i], v[i] ([n_tokens, n_heads, d_head]).

        Intended meaning of cpp/chunk_attn/attention.cpp:227-261 ("duplicate a seq ... in beam
        search", attention.h:43-44): copies of the leaf become its next siblings, every copy takes one
        of the candidate tokens, leaves that fill up get their empty successor.  The reference's
        function is not exported to Python and does not maintain the ancestors' sharer counts or its
        row list, so there is no reference behaviour to pin this against; the check is the dense one
        (every resulting row attends over its full token history).
        """
        if not tokens:
            raise RuntimeError("append_completion: at least one token is required")
        self.reserve()
        self.duplicate(seq_idx, len(tokens) - 1)
        k = np.asarray(k, np.float32).transpose(1, 0, 2)
        v = np.asarray(v, np.float32).transpose(1, 0, 2)
        for i in range(len(tokens)):
            self.tails[seq_idx + i].append_tokens(tokens, k, v, i, i + 1)
        self.reserve()
        return seq_idx

    def clear(self):
        """Intended meaning of cpp/chunk_attn/attention.cpp:280-285: drop every sequence."""
        while self.tails:
            self.remove_seq(len(self.tails) - 1)

    # ---- work list ----------------------------------------------------------------------------
    def get_chunks(self):
        """[(chunk, seq_begin, seq_end)] for every non-root chunk, empty leaves included, in the
        reference's order: explicit-stack pre-order, children pushed first-to-last and therefore
        visited last-to-first (cpp/chunk_attn/attention.cpp:342-372)."""
        infos = []
        stack = [(0, self.root)]
        while stack:
            seq_begin, chunk = stack.pop()
            seq_end = seq_begin + chunk.n_seqs
            start = seq_begin
            for child in chunk.children:
                stack.append((start, child))
                start += child.n_seqs
            if chunk is not self.root:
                infos.append((chunk, seq_begin, seq_end))
        return infos

    # ---- attention ----------------------------------------------------------------------------
    def forward(self, q, partition=0):
        """q: [n_seqs, n_heads, d_head] fp32 -> [n_seqs, n_heads, d_head]
        (cpp/chunk_attn/kernel_cpu_mkl.cpp:364-372: partition 0/1 chunk-first, 2 seq-first)."""
        q = np.ascontiguousarray(q, np.float32)
        if partition in (0, 1):
            return self._chunk_first(q)
        if partition == 2:
            return self._seq_first(q)
        raise RuntimeError("Unsupported partition type")

    def _chunk_first(self, q):
        """cpp/chunk_attn/kernel_cpu_mkl.cpp:245-353 with attn_one_chunk :16-120, all heads of a
        chunk at once (the reference runs the same arithmetic one head per task)."""
        n_seqs, H, d = q.shape
        d_sqrt = np.float32(math.sqrt(d))
        out = np.zeros((n_seqs, H, d), np.float32)          # attention.cpp:69 (zeros on MKL)
        wmax = np.full((H, n_seqs), F32_LOWEST, np.float32)  # kernel_cpu_mkl.cpp:248-250
        wsum = np.zeros((H, n_seqs), np.float32)
        for chunk, b, e in self.get_chunks():
            t = chunk.n_tokens
            if t <= 0:
                continue                                     # :30-32
            qh = q[b:e].transpose(1, 0, 2)                   # [H, n, d]
            w = np.matmul(qh, chunk.k[:, :t, :].transpose(0, 2, 1))      # sgemm :41-55
            m = w.max(axis=2, keepdims=True)                 # :59-62
            w = np.exp((w - m) / d_sqrt, dtype=np.float32)   # :67-69
            m_local = (m[:, :, 0] / d_sqrt).astype(np.float32)            # :71
            o_local = np.matmul(w, chunk.v[:, :t, :])        # sgemm :74-88, [H, n, d]
            m_new = np.maximum(wmax[:, b:e], m_local)        # :93-98
            s1 = np.exp(m_local - m_new, dtype=np.float32)   # :99
            s2 = np.exp(wmax[:, b:e] - m_new, dtype=np.float32)           # :100
            wmax[:, b:e] = m_new
            o_prev = out[b:e].transpose(1, 0, 2)
            out[b:e] = (s1[:, :, None] * o_local + s2[:, :, None] * o_prev).transpose(1, 0, 2)  # :103-107
            wsum[:, b:e] = s1 * w.sum(axis=2, dtype=np.float32) + s2 * wsum[:, b:e]            # :110-116
        with np.errstate(divide="ignore", invalid="ignore"):
            out /= wsum.T[:, :, None]                        # :352
        return out

    def _seq_first(self, q):
        """cpp/chunk_attn/kernel_cpu_mkl.cpp:215-242 with attn_one_seq :122-213, all heads of a
        sequence at once."""
        n_seqs, H, d = q.shape
        d_sqrt = np.float32(math.sqrt(d))
        out = np.zeros((n_seqs, H, d), np.float32)
        infos = self.get_chunks()
        for s in range(n_seqs):
            qs = q[s][:, None, :]                            # [H, 1, d]
            o = np.zeros((H, 1, d), np.float32)
            wmax = np.full((H, 1, 1), F32_LOWEST, np.float32)
            wsum = np.zeros((H, 1, 1), np.float32)
            for chunk, b, e in infos:
                if s < b or s >= e:
                    continue                                 # :140-142
                t = chunk.n_tokens
                if t <= 0:
                    continue                                 # :146-148
                w = np.matmul(qs, chunk.k[:, :t, :].transpose(0, 2, 1))  # :153-167
                m = np.maximum(wmax, w.max(axis=2, keepdims=True))        # :170-173
                w = np.exp((w - m) / d_sqrt, dtype=np.float32)            # :177-180
                s2 = np.exp((wmax - m) / d_sqrt, dtype=np.float32)        # :182
                o = np.matmul(w, chunk.v[:, :t, :]) + s2 * o              # :185-199
                wsum = w.sum(axis=2, keepdims=True, dtype=np.float32) + s2 * wsum  # :202-206
                wmax = m
            with np.errstate(divide="ignore", invalid="ignore"):
                out[s] = (o / wsum)[:, 0, :]                 # :210-212
        return out

    # ---- helpers used by the tests --------------------------------------------------------------
    def seq_kv(self, seq_idx):
        """Dense K, V ([n_heads, ctx, d_head]) of one sequence, gathered root -> leaf."""
        path, node = [], self.tails[seq_idx]
        while node is not None and node is not self.root:
            path.append(node)
            node = node.parent
        path.reverse()
        k = np.concatenate([c.k[:, :c.n_tokens, :] for c in path], axis=1)
        v = np.concatenate([c.v[:, :c.n_tokens, :] for c in path], axis=1)
        return k, v

    def shape(self):
        """Nested (n_seqs, tokens, [children...]) description of the tree, for comparisons."""
        def rec(c):
            return (c.n_seqs, list(c.tokens), [rec(x) for x in c.children])
        return rec(self.root)

    def unique_tokens(self):
        return sum(c.n_tokens for c, _, _ in self.get_chunks())


def dense_attention(q, k, v):
    """softmax(q k^T / sqrt(d)) v in float64 for one sequence: q [H, d], k/v [H, ctx, d]."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    s = np.einsum("hd,htd->ht", q, k) / math.sqrt(q.shape[-1])
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    return np.einsum("ht,htd->hd", p, v)


def dense_forward(attn, q):
    """Dense fp64 attention for every live sequence of an oracle Attention."""
    q = np.asarray(q)
    out = np.zeros(q.shape, np.float64)
    for s in range(q.shape[0]):
        k, v = attn.seq_kv(s)
        out[s] = dense_attention(q[s], k, v)
    return out
