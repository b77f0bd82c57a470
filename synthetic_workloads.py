"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five benchmark
configurations (they stand in for any real serving trace; the reference's own benchmarks are
synthetic `torch.randn` too, tests/benchmark_attn_pytorch.py:14-28).

Values: q, k, v ~ N(0, 1) * scale from `torch.Generator().manual_seed(seed)`, drawn in a fixed
order (shared-prefix K, shared-prefix V, then for each sequence its unique K and V, finally q) in
fp32 and then cast.  Token ids: shared prefix 0..s-1, group prefixes 10_000*(g+1)+j, unique tails
1_000_000*(uid+1)+j, so that nothing matches by accident.

A workload is engine-agnostic: `populate()` feeds any object with the `add_seq` method (the CUDA
engine, the oracle, the reference build).
"""
import random
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class Segment:
    """A span of a sequence's context: token ids plus the K/V rows [n, H, d] (fp32, CPU or CUDA)."""
    tokens: List[int]
    k: torch.Tensor
    v: torch.Tensor


@dataclass
class Workload:
    name: str
    n_heads: int
    d_head: int
    chunk_size: int
    dtype: torch.dtype
    seed: int
    scale: float
    seqs: List[List[Segment]] = field(default_factory=list)   # per sequence: its segments, root first
    q: Optional[torch.Tensor] = None                          # [n_seqs, H, d] in insertion order

    @property
    def n_seqs(self):
        return len(self.seqs)

    def context_len(self, i):
        return sum(len(s.tokens) for s in self.seqs[i])


def _randn(gen, n, H, d, scale):
    return torch.randn((n, H, d), generator=gen, device=gen.device, dtype=torch.float32) * scale


def single_level(name, n_heads, d_head, chunk_size, dtype, n_seqs, shared, unique, seed, scale, gen_device="cpu"):
    gen = torch.Generator(device=gen_device).manual_seed(seed)
    w = Workload(name, n_heads, d_head, chunk_size, dtype, seed, scale)
    pref = None
    if shared > 0:
        pref = Segment(list(range(shared)), _randn(gen, shared, n_heads, d_head, scale),
                       _randn(gen, shared, n_heads, d_head, scale))
    for s in range(n_seqs):
        segs = [pref] if pref is not None else []
        if unique > 0:
            segs.append(Segment([1_000_000 * (s + 1) + j for j in range(unique)],
                                _randn(gen, unique, n_heads, d_head, scale),
                                _randn(gen, unique, n_heads, d_head, scale)))
        w.seqs.append(segs)
    w.q = _randn(gen, n_seqs, n_heads, d_head, scale)
    return w


def config1():
    """CPU plumbing case: H8 d64 c32 fp32, 4 sequences = 256 shared + 32 unique, N(0,1), seed 0."""
    return single_level("cfg1", 8, 64, 32, torch.float32, 4, 256, 32, 0, 1.0)


def config2(n_heads=32, n_seqs=32, shared=2048, unique=512, gen_device="cpu"):
    """Headline: H32 d128 c64 fp16, 32 sequences = 2048 shared + 512 unique, N(0,1)*0.5, seed 1."""
    return single_level("cfg2", n_heads, 128, 64, torch.float16, n_seqs, shared, unique, 1, 0.5, gen_device)


def config3(shared, n_heads=32, n_seqs=64, ctx=4096, gen_device="cpu"):
    """Prefix-sharing sweep: batch 64, context 4096, `shared` of it common to all; seed 2."""
    return single_level("cfg3_s%d" % shared, n_heads, 128, 64, torch.float16, n_seqs, shared, ctx - shared, 2, 0.5,
                        gen_device)


def config5(n_heads=64, n_seqs=256, shared=4096, unique=1024, gen_device="cpu"):
    """Head-sharded large batch: H64 (split across GPUs), 256 sequences = 4096 shared + 1024 unique; seed 4."""
    return single_level("cfg5", n_heads, 128, 64, torch.float16, n_seqs, shared, unique, 4, 0.5, gen_device)


@dataclass
class Config4:
    """Two-level tree with incremental decode: 4 groups under a root prefix; every `churn_every`
    steps `churn` random sequences leave and as many new ones join random groups; seed 3."""
    n_heads: int = 32
    d_head: int = 128
    chunk_size: int = 64
    dtype: torch.dtype = torch.float16
    n_groups: int = 4
    per_group: int = 32
    root_len: int = 1024
    group_len: int = 1024
    unique_len: int = 256
    steps: int = 64
    churn_every: int = 16
    churn: int = 8
    seed: int = 3
    scale: float = 0.5
    gen_device: str = "cpu"

    def __post_init__(self):
        self.gen = torch.Generator(device=self.gen_device).manual_seed(self.seed)
        self.rng = random.Random(self.seed)
        H, d = self.n_heads, self.d_head
        self.root = Segment(list(range(self.root_len)), _randn(self.gen, self.root_len, H, d, self.scale),
                            _randn(self.gen, self.root_len, H, d, self.scale))
        self.groups = [Segment([10_000 * (g + 1) + j for j in range(self.group_len)],
                               _randn(self.gen, self.group_len, H, d, self.scale),
                               _randn(self.gen, self.group_len, H, d, self.scale)) for g in range(self.n_groups)]
        self.next_uid = 0

    def new_sequence(self, group):
        uid = self.next_uid
        self.next_uid += 1
        H, d = self.n_heads, self.d_head
        uniq = Segment([1_000_000 * (uid + 1) + j for j in range(self.unique_len)],
                       _randn(self.gen, self.unique_len, H, d, self.scale),
                       _randn(self.gen, self.unique_len, H, d, self.scale))
        return [self.root, self.groups[group], uniq]

    def initial(self):
        return [self.new_sequence(g) for g in range(self.n_groups) for _ in range(self.per_group)]

    def step_inputs(self, n_seqs):
        H, d = self.n_heads, self.d_head
        return (_randn(self.gen, n_seqs, H, d, self.scale), _randn(self.gen, n_seqs, H, d, self.scale),
                _randn(self.gen, n_seqs, H, d, self.scale))  # q, new k, new v (rows in current row order)


def cat_segments(segs, head_slice=None, device=None, dtype=None):
    """tokens, k, v of a whole sequence; K/V optionally restricted to a head slice and cast."""
    tokens = [t for s in segs for t in s.tokens]
    ks = [s.k if head_slice is None else s.k[:, head_slice] for s in segs]
    vs = [s.v if head_slice is None else s.v[:, head_slice] for s in segs]
    if device is not None or dtype is not None:
        ks = [x.to(device=device, dtype=dtype) for x in ks]
        vs = [x.to(device=device, dtype=dtype) for x in vs]
    return tokens, torch.cat(ks, dim=0), torch.cat(vs, dim=0)


def populate(attn, workload, device=None, dtype=None, head_slice=None, as_numpy=False):
    """add_seq every sequence of the workload.  Returns `rows`: rows[i] = index into workload.seqs of
    the sequence that sits in row i of q / out (add_seq returns the insertion row; later rows shift)."""
    rows = []
    refs = {}
    for segs in workload.seqs:
        for s in segs:
            refs[id(s)] = refs.get(id(s), 0) + 1
    cache = {}  # cast segments that several sequences share only once
    for si, segs in enumerate(workload.seqs):
        parts = []
        for s in segs:
            if id(s) in cache:
                k, v = cache[id(s)]
            else:
                k = s.k if head_slice is None else s.k[:, head_slice]
                v = s.v if head_slice is None else s.v[:, head_slice]
                if device is not None or dtype is not None:
                    k, v = k.to(device=device, dtype=dtype), v.to(device=device, dtype=dtype)
                if refs[id(s)] > 1:
                    cache[id(s)] = (k, v)
            parts.append((s.tokens, k, v))
        tokens = [t for p in parts for t in p[0]]
        k = torch.cat([p[1] for p in parts], dim=0) if len(parts) > 1 else parts[0][1]
        v = torch.cat([p[2] for p in parts], dim=0) if len(parts) > 1 else parts[0][2]
        if as_numpy:
            idx = attn.add_seq(tokens, k.float().cpu().numpy(), v.float().cpu().numpy())
        else:
            idx = attn.add_seq(tokens=tokens, k=k, v=v)
        rows.insert(idx, si)
    return rows


def unique_kv_bytes(workload, n_heads=None):
    """Algorithmic bytes of one decode step: every distinct K/V token once."""
    seen, tokens = set(), 0
    for segs in workload.seqs:
        for s in segs:
            if id(s) not in seen:
                seen.add(id(s))
                tokens += len(s.tokens)
    H = n_heads if n_heads is not None else workload.n_heads
    return tokens * H * workload.d_head * 2 * torch.empty((), dtype=workload.dtype).element_size()
