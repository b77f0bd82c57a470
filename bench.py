#!/usr/bin/env python
"""Benchmark of the ChunkAttention decode step (one JSON line on stdout, printed by rank 0).

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path, same workload

A step is one `Attention.forward(q)` over the current batch on an up-to-date work list (the
reference's own protocol times exactly that, tests/benchmark_chunk_attn.py:60-69,84-97).

Workloads (synthetic, seeded; synthetic_workloads.py):
  N = 1  cfg2: H32 d128 c64 fp16, 32 sequences = 2048 shared + 512 unique tokens (302 MB of unique
         K/V, larger than the 126 MB L2, so nothing needs flushing between steps); the other four
         configurations (cfg3 at its five prefix lengths, cfg4) are measured beside it in `other_configs`
  N > 1  cfg5: H64 split evenly over the ranks, 256 sequences = 4096 shared + 1024 unique tokens,
         output gathered on every rank; strong scaling: total work is fixed
  N = 1 on a machine that shows several GPUs is taken for the one-GPU point of the N = 1, 2, 4, 8 series and
         runs cfg5 on one GPU (cfg2 beside it in `headline_cfg2`); CA_BENCH_N1=cfg2 forces cfg2.  The choice
         is recorded in `config.workload_choice`.
`--workload` overrides the choice (cfg2, cfg5, cfg3_s<shared>, cfg4, short<n_seqs>: a 1024-token common
prompt with 20-token private suffixes, sys<n_seqs>: a 2048-token system prompt with 8-token suffixes, llama: the
decoder loop).

Every line carries `parity`: sampled (row, head) outputs of the very tensors that are timed, compared with dense
fp64 attention computed from the seeded inputs (on N > 1 including heads owned by other ranks, regenerated from
their seeds); the run exits non-zero above 2e-3.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "chunk-attention_b200"))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_attn_us_per_step"
PARITY_TOL = 2e-3   # max-abs bar for fp16 outputs against the reference arithmetic (dense attention)
SPREAD_BLOCKS = 5   # further event-timed blocks of K steps each, after the block `value` comes from
MIN_WARMUP_STEPS = 50  # untimed steps before the timed region are max(--warmup, this): the clock sampler's start leaves
                       # the GPU idle for milliseconds, and five 50-200 us steps do not bring it back to speed
CFG3_SHARED = (0, 1024, 2048, 3072, 4096)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--split-phases", type=int, default=0)
    ap.add_argument("--ctas", type=int, default=0, help="persistent CTAs (0 = two per SM)")
    ap.add_argument("--tails", default="tensor", choices=["tensor", "simt"],
                    help="private tails on tensor cores (default) or on CUDA cores")
    ap.add_argument("--wide", default="auto", choices=["auto", "on", "off"],
                    help="wide shared runs on the tcgen05 / TMEM path: by the planner's threshold, always, never")
    ap.add_argument("--overlap", action="store_true",
                    help="run the short-tails kernel beside the wide-runs kernel (second stream) instead of before it")
    ap.add_argument("--no-finish", action="store_true",
                    help="short private tails always as partial rows + merge kernel (default: the short-tails kernel stores "
                         "the output rows itself when every row has a short tail)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the reference's own CUDA kernels")
    ap.add_argument("--no-scale-point", action="store_true", help="N = 1: skip the one-GPU point of the cfg5 series")
    ap.add_argument("--no-other-configs", action="store_true", help="N = 1: skip the cfg3 / cfg4 block")
    ap.add_argument("--other-budget", type=float, default=60.0, help="seconds the cfg3 / cfg4 block may take")
    ap.add_argument("--llama-batch", type=int, default=64)
    ap.add_argument("--llama-prompt", type=int, default=1024)
    ap.add_argument("--llama-shared", type=int, default=0)
    ap.add_argument("--llama-completion", type=int, default=64)
    ap.add_argument("--runs", type=int, default=3, help="llama workload: timed repetitions")
    ap.add_argument("--warmup-runs", type=int, default=1, help="llama workload: untimed repetitions")
    ap.add_argument("--gather", default="p2p", choices=["nccl", "p2p"],
                    help="N > 1: all-gather with NCCL, or rows stored into peers' outputs by the merge kernel")
    ap.add_argument("--barrier", default="own", choices=["own", "torch"],
                    help="N > 1, p2p: this library's bounded barrier kernel, or torch's symmetric-memory barrier")
    ap.add_argument("--no-multicast", action="store_true", help="N > 1, p2p: unicast peer stores instead of multimem.st")
    return ap.parse_args()


def workload_name(args):
    """cfg2 on a one-GPU machine (the configuration the metric is quoted on), cfg5 for N > 1.  A one-GPU run on
    a machine that shows several GPUs is taken for the N = 1 point of the N = 1, 2, 4, 8 series and runs cfg5
    as well, so that the series compares like with like; cfg2 is then reported beside it (`headline_cfg2`)."""
    if args.workload != "auto":
        return args.workload, "--workload"
    if args.gpus > 1:
        return "cfg5", "N > 1: the head-sharded configuration"
    if visible_gpus() > 1 and os.environ.get("CA_BENCH_N1", "") != "cfg2":
        return "cfg5", "N = 1 with %d GPUs visible: the one-GPU point of the cfg5 scaling series" % visible_gpus()
    return "cfg2", "N = 1: the configuration the metric is quoted on"


def visible_gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def describe(name, n_gpus):
    if name == "cfg2":
        return "cfg2: H32 d128 c64 fp16, 32 seqs x (2048 shared + 512 unique tokens), 1 query/seq"
    if name == "cfg5":
        return ("cfg5: H64 (H/%d per GPU) d128 c64 fp16, 256 seqs x (4096 shared + 1024 unique tokens), "
                "1 query/seq, output all-gathered" % n_gpus)
    if name == "cfg4":
        return ("cfg4: H32 d128 c64 fp16, 128 seqs in 4 groups (1024 root + 1024 group + 256 unique), 64 decode steps "
                "appending 1 token/seq, 8 seqs replaced every 16 steps; value = append + work-list update + forward")
    if name.startswith("short"):
        return ("%s: H32 d128 c64 fp16, %s seqs x (1024 shared + 20 unique tokens): a long common prompt with short "
                "private suffixes" % (name, name[5:] or "256"))
    if name.startswith("sys"):
        return ("%s: H32 d128 c64 fp16, %s seqs x (2048 shared + 8 unique tokens): many requests over one system "
                "prompt" % (name, name[3:] or "1024"))
    return "%s: H32 d128 c64 fp16, 64 seqs, context 4096, shared prefix %s" % (name, name.split("_s")[-1])


def make_workload(name, n_heads_local, gen_device, rank=0):
    import torch
    import synthetic_workloads as W
    if name == "cfg2":
        return W.config2(n_heads=n_heads_local, gen_device=gen_device)
    if name == "cfg5":
        # every rank draws its own head slice from its own seed, 4 + 1000 * rank
        return W.single_level("cfg5", n_heads_local, 128, 64, torch.float16, 256, 4096, 1024, 4 + 1000 * rank, 0.5,
                              gen_device)
    if name.startswith("cfg3_s"):
        return W.config3(int(name[6:]), n_heads=n_heads_local, gen_device=gen_device)
    if name.startswith("short"):  # short<n_seqs>: not one of the five configurations; the short-suffix serving shape
        return W.single_level(name, n_heads_local, 128, 64, torch.float16, int(name[5:] or 256), 1024, 20, 5, 0.5,
                              gen_device)
    if name.startswith("sys"):    # sys<n_seqs>: many requests over one system prompt (contraction-bound)
        return W.single_level(name, n_heads_local, 128, 64, torch.float16, int(name[3:] or 1024), 2048, 8, 6, 0.5,
                              gen_device)
    raise SystemExit("unknown workload " + name)


def total_heads(name):
    return 64 if name == "cfg5" else 32


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, an earlier measurement on this pool)"


def cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def host_threads():
    """All the host threads the process may use (torchrun exports OMP_NUM_THREADS=1 to its workers; the
    reference sizes its OpenMP team from torch's thread count when a cache is constructed)."""
    import torch
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    cores = max(torch.get_num_threads(), avail)
    torch.set_num_threads(cores)
    return cores


# ---- parity of the timed tensors ------------------------------------------------------------------------------
def dense_parity(w, rows, out, q, pairs, head_offset=0, extra=None):
    """Max-abs error of sampled (row, local head) outputs against dense fp64 softmax(q K^T / sqrt(d)) V computed
    from the fp16-rounded seeded inputs of workload `w` (whose heads sit at head_offset.. of `out`).  `rows[r]`
    names the sequence in row r; `extra`, when given, maps a row to (k rows, v rows) appended after the prefill."""
    import math
    import torch
    import synthetic_workloads as W
    worst = 0.0
    for r, h in pairs:
        segs = rows[r] if isinstance(rows[r], list) else w.seqs[rows[r]]
        _, k, v = W.cat_segments(segs, head_slice=slice(h, h + 1))
        k, v = k.to(out.device).half().double()[:, 0], v.to(out.device).half().double()[:, 0]
        if extra is not None and extra[r][0]:
            k = torch.cat([k, torch.stack([x[h] for x in extra[r][0]]).to(out.device).double()])
            v = torch.cat([v, torch.stack([x[h] for x in extra[r][1]]).to(out.device).double()])
        s = (k @ q[r, h].to(out.device).half().double()) / math.sqrt(k.shape[1])
        ref = torch.softmax(s, 0) @ v
        worst = max(worst, float((out[r, head_offset + h].double() - ref).abs().max()))
    return worst


def sample_pairs(n_rows, n_heads, n, seed):
    """n (row, head) pairs: rows spread over the batch, the first and the last head always among them."""
    import random
    rnd = random.Random(seed)
    pairs = [(rnd.randrange(n_rows), 0), (rnd.randrange(n_rows), n_heads - 1), (0, rnd.randrange(n_heads)),
             (n_rows - 1, rnd.randrange(n_heads))]
    while len(pairs) < n:
        pairs.append((rnd.randrange(n_rows), rnd.randrange(n_heads)))
    return pairs[:n]


def spread_of(block_us):
    return {"value_median": statistics.median(block_us), "value_min": min(block_us), "value_max": max(block_us),
            "blocks": len(block_us)}


# ---- this engine: building and timing -----------------------------------------------------------------------------
def build_engine(name, n_heads_local, dev, args, sharded=False, rank=0, keep_workload=False):
    """The cache of one GPU filled with its head slice of workload `name`.  Returns (attn, engine, q, unique K/V
    bytes, workload or None, rows): `attn` is what a step calls (the head-sharded wrapper when `sharded`),
    `engine` the local Attention underneath."""
    import torch
    from chunk_attn import Attention, cabi
    from chunk_attn.sharded import HeadShardedAttention
    import synthetic_workloads as W
    gen_device = "cpu" if name == "cfg2" else dev
    w = make_workload(name, n_heads_local, gen_device, rank if sharded else 0)
    chunk_bytes = n_heads_local * 2 * 64 * 128 * 2
    n_chunks = W.unique_kv_bytes(w) // chunk_bytes + w.n_seqs + 8   # + one empty tail per sequence
    need_mb = (n_chunks * chunk_bytes + 2 ** 20 - 1) // 2 ** 20 + 1
    if sharded:
        attn = HeadShardedAttention(total_heads(name), 128, 64, memory_mb=need_mb, dtype=torch.float16, device=dev,
                                    gather=args.gather, barrier=args.barrier, multicast=not args.no_multicast)
        engine = attn.local
    else:
        attn = Attention(n_heads=n_heads_local, d_head=128, chunk_size=64, memory_mb=need_mb,
                         dtype=torch.float16, device=dev)
        engine = attn
    if args.split_phases:
        engine.set_option(cabi.CA_OPT_SPLIT_PHASES, 1)
    if args.ctas:
        engine.set_option(cabi.CA_OPT_NUM_CTAS, args.ctas)
    if args.tails == "simt":
        engine.set_option(cabi.CA_OPT_SEQ_FIRST_TENSOR, 0)
    if args.wide != "auto":
        engine.set_option(cabi.CA_OPT_WIDE_RUNS, 2 if args.wide == "on" else 0)
    if args.overlap:
        engine.set_option(cabi.CA_OPT_OVERLAP_KERNELS, 1)
    if args.no_finish:
        engine.set_option(cabi.CA_OPT_FINISH_IN_TAILS, 0)
    rows = W.populate(engine, w, device=dev, dtype=torch.float16)
    q = w.q[rows].to(dev, torch.float16).contiguous()
    ukv = W.unique_kv_bytes(w)
    if not keep_workload:
        w = None
    torch.cuda.empty_cache()
    return attn, engine, q, ukv, w, rows


def time_blocks(step, K, n_blocks, sync, align=None):
    """n_blocks blocks of K back-to-back steps, each block between two CUDA events on the launching stream.
    Returns the per-step milliseconds of every block (this rank's)."""
    import torch
    out = []
    for _ in range(n_blocks):
        sync()
        if align:
            align()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        sync()
        out.append(e0.elapsed_time(e1) / K)
    return out


def kernel_times(engine, q, K, split_phases):
    """Durations of the step's kernels, CUDA events on the launching stream around every single launch, plus
    the attention kernel's period when launched back to back with no event in between."""
    import torch
    kern = {}
    out2 = torch.empty_like(q)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    for i in range(K):
        evs[i][0].record()
        if split_phases:
            engine.attn_partials(q, 1)
            evs[i][3].record()
            engine.attn_partials(q, 2)
        else:
            engine.attn_partials(q, 3)
        evs[i][1].record()
        engine.attn_merge(out2)
        evs[i][2].record()
    torch.cuda.synchronize()
    if not split_phases:
        eb0, eb1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            engine.attn_partials(q, 3)
        eb0.record()
        for _ in range(K):
            engine.attn_partials(q, 3)
        eb1.record()
        torch.cuda.synchronize()
        kern["partials_back_to_back"] = eb0.elapsed_time(eb1) / K
    kern["partials"] = [e[0].elapsed_time(e[1]) for e in evs]
    kern["merge"] = [e[1].elapsed_time(e[2]) for e in evs]
    if split_phases:
        kern["chunk_first"] = [e[0].elapsed_time(e[3]) for e in evs]
        kern["seq_first"] = [e[3].elapsed_time(e[1]) for e in evs]
    return kern


# DRAM bytes of one attention-kernel launch at config 2 from the ncu capture summarised in
# profiles/attn_partial_kernel_cfg2.md (dram__bytes_read.sum 302.97 MB + dram__bytes_write.sum 10.1 MB).  Other
# workloads hold too much on the device to capture under the size rule: their figure is this one scaled by the
# unique K/V bytes of a launch (reads are the K/V once, the partial rows written grow with them).
NCU_CFG2_TRAFFIC = 313.0e6
NCU_CFG2_SOURCE = "constant from profiles/attn_partial_kernel_cfg2.md (one launch, ncu dram__bytes_read+write)"


def roofline_of(name, ukv_local, kern, peak, peak_src, single_gpu):
    dur_ms = statistics.mean(kern["partials"])
    achieved = ukv_local / (dur_ms * 1e-3) / 1e9
    exact = name == "cfg2" and single_gpu
    roof = {"bound": "hbm", "kernel": "attn_partial_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": peak_src,
            "traffic": NCU_CFG2_TRAFFIC if exact else ukv_local * (NCU_CFG2_TRAFFIC / 301989888),
            "traffic_source": NCU_CFG2_SOURCE if exact else NCU_CFG2_SOURCE + ", scaled by unique K/V bytes per launch",
            "algorithmic_bytes_per_launch": ukv_local,
            "kernel_ms": {"partials_mean": dur_ms, "partials_min": min(kern["partials"]),
                          "merge_mean": statistics.mean(kern["merge"]),
                          "partials_back_to_back": kern.get("partials_back_to_back")}}
    if kern.get("chunk_first"):
        roof["kernel_ms"]["chunk_first_mean"] = statistics.mean(kern["chunk_first"])
        roof["kernel_ms"]["seq_first_mean"] = statistics.mean(kern["seq_first"])
    if kern.get("partials_back_to_back"):
        roof["frac_back_to_back"] = ukv_local / (kern["partials_back_to_back"] * 1e-3) / 1e9 / peak
    return roof


def measure_static(name, dev, K, W_, args, n_parity=8, ref_cuda=True):
    """One of the static one-GPU configurations, complete with its own clock record: us/step over K steps (mean of
    the first block, spread over the following ones), the attention kernel's own duration and roofline fraction,
    parity of the timed output against dense fp64, and the reference's CUDA kernels on the same inputs."""
    import torch
    H = total_heads(name)
    attn, engine, q, ukv, w, rows = build_engine(name, H, dev, args, keep_workload=True)
    out = attn.forward(q=q)
    pairs = sample_pairs(q.shape[0], H, n_parity, 11)
    err = dense_parity(w, rows, out, q, pairs)
    del w
    torch.cuda.empty_cache()
    sampler = ClockSampler(dev.index or 0).start()
    for _ in range(max(W_, MIN_WARMUP_STEPS)):
        attn.forward(q=q)
    blocks = time_blocks(lambda: attn.forward(q=q), K, 1 + SPREAD_BLOCKS, torch.cuda.synchronize)
    kern = kernel_times(engine, q, K, args.split_phases) if engine.plan_stats()["fast_path"] else None
    clocks = sampler.stop()
    peak, peak_src = measured_peak()
    us = blocks[0] * 1e3
    res = {"workload": describe(name, 1), "us_per_step": us, "steps": K, "warmup": W_,
           "warmup_steps_run": max(W_, MIN_WARMUP_STEPS),
           "unique_kv_bytes": ukv, "hbm_frac": ukv / (us * 1e-6) / 1e9 / peak,
           "l2": "unique K/V (%.0f MB) %s the 126 MB L2" % (ukv / 1e6, "exceeds" if ukv > 126e6 else "fits in"),
           "parity": {"max_abs": err, "samples": len(pairs), "tol": PARITY_TOL, "against": "dense fp64"},
           "clocks": clocks, "plan": engine.plan_stats(), "device_status": engine.device_status()}
    res.update(spread_of([b * 1e3 for b in blocks]))
    if kern:
        res["roofline"] = roofline_of(name, ukv, kern, peak, peak_src, True)
    if err > PARITY_TOL:
        raise SystemExit("parity: %s max-abs %.3g against dense fp64 exceeds %.1g" % (name, err, PARITY_TOL))
    del attn, engine
    torch.cuda.empty_cache()
    if ref_cuda:
        try:
            res["reference_cuda"] = time_reference_cuda(name, dev, min(K, 50), 3)
        except Exception as exc:  # reported, never a gate
            res["reference_cuda"] = {"us_per_step": None, "note": "failed: %s" % str(exc)[:200]}
    return res


def measure_cfg4(dev, args, passes=1, with_e2e=True):
    """Two-level prefix tree with incremental decode (configuration 4): 128 sequences in 4 groups, 64 decode steps
    of append_token + forward, 8 sequences replaced every 16 steps.  The first pass over the trace is the warm-up;
    every later pass is timed per step with CUDA events: the whole step (append + work-list update + forward), the
    forward alone, the attention kernel alone (a second launch on the same work list), and the host time of
    append + update.  A last pass runs the same steps from pinned HOST buffers (queries and new K/V rows copied in,
    result rows stored to host memory) for the end-to-end figure."""
    import torch
    from chunk_attn import Attention
    import synthetic_workloads as W
    attn = Attention(n_heads=32, d_head=128, chunk_size=64, memory_mb=1400, dtype=torch.float16, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    step_ms, fwd_ms, kern_ms, host_ms, ukv, e2e_ms, pipe_ms, host_parts, pipe_host_ms = [], [], [], [], [], [], [], [], []
    parity = {"max_abs": 0.0, "samples": 0, "tol": PARITY_TOL, "against": "dense fp64 over prefill + appended rows",
              "steps_checked": []}
    q_host = out_host = k_host = v_host = None
    sampler = None
    launches_per_step = 3
    n_passes = 1 + 2 * passes + (1 if with_e2e else 0)
    for rep in range(n_passes):
        timed = 1 <= rep <= passes      # every step alone on an idle GPU, for the per-step break-down
        e2e_pass = with_e2e and rep == n_passes - 1
        pipe_pass = passes < rep <= 2 * passes   # the steps between two replacements enqueued back to back: the step time
        pre, pe0 = [], None
        cfg = W.Config4(gen_device=dev)
        seqs = []

        def add(segs):
            tokens, k, v = W.cat_segments(segs, device=dev, dtype=torch.float16)
            seqs.insert(attn.add_seq(tokens=tokens, k=k, v=v), {"segs": segs, "k": [], "v": []})

        for segs in cfg.initial():
            add(segs)
        if rep == 1:
            torch.cuda.synchronize()
            sampler = ClockSampler(dev.index or 0).start()
        for step in range(cfg.steps):
            if step and step % cfg.churn_every == 0:
                for _ in range(cfg.churn):
                    i = cfg.rng.randrange(len(seqs))
                    attn.remove_seq(i)
                    seqs.pop(i)
                for _ in range(cfg.churn):
                    add(cfg.new_sequence(cfg.rng.randrange(cfg.n_groups)))
            if pipe_pass:
                if not pre:
                    n_seg = min(cfg.churn_every - step % cfg.churn_every, cfg.steps - step)
                    pre = [tuple(t.to(torch.float16) for t in cfg.step_inputs(len(seqs))) for _ in range(n_seg)]
                    torch.cuda.synchronize()
                    pe0 = ev()
                    pe0.record()
                q, nk, nv = pre.pop(0)
                toks = [7_000_000 + step] * len(seqs)
                th0 = time.perf_counter()
                attn.append_token(tokens=toks, k=nk, v=nv)
                attn.refresh_kernel_context(False)
                pipe_host_ms.append((time.perf_counter() - th0) * 1e3)
                out = attn.forward(q=q)
                if not pre:
                    pe1 = ev()
                    pe1.record()
                    torch.cuda.synchronize()
                    pipe_ms.append(pe0.elapsed_time(pe1) / n_seg)
                    launches_per_step = 1 + attn.plan_stats()["kernels_per_step"]   # append_kv + the step's attention kernels
                continue
            q, nk, nv = (t.to(torch.float16) for t in cfg.step_inputs(len(seqs)))
            toks = [7_000_000 + step] * len(seqs)
            for i, sq in enumerate(seqs):
                sq["k"].append(nk[i])
                sq["v"].append(nv[i])
            if e2e_pass:
                if q_host is None:
                    q_host, k_host, v_host, out_host = (torch.empty(q.shape, dtype=torch.float16).pin_memory() for _ in range(4))
                    kd, vd = torch.empty_like(nk), torch.empty_like(nv)
                q_host.copy_(q)
                k_host.copy_(nk)
                v_host.copy_(nv)
                torch.cuda.synchronize()
                e0, e1 = ev(), ev()
                e0.record()
                kd.copy_(k_host, non_blocking=True)
                vd.copy_(v_host, non_blocking=True)
                attn.append_token(tokens=toks, k=kd, v=vd)
                attn.forward_host(q=q_host, out=out_host)     # returns when the rows are in out_host
                e1.record()
                torch.cuda.synchronize()
                e2e_ms.append(e0.elapsed_time(e1))
                continue
            torch.cuda.synchronize()
            e0, e1, e2 = ev(), ev(), ev()
            ht0 = attn.host_times()
            t0 = time.perf_counter()
            e0.record()
            attn.append_token(tokens=toks, k=nk, v=nv)
            attn.refresh_kernel_context(False)
            t1 = time.perf_counter()
            ht1 = attn.host_times()
            e1.record()
            out = attn.forward(q=q)
            e2.record()
            torch.cuda.synchronize()
            if timed:
                step_ms.append(e0.elapsed_time(e2))
                fwd_ms.append(e1.elapsed_time(e2))
                host_ms.append((t1 - t0) * 1e3)
                host_parts.append({k: ht1[k] - ht0[k] for k in ("walk_us", "plan_us", "upload_us")})
                ukv.append(attn.plan_stats()["unique_kv_bytes"])   # as of the last work-list update (appended rows not counted)
                k0, k1 = ev(), ev()
                k0.record()
                attn.attn_partials(q, 3)
                k1.record()
                torch.cuda.synchronize()
                kern_ms.append(k0.elapsed_time(k1))
            if rep == 1 and step in (0, 16, 40, 63):
                pairs = sample_pairs(len(seqs), 32, 4, 100 + step)
                err = dense_parity(None, [s["segs"] for s in seqs], out, q, pairs,
                                   extra=[(s["k"], s["v"]) for s in seqs])
                parity["max_abs"] = max(parity["max_abs"], err)
                parity["samples"] += len(pairs)
                parity["steps_checked"].append(step)
        if rep == 2 * passes and sampler is not None:
            clocks = sampler.stop()
            sampler = None
        while seqs:   # back to an empty cache so that every pass sees the same sizes
            attn.remove_seq(len(seqs) - 1)
            seqs.pop()
    if parity["max_abs"] > PARITY_TOL:
        raise SystemExit("parity: cfg4 max-abs %.3g against dense fp64 exceeds %.1g" % (parity["max_abs"], PARITY_TOL))
    peak, peak_src = measured_peak()
    n_seqs_bytes = 128 * 32 * 128 * 2
    churn_steps = [i for i in range(len(host_ms)) if (i % 64) and (i % 64) % 16 == 0]
    res = {"workload": describe("cfg4", 1), "us_per_step": statistics.mean(pipe_ms) * 1e3, "steps": 16 * len(pipe_ms),
           "warmup": 64, "us_per_step_each_step_alone": statistics.mean(step_ms) * 1e3,
           "forward_us": statistics.mean(fwd_ms) * 1e3,
           "forward_us_median": statistics.median(fwd_ms) * 1e3,
           "unique_kv_bytes_mean": statistics.mean(ukv),
           "hbm_frac": statistics.mean(ukv) / (statistics.mean(pipe_ms) * 1e-3) / 1e9 / peak,
           "hbm_frac_forward_alone": statistics.mean(ukv) / (statistics.mean(fwd_ms) * 1e-3) / 1e9 / peak,
           "l2": "unique K/V (620-760 MB) exceeds the 126 MB L2",
           "host_us_append_and_update": {"mean": statistics.mean(host_ms) * 1e3, "median": statistics.median(host_ms) * 1e3,
                                         "max": max(host_ms) * 1e3,
                                         "mean_at_replace_steps": statistics.mean(host_ms[i] for i in churn_steps) * 1e3
                                         if churn_steps else None,
                                         "work_list_update_at_replace_steps": {
                                             k: statistics.mean(host_parts[i][k] for i in churn_steps)
                                             for k in ("walk_us", "plan_us", "upload_us")} if churn_steps else None},
           "step_minus_forward_us": (statistics.mean(step_ms) - statistics.mean(fwd_ms)) * 1e3,
           "host_us_append_and_update_back_to_back": {
               "mean": statistics.mean(pipe_host_ms) * 1e3, "median": statistics.median(pipe_host_ms) * 1e3,
               "mean_at_replace_steps": statistics.mean(pipe_host_ms[i] for i in range(len(pipe_host_ms))
                                                        if i and i % cfg.churn_every == 0) * 1e3} if pipe_host_ms else None,
           "timing": "us_per_step: the 16 steps between two replacements enqueued back to back between two CUDA events, as "
                     "the other workloads' steps are (append_token + work-list update + forward each); "
                     "us_per_step_each_step_alone, forward_us, step_minus_forward_us, host_us_append_and_update: a pass "
                     "in which every step runs alone on an idle GPU, so that the host's work shows",
           "parity": parity, "clocks": clocks, "device_status": attn.device_status(),
           "gpu_launches_per_step": launches_per_step}
    res.update(spread_of([x * 1e3 for x in pipe_ms]))
    ach = statistics.mean(u / (k * 1e-3) / 1e9 for u, k in zip(ukv, kern_ms))
    res["roofline"] = {"bound": "hbm", "kernel": "attn_partial_kernel", "achieved": ach, "peak": peak, "unit": "GB/s",
                       "frac": ach / peak, "peak_source": peak_src,
                       "traffic": statistics.mean(ukv) * (NCU_CFG2_TRAFFIC / 301989888),
                       "traffic_source": NCU_CFG2_SOURCE + ", scaled by unique K/V bytes per launch",
                       "algorithmic_bytes_per_launch": statistics.mean(ukv),
                       "kernel_ms": {"partials_mean": statistics.mean(kern_ms), "partials_min": min(kern_ms)}}
    if e2e_ms:
        res["e2e"] = {"value": statistics.mean(e2e_ms) * 1e3, "unit": "us", "h2d_bytes_per_step": 3 * n_seqs_bytes,
                      "d2h_bytes_per_step": n_seqs_bytes,
                      "call": "copy_(k), copy_(v) from pinned memory + append_token + forward_host(q_pinned, out_pinned)"}
    del attn
    torch.cuda.empty_cache()
    return res


# ---- reference arm / CPU baseline -----------------------------------------------------------------------
def time_reference_cpu(name, steps, warmup, max_seconds=150.0):
    """The reference's own CPU (MKL) implementation of the step, unmodified, built into oracle/_ref;
    when that build is absent, the numpy restatement in oracle/.  fp32 (its only dtype), all host
    threads.  cfg5 is sampled on 8 of its 64 heads and scaled by 8 (the work is linear in heads)."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from ref_loader import load_reference
    import synthetic_workloads as W
    if name == "cfg4":
        return time_reference_cpu_cfg4(steps, max_seconds)
    heads_full = total_heads(name)
    heads = 8 if name == "cfg5" else heads_full
    scale_up = heads_full / heads
    w = make_workload(name, heads, "cpu")
    ref = load_reference("cpu")
    cores = host_threads()
    if ref is not None:
        kind = "reference"
        need_mb = int(W.unique_kv_bytes(w) * 2 / 2 ** 20 * 1.1) + w.n_seqs * 2 + 64  # fp32 pool + empty tails
        attn = ref.Attention(n_heads=heads, d_head=w.d_head, chunk_size=w.chunk_size, memory_mb=need_mb,
                             dtype=torch.float32, device=torch.device("cpu"))
        rows = W.populate(attn, w)
        q = w.q[rows].contiguous()
        fwd = lambda: attn.forward(q, 0)
    else:
        kind = "port"
        cores = 1
        from chunk_attn_oracle import Attention as OracleAttention
        attn = OracleAttention(heads, w.d_head, w.chunk_size)
        rows = W.populate(attn, w, as_numpy=True)
        q = w.q[rows].numpy()
        fwd = lambda: attn.forward(q, 0)
    n_warm, t_w0 = 0, time.perf_counter()
    while n_warm < max(1, warmup) and (n_warm == 0 or time.perf_counter() - t_w0 < 30.0):
        fwd()
        n_warm += 1
    per = (time.perf_counter() - t_w0) / n_warm
    n = max(1, min(steps, int(max_seconds / max(per, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(n):
        fwd()
    dt = (time.perf_counter() - t0) / n
    us = dt * 1e6 * scale_up
    sample = "%s in fp32, %d of %d heads%s, %d timed forwards (partition 0, chunk-first) after %d warm-up" % (
        name, heads, heads_full, " (time x%g)" % scale_up if scale_up != 1 else "", n, n_warm)
    res = {"value": us, "unit": "us", "cores": cores, "kind": kind, "sample": sample, "cpu_model": cpu_model(),
           "warmup": n_warm}
    if kind == "reference":  # its sequence-first-only path as well, a few forwards
        try:
            attn.forward(q, 2)
            m = max(1, min(n, 5))
            t0 = time.perf_counter()
            for _ in range(m):
                attn.forward(q, 2)
            res["partition2_sequence_first_us"] = (time.perf_counter() - t0) / m * 1e6 * scale_up
        except Exception as exc:  # reported, never a gate
            res["partition2_sequence_first_us"] = "failed: %s" % str(exc)[:120]
    return res, n


def time_reference_cpu_cfg4(steps, max_seconds):
    """Configuration 4 on the reference's CPU path: the initial tree (128 sequences), then decode steps of
    append_token + forward, timed whole, as many as fit in the budget (the replacements of the full trace are
    left out of the sample; they cost the CPU path nothing measurable beside a forward)."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from ref_loader import load_reference
    import synthetic_workloads as W
    ref = load_reference("cpu")
    cores = host_threads()
    cfg = W.Config4(gen_device="cpu")
    if ref is not None:
        kind = "reference"
        attn = ref.Attention(n_heads=32, d_head=128, chunk_size=64, memory_mb=2000, dtype=torch.float32,
                             device=torch.device("cpu"))
        conv = lambda t: t
    else:
        kind, cores = "port", 1
        from chunk_attn_oracle import Attention as OracleAttention
        attn = OracleAttention(32, 128, 64)
        conv = lambda t: t.numpy()
    n_seqs = 0
    for segs in cfg.initial():
        tokens, k, v = W.cat_segments(segs)
        if kind == "reference":
            attn.add_seq(tokens=tokens, k=k, v=v)
        else:
            attn.add_seq(tokens, k.numpy(), v.numpy())
        n_seqs += 1
    times = []
    t_begin = time.perf_counter()
    for step in range(min(steps + 1, cfg.steps)):
        q, nk, nv = cfg.step_inputs(n_seqs)
        t0 = time.perf_counter()
        if kind == "reference":
            attn.append_token(tokens=[7_000_000 + step] * n_seqs, k=nk, v=nv)
            attn.forward(q, 0)
        else:
            attn.append_token([7_000_000 + step] * n_seqs, nk.numpy(), nv.numpy())
            attn.forward(q.numpy(), 0)
        if step > 0:
            times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > max_seconds and times:
            break
    us = statistics.mean(times) * 1e6
    return {"value": us, "unit": "us", "cores": cores, "kind": kind, "cpu_model": cpu_model(), "warmup": 1,
            "sample": "cfg4 in fp32: initial tree of 128 sequences, %d timed decode steps of append_token + forward "
                      "(partition 0) after 1 warm-up step, no replacements" % len(times)}, len(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name, why = workload_name(args)
    base, n = time_reference_cpu(name, args.steps, args.warmup)
    cfg = {"workload": describe(name, args.gpus), "workload_choice": why, "device": "host CPU, %d threads" % base["cores"]}
    if name == "cfg5":
        cfg["sample"] = "8 of 64 heads timed, time x 8 (the work is linear in heads)"
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "us", "n_gpus": args.gpus,
            "steps": n, "warmup": base["warmup"], "ms_per_step": base["value"] / 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": cfg, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def time_reference_cuda(name, dev, steps, warmup):
    """The reference's own CUDA kernels (unmodified sources recompiled for sm_100a into oracle/_ref/cuda)
    on the same workload, same GPU, same run: CUDA events around `steps` forwards.  Its chunk-first
    kernel reads q rows past the batch, so q is the head of a zero-padded buffer; it only supports
    batches of 16/32/48/64/96/128 rows with sharing."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from ref_loader import load_reference
    import synthetic_workloads as W
    ref = load_reference("cuda")
    if ref is None:
        return {"us_per_step": None, "note": "oracle/_ref/cuda is not built"}
    w = make_workload(name, total_heads(name), "cpu" if name == "cfg2" else dev)
    if w.n_seqs > 128:
        return time_reference_cuda_standins(ref, w, dev, max(3, min(steps, 10)))
    chunk_bytes = w.n_heads * 2 * 64 * 128 * 2
    n_chunks = W.unique_kv_bytes(w) // chunk_bytes + w.n_seqs + 8
    ra = ref.Attention(n_heads=w.n_heads, d_head=128, chunk_size=64, memory_mb=(n_chunks * chunk_bytes >> 20) + 2,
                       dtype=torch.float16, device=dev)
    rows = W.populate(ra, w, device=dev, dtype=torch.float16)
    qbuf = torch.zeros(w.n_seqs + 160, w.n_heads, 128, device=dev, dtype=torch.float16)
    qbuf[:w.n_seqs] = w.q[rows].to(dev, torch.float16)
    q = qbuf[:w.n_seqs]
    for _ in range(max(3, warmup)):
        ra.forward(q)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ra.forward(q)
    e1.record()
    torch.cuda.synchronize()
    return {"us_per_step": e0.elapsed_time(e1) / steps * 1e3, "steps": steps,
            "note": "reference CUDA kernels recompiled for sm_100a, same inputs, same GPU, same run"}


def time_reference_cuda_standins(ref, w, dev, steps):
    """The reference's chunk-first kernel exists for batches of 16 to 128 rows only
    (cpp/chunk_attn/kernel_cuda.cu:1166-1187).  For a larger batch two stand-ins are timed: (a) the batch
    cut into caches of at most 128 sequences run one after the other (the shared prefix is then stored and
    read once per cache), (b) one cache with tpp_threshold above the batch size, i.e. its sequence-first
    kernel alone (the shared prefix is read once per sequence)."""
    import dataclasses
    import torch
    import synthetic_workloads as W
    chunk_bytes = w.n_heads * 2 * 64 * 128 * 2
    out = {"us_per_step": None, "note": "the reference's chunk-first kernel supports at most 128 rows: stand-ins timed"}

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps * 1e3

    def padded_q(q):
        buf = torch.zeros(q.shape[0] + 160, w.n_heads, 128, device=dev, dtype=torch.float16)
        buf[:q.shape[0]] = q.to(dev, torch.float16)
        return buf[:q.shape[0]]

    try:
        parts = []
        for lo in range(0, w.n_seqs, 128):
            sub = dataclasses.replace(w, seqs=w.seqs[lo:lo + 128], q=w.q[lo:lo + 128])
            n_chunks = W.unique_kv_bytes(sub) // chunk_bytes + sub.n_seqs + 8
            ra = ref.Attention(n_heads=w.n_heads, d_head=128, chunk_size=64, memory_mb=(n_chunks * chunk_bytes >> 20) + 2,
                               dtype=torch.float16, device=dev)
            rows = W.populate(ra, sub, device=dev, dtype=torch.float16)
            parts.append((ra, padded_q(sub.q[rows])))
        out["split_into_caches_of_128_us_per_step"] = timed(lambda: [ra.forward(q) for ra, q in parts])
        del parts
        torch.cuda.empty_cache()
    except Exception as exc:  # reported, never a gate
        out["split_into_caches_of_128_us_per_step"] = "failed: %s" % str(exc)[:160]
    try:
        n_chunks = W.unique_kv_bytes(w) // chunk_bytes + w.n_seqs + 8
        ra = ref.Attention(n_heads=w.n_heads, d_head=128, chunk_size=64, memory_mb=(n_chunks * chunk_bytes >> 20) + 2,
                           tpp_threshold=w.n_seqs, dtype=torch.float16, device=dev)
        rows = W.populate(ra, w, device=dev, dtype=torch.float16)
        q = padded_q(w.q[rows])
        out["sequence_first_only_us_per_step"] = timed(lambda: ra.forward(q))
        del ra
        torch.cuda.empty_cache()
    except Exception as exc:
        out["sequence_first_only_us_per_step"] = "failed: %s" % str(exc)[:160]
    out["steps"] = steps
    return out



# ---- this engine: the benchmark line ----------------------------------------------------------------------------------
def run_b200(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    name, why = workload_name(args)
    H = total_heads(name)
    if H % world:
        raise SystemExit("%d heads do not split over %d GPUs" % (H, world))
    h_local = H // world
    t_start = time.perf_counter()

    attn, engine, q, ukv_local, w, rows = build_engine(name, h_local, dev, args, sharded=world > 1, rank=rank,
                                                       keep_workload=True)
    gather_note = None
    if world > 1 and args.gather == "p2p":
        # the peer-store path must give exactly what the NCCL all-gather gives; if symmetric memory cannot
        # be set up on this machine, say so and time the NCCL path instead
        try:
            out_p2p = attn.forward(q, gather=True).clone()
            out_nccl = attn.gather(attn.forward_local(q))
            ok = torch.equal(out_p2p, out_nccl)
            flag = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) != 1:
                raise SystemExit("p2p gather differs from the NCCL all-gather")
            gather_note = "p2p, %s, %s barrier (verified equal to the NCCL all-gather on this batch)" % (
                "multimem.st through the switch" if attn.multicast_in_use() else "unicast peer stores", attn.barrier_kind)
        except SystemExit:
            raise
        except Exception as exc:
            attn.gather_mode = "nccl"
            gather_note = "nccl (p2p unavailable: %s)" % str(exc)[:120]
    elif world > 1:
        gather_note = "nccl"
    stats = engine.plan_stats()
    assert stats["unique_kv_bytes"] == ukv_local
    own_barrier_kernel = world > 1 and attn.gather_mode == "p2p" and attn.barrier_kind == "own"
    step = (lambda: attn.forward(q, gather=True)) if world > 1 else (lambda: attn.forward(q=q))

    # ---- parity of the tensor that is timed: sampled rows against dense fp64 from the seeded inputs ------------------
    out = step().clone()
    n_own = 12 if world == 1 else 6
    err = dense_parity(w, rows, out, q, sample_pairs(q.shape[0], h_local, n_own, 7 + rank), head_offset=rank * h_local)
    n_samples = n_own
    del w
    torch.cuda.empty_cache()
    if world > 1:
        # heads owned by another rank, regenerated here from that rank's seed (the trees are replicated, so the
        # rows are in the same order everywhere)
        other = (rank + 1) % world
        w2 = make_workload(name, h_local, dev, other)
        q2 = w2.q[rows].to(dev, torch.float16)
        err = max(err, dense_parity(w2, rows, out, q2, sample_pairs(q.shape[0], h_local, 6, 70 + rank),
                                    head_offset=other * h_local))
        n_samples += 6
        del w2, q2
        torch.cuda.empty_cache()
        t = torch.tensor([err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err = float(t.item())
        n_samples *= world
    parity = {"max_abs": err, "samples": n_samples, "tol": PARITY_TOL,
              "against": "dense fp64 on the seeded inputs" + (", own heads and another rank's heads of the gathered output" if world > 1 else "")}
    if not (err <= PARITY_TOL):
        raise SystemExit("parity: max-abs %.3g against dense fp64 exceeds %.1g" % (err, PARITY_TOL))
    del out

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    align_buf = torch.zeros(1, device=dev)

    def align():
        # Start every rank's timed region together ON THE DEVICE: a tiny all-reduce completes on all streams at the
        # same time whatever the processes' host-side skew, and a short device-side pause behind it lets every host
        # run ahead of its GPU before the first timed kernel starts.
        if world > 1:
            dist.all_reduce(align_buf)
            torch.cuda._sleep(400_000)

    W_, K = max(3, args.warmup), max(1, args.steps)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()      # before the warm-up: starting it takes milliseconds in which the GPU would idle
    for _ in range(max(W_, MIN_WARMUP_STEPS)):
        step()
    blocks = time_blocks(step, K, 1 + SPREAD_BLOCKS, sync_all, align)
    per_rank = None
    if world > 1:
        t = torch.tensor(blocks, device=dev, dtype=torch.float64)
        allb = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(allb, t)
        allb = torch.stack(allb).cpu()                       # [rank, block]
        blocks = [float(x) for x in allb.max(dim=0).values]  # a block takes as long as its slowest rank
        first = allb[:, 0] * 1e3
        per_rank = {"first_block_us_by_rank": [float(x) for x in first],
                    "min": float(first.min()), "median": float(first.median()), "max": float(first.max())}
    ms = blocks[0]

    # N > 1: where the step's time beyond the local attention goes (max over ranks each)
    breakdown = None
    if world > 1:
        def timed_loop(fn):
            for _ in range(3):
                fn()
            v = time_blocks(fn, K, 1, sync_all, align)[0] * 1e3
            t = torch.tensor([v], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        breakdown = {"step_us_per_rank": per_rank,
                     "local_forward_no_gather_us": timed_loop(lambda: attn.forward(q, gather=False))}
        if attn.gather_mode == "p2p":
            ql = attn._mine(q).contiguous()
            bufs = attn._symm_buffers(ql.shape[0], ql.dtype, ql.device)
            # rows stored into every rank's buffer, no barrier after the step (nobody reads the rows here)
            # = the step as the producer sees it when the READER of the gathered rows takes the barrier
            breakdown["rows_stored_into_peers_no_barrier_us"] = timed_loop(
                lambda: attn.local.forward_to_peers(q=ql, peer_out_ptrs=bufs[0][2], total_heads=attn.n_heads,
                                                    head_offset=attn.rank * attn.h_local, multicast_ptr=bufs[0][3]))
            if bufs[0][3]:
                breakdown["rows_stored_unicast_no_barrier_us"] = timed_loop(
                    lambda: attn.local.forward_to_peers(q=ql, peer_out_ptrs=bufs[0][2], total_heads=attn.n_heads,
                                                        head_offset=attn.rank * attn.h_local, multicast_ptr=0))
            breakdown["barrier_alone_us"] = timed_loop(lambda: attn._barrier(bufs[0][1]))
            breakdown["torch_symm_mem_barrier_alone_us"] = timed_loop(lambda: bufs[0][1].barrier(channel=0))
            breakdown["barrier_status"] = attn.barrier_status()

    kern = kernel_times(engine, q, K, args.split_phases) if stats["fast_path"] else None
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the public API with HOST buffers: pinned q -> device, forward (+ gather), this rank's
    # result rows back to pinned host memory, every step
    q_host = q.cpu().pin_memory()
    out_host = torch.empty((q.shape[0], h_local, 128), dtype=torch.float16).pin_memory()
    q_dev = torch.empty_like(q)
    own = slice(rank * h_local, (rank + 1) * h_local)

    def e2e_copies():
        # the reference's call pattern for host data: copy in, forward on device tensors, copy out.  On N > 1 the
        # gathered tensor stays on the device (its consumer is there); each rank hands the host its own head slice,
        # so the job as a whole moves every result row to the host once.
        q_dev.copy_(q_host, non_blocking=True)
        o = attn.forward(q_dev, gather=True)[:, own] if world > 1 else attn.forward(q=q_dev)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result on the host

    def e2e_host_call():
        # one call: queries copied in, result rows stored into out_host by the last kernel, returns when
        # they are there (ca_attention_host)
        attn.forward_host(q=q_host, out=out_host)

    e2e_step = e2e_host_call if world == 1 else e2e_copies
    e2e_call = "Attention.forward_host(q_pinned, out_pinned)" if world == 1 else \
        "copy_(q) + HeadShardedAttention.forward(gather=True) + copy_ of the rank's own head slice + stream sync"
    for _ in range(3):
        e2e_step()
    e2e_ms = time_blocks(e2e_step, K, 1, sync_all, align)[0]
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_alt = None
    if world == 1:  # the same round trip through forward() on device tensors and two explicit copies
        for _ in range(3):
            e2e_copies()
        e2e_alt = time_blocks(e2e_copies, K, 1, torch.cuda.synchronize)[0] * 1e3
    status = engine.device_status()

    # strong-scaling reference point: the same full-width workload on one GPU, same run (rank 0)
    single = None
    if world > 1 and rank == 0:
        del attn, engine
        torch.cuda.empty_cache()
        a1, eng1, q1, _, _, _ = build_engine(name, H, dev, args)
        for _ in range(W_):
            a1.forward(q=q1)
        single = {"n_gpus": 1, "us_per_step": time_blocks(lambda: a1.forward(q=q1), K, 1, torch.cuda.synchronize)[0] * 1e3}
        del a1, eng1
    if world > 1:
        dist.barrier()

    if rank == 0:
        peak, peak_src = measured_peak()
        line = {"metric": METRIC, "value": ms * 1e3, "unit": "us", "n_gpus": world, "steps": K, "warmup": W_,
                "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": describe(name, world), "workload_choice": why,
                           "warmup_steps_run": max(W_, MIN_WARMUP_STEPS),
                           "l2": "unique K/V per GPU (%.0f MB) exceeds the 126 MB L2: no flush between steps" % (ukv_local / 1e6)
                           if ukv_local > 126e6 else "unique K/V per GPU (%.0f MB) fits in L2" % (ukv_local / 1e6),
                           "parallelism": "heads/%d" % world, "gather": gather_note,
                           "phases": "split" if args.split_phases else "fused", "tails": args.tails, "wide_runs": args.wide,
                           "plan": stats},
                "parity": parity,
                "unique_kv_bytes": ukv_local * world,
                "unique_kv_gbs_per_gpu": ukv_local / (ms * 1e-3) / 1e9,
                "hbm_frac_whole_step": ukv_local / (ms * 1e-3) / 1e9 / peak,
                "roofline": roofline_of(name, ukv_local, kern, peak, peak_src, world == 1) if kern else None,
                "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": q_host.numel() * 2 * world,
                        "d2h_bytes_per_step": out_host.numel() * 2 * world, "call": e2e_call,
                        "via_forward_and_two_copies_us": e2e_alt},
                "multi_gpu_breakdown": breakdown,
                # this library's kernels per step: the attention kernels, plus its own barrier kernel after the fused gather
                # (an NCCL all-gather or torch's barrier are library kernels and not counted)
                "gpu_launches": K * (stats["kernels_per_step"] + (1 if own_barrier_kernel else 0)),
                "clocks": clocks, "device_status": status}
        line.update(spread_of([b * 1e3 for b in blocks]))
        if single:
            line["strong_scaling_ref"] = single
        attn = engine = None
        torch.cuda.empty_cache()
        auto = world == 1 and args.workload == "auto"
        if auto and name == "cfg5" and not args.no_scale_point:
            # this run is the N = 1 point of the cfg5 series: the headline configuration beside it, same run
            try:
                line["headline_cfg2"] = measure_static("cfg2", dev, 200, 10, args, ref_cuda=not args.no_ref_cuda)
                line["config"]["series"] = "N = 1 point of the cfg5 series (several GPUs visible); cfg2 in headline_cfg2"
            except Exception as exc:
                line["headline_cfg2"] = {"us_per_step": None, "note": "failed: %s" % str(exc)[:200]}
        if auto and name == "cfg2" and not args.no_scale_point:
            # The multi-GPU runs of this benchmark use cfg5 (strong scaling over heads).  Its one-GPU point,
            # measured here in the same run, is what their values compare with — not `value` above.
            try:
                a5, _, q5, ukv5, _, _ = build_engine("cfg5", total_heads("cfg5"), dev, args)
                for _ in range(5):
                    a5.forward(q=q5)
                us5 = time_blocks(lambda: a5.forward(q=q5), 30, 1, torch.cuda.synchronize)[0] * 1e3
                line["scale_series_n1"] = {"workload": describe("cfg5", 1), "us_per_step": us5, "steps": 30,
                                           "hbm_frac_whole_step": ukv5 / (us5 * 1e-6) / 1e9 / peak}
                del a5, q5
                torch.cuda.empty_cache()
            except Exception as exc:
                line["scale_series_n1"] = {"us_per_step": None, "note": "failed: %s" % str(exc)[:200]}
        if world == 1 and not args.no_ref_cuda:
            try:
                line["reference_cuda"] = time_reference_cuda(name, dev, min(K, 100), W_)
            except Exception as exc:  # reported, never a gate
                line["reference_cuda"] = {"us_per_step": None, "note": "failed: %s" % str(exc)[:200]}
        if auto and not args.no_other_configs:   # also beside the cfg5 point of a series: every configuration in every one-GPU line
            line["other_configs"] = other_configs(dev, args, t_start)
        if not args.no_cpu_baseline and world == 1:
            try:
                line["cpu_baseline"], _ = time_reference_cpu(name, 10, 1, max_seconds=25.0)
            except Exception as exc:  # the baseline is reported, never a gate
                line["cpu_baseline"] = {"value": None, "unit": "us", "cores": 0, "kind": "unavailable",
                                        "sample": "failed: %s" % exc}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def other_configs(dev, args, t_start):
    """The configurations the headline is not quoted on, each measured in this same run with its own clock record:
    cfg3 at its five shared-prefix lengths and cfg4, within a stated time budget (what does not fit is listed as
    skipped, never guessed)."""
    out = {"budget_s": args.other_budget, "entries": {}}
    t0 = time.perf_counter()
    for s in CFG3_SHARED:
        key = "cfg3_s%d" % s
        if time.perf_counter() - t0 > args.other_budget:
            out["entries"][key] = {"skipped": "time budget"}
            continue
        try:
            out["entries"][key] = measure_static(key, dev, 30, 5, args, n_parity=4, ref_cuda=not args.no_ref_cuda)
        except SystemExit:
            raise
        except Exception as exc:
            out["entries"][key] = {"us_per_step": None, "note": "failed: %s" % str(exc)[:200]}
    if time.perf_counter() - t0 > args.other_budget:
        out["entries"]["cfg4"] = {"skipped": "time budget"}
    else:
        try:
            out["entries"]["cfg4"] = measure_cfg4(dev, args, passes=1, with_e2e=True)
        except SystemExit:
            raise
        except Exception as exc:
            out["entries"]["cfg4"] = {"us_per_step": None, "note": "failed: %s" % str(exc)[:200]}
    out["seconds"] = time.perf_counter() - t0
    return out


def run_cfg4(args):
    """`--workload cfg4`: the full line for configuration 4 (value = append + work-list update + forward)."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    res = measure_cfg4(dev, args, passes=max(1, args.steps // 64), with_e2e=True)
    line = {"metric": METRIC, "value": res["us_per_step"], "unit": "us", "n_gpus": 1, "steps": res["steps"],
            "warmup": res["warmup"], "ms_per_step": res["us_per_step"] / 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": res["workload"], "workload_choice": "--workload", "l2": res["l2"]},
            "gpu_launches": res["steps"] * res["gpu_launches_per_step"]}
    for k in ("parity", "roofline", "e2e", "clocks", "device_status", "forward_us", "forward_us_median",
              "unique_kv_bytes_mean", "hbm_frac", "host_us_append_and_update", "step_minus_forward_us",
              "us_per_step_each_step_alone", "hbm_frac_forward_alone", "host_us_append_and_update_back_to_back", "timing", "value_median",
              "value_min", "value_max", "blocks"):
        line[k] = res.get(k)
    if not args.no_cpu_baseline:
        try:
            line["cpu_baseline"], _ = time_reference_cpu("cfg4", 10, 1, max_seconds=25.0)
        except Exception as exc:
            line["cpu_baseline"] = {"value": None, "unit": "us", "cores": 0, "kind": "unavailable",
                                    "sample": "failed: %s" % exc}
    emit(line)



def run_llama(args):
    """The reference's offline decoder benchmark (tests/benchmark_chunk_attn.py:131-175): a ONE-layer
    Llama-7B-shaped decoder (hidden 4096, 32 heads, MLP 11008, vocabulary 32000; random weights, there
    are no checkpoints here), `batch` prompts of `n_prompt` tokens of which `n_shared` are common,
    prefill + `n_completion` greedy decode steps; tokens/s = batch * n_completion / wall time of
    prefill + decode, as the reference computes it.  The decode step is also split with CUDA events
    into the attention calls (append_token + forward) and the rest (GEMMs, norms, rotary, sampling)."""
    import random
    import torch
    from chunk_attn.models.llama_hf import LlamaConfig, LlamaForCausalLM
    from chunk_attn.models.sequence import Sequence
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    batch, n_prompt, n_completion = args.llama_batch, args.llama_prompt, args.llama_completion
    n_shared = args.llama_shared
    cfg = LlamaConfig(num_hidden_layers=1, chunk_attn_kvcache_gb=8.0, torch_dtype=torch.float16, torch_device="cuda:0")
    model = LlamaForCausalLM(cfg, seed=0).to(device=dev, dtype=torch.float16).eval()
    rnd = random.Random(0)

    def prompts():
        return [[42] * n_shared + [rnd.randint(10, 100) for _ in range(n_prompt - n_shared)] for _ in range(batch)]

    model([Sequence(prompt_tokens=[42])], None, prefill=True)  # warm-up of the GEMM paths, as the reference does
    kv_caches = model.create_kv_caches()
    attn_ms = []
    kv = kv_caches[0]
    orig_append, orig_forward = kv.append_token, kv.forward

    class Timed:
        """Stands in front of the layer's cache: CUDA events around append_token .. forward."""
        def __init__(self):
            self.pairs = []
        def __getattr__(self, name):
            return getattr(kv, name)
        def append_token(self, **kw):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._e0 = e
            return orig_append(**kw)
        def forward(self, **kw):
            out = orig_forward(**kw)
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.pairs.append((self._e0, e))
            return out

    runs = []
    for rep in range(args.warmup_runs + args.runs):
        for c in kv_caches:
            c.clear()
        timed = Timed()
        seq_ids = prompts()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        seqs = [Sequence(prompt_tokens=p) for p in seq_ids]
        new_tokens = model(seqs, [timed], prefill=True)
        for s, t in zip(seqs, new_tokens):
            s.append(t)
        order = []
        for s in seqs:
            order.insert(s.index, s)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        for _ in range(n_completion):
            new_tokens = model(order, [timed], prefill=False)
            for s, t in zip(order, new_tokens):
                s.append(t)
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        if rep >= args.warmup_runs:
            runs.append({"tps": batch * n_completion / (t3 - t1), "prefill_ms": (t2 - t1) * 1e3,
                         "decode_ms_per_step": (t3 - t2) * 1e3 / n_completion,
                         "attention_us_per_step": statistics.mean(a.elapsed_time(b) for a, b in timed.pairs) * 1e3})
    best = max(runs, key=lambda r: r["tps"])
    st = kv.plan_stats()
    line = {"metric": "llama_1layer_offline_tps", "value": statistics.median(r["tps"] for r in runs), "unit": "tokens/s",
            "n_gpus": 1, "steps": len(runs) * n_completion, "warmup": args.warmup_runs * n_completion,
            "ms_per_step": statistics.median(r["decode_ms_per_step"] for r in runs), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama: 1-layer Llama-7B-shaped decoder (hidden 4096, 32 heads, d128, chunk 64, random fp16 "
                                   "weights), batch %d, prompt %d (%d shared), %d greedy decode steps; tokens/s over prefill + "
                                   "decode wall time" % (batch, n_prompt, n_shared, n_completion)},
            "runs": runs, "best_tps": best["tps"], "unique_kv_bytes_final": st["unique_kv_bytes"],
            "n_shared_chunks_final": st["n_shared_chunks"], "device_status": kv.device_status()}
    emit(line)




def emit(line):
    """The one JSON line goes to the process's original stdout; everything else any library prints
    (NCCL's version banner, the reference's logger) was diverted to stderr in main()."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = 1


def main():
    global _REAL_STDOUT
    args = parse()
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)  # C-level and Python-level prints now land on stderr
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "cfg4":
        run_cfg4(args)
    elif args.workload == "llama":
        run_llama(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
