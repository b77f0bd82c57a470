"""ctypes binding of the C ABI in include/chunk_attn_b200.h (libchunk_attn_b200.so).

The `Attention` class most users want lives in the compiled module `chunk_attn.lib.chunk_attn_c`;
this thin binding exposes the layer underneath it (contexts, work lists, single kernels) for the
parity tests, the benchmark's per-kernel timing and the host-only planner checks.  It never
computes anything itself and has no fallback: a missing library is an ImportError.
"""
import ctypes as C
import os

import numpy as np

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libchunk_attn_b200.so")

CA_OK = 0
CA_ERR_INVALID, CA_ERR_CUDA, CA_ERR_STATE, CA_ERR_DEVICE_STATUS = -1, -2, -3, -4
CA_DTYPE_F16, CA_DTYPE_F32 = 0, 1
CA_OPT_SPLIT_PHASES, CA_OPT_NUM_CTAS, CA_OPT_SEQ_FIRST_TENSOR, CA_OPT_TRACE, CA_OPT_DEPENDENT_LAUNCH = 1, 2, 3, 4, 5
CA_OPT_WIDE_RUNS, CA_OPT_WAIT_LIMIT_CYCLES, CA_OPT_TEST_WITHHOLD_ITEM, CA_OPT_OVERLAP_KERNELS, CA_OPT_FINISH_IN_TAILS = 6, 7, 8, 9, 10
STATUS_FULL_WAIT_TIMEOUT, STATUS_EMPTY_WAIT_TIMEOUT, STATUS_DRAIN_TIMEOUT, STATUS_BAD_WORK_LIST, STATUS_BAD_POSITION = 1, 2, 3, 4, 5
PLAN_ITEMS = 0
(PLAN_MERGE_OFF, PLAN_MERGE_SLOTS, PLAN_PATH_OFF, PLAN_PATH_CHUNKS, PLAN_PATH_TOKENS, PLAN_TAIL_CHUNK,
 PLAN_TAIL_TOKENS, PLAN_WIDE_CHUNKS) = range(3, 11)

# every symbol include/chunk_attn_b200.h declares
EXPORTED = [
    "ca_last_error", "ca_version", "ca_chunk_bytes", "ca_tile_elem_offset", "ca_context_create",
    "ca_context_destroy", "ca_context_set_option", "ca_refresh_kernel_context", "ca_append_kv",
    "ca_context_delta_tokens", "ca_attention", "ca_attention_host", "ca_attention_to_peers", "ca_peer_barrier", "ca_attn_partials", "ca_attn_merge",
    "ca_scatter_prefill", "ca_scatter_rows", "ca_copy_chunks", "ca_read_chunk", "ca_status_read", "ca_status_clear", "ca_context_stats",
    "ca_context_read_trace",
    "ca_plan_build", "ca_plan_build_for_context", "ca_refresh_from_plan", "ca_plan_array", "ca_plan_stats_get", "ca_plan_destroy", "ca_attention_static", "ca_attention_static_status",
    "ca_rms_norm", "ca_fused_add_rms_norm", "ca_rotary_embedding",
]
CA_STATIC_MAX_SLOTS = 16384


class ChunkInfo(C.Structure):
    _fields_ = [("chunk_id", C.c_int32), ("n_tokens", C.c_int32), ("seq_begin", C.c_int32),
                ("seq_end", C.c_int32)]


class PlanStats(C.Structure):
    _fields_ = [("unique_kv_bytes", C.c_int64), ("n_chunks", C.c_int32), ("n_shared_chunks", C.c_int32),
                ("n_runs", C.c_int32), ("n_items", C.c_int32), ("n_slots", C.c_int32),
                ("n_ctas", C.c_int32), ("fast_path", C.c_int32), ("kernels_per_step", C.c_int32),
                ("n_items_cf", C.c_int32), ("n_items_short", C.c_int32), ("n_items_wide", C.c_int32)]

    def as_dict(self):
        return {f: getattr(self, f) for f, _ in self._fields_}


class CAError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("chunk_attn_b200 error %d: %s" % (code, msg))
        self.code = code


def _load():
    if not os.path.exists(_LIB_PATH):
        raise ImportError("libchunk_attn_b200.so is not built: run `python build.py` in chunk-attention_b200/")
    lib = C.CDLL(_LIB_PATH)
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    sig = {
        "ca_last_error": (C.c_char_p, []),
        "ca_version": (i32, []),
        "ca_chunk_bytes": (i64, [i32, i32, i32, i32]),
        "ca_tile_elem_offset": (i64, [i32, i32, i32, i32, i32]),
        "ca_context_create": (i32, [C.POINTER(vp), i32, i32, i32, i32, i32, vp, i64, i32]),
        "ca_context_destroy": (None, [vp]),
        "ca_context_set_option": (i32, [vp, i32, i64]),
        "ca_refresh_kernel_context": (i32, [vp, C.POINTER(ChunkInfo), i32, i32, vp]),
        "ca_append_kv": (i32, [vp, vp, vp, i32, vp]),
        "ca_context_delta_tokens": (i32, [vp]),
        "ca_attention": (i32, [vp, vp, vp, i32, i32, vp]),
        "ca_attention_host": (i32, [vp, vp, vp, i32, i32, vp]),
        "ca_attention_to_peers": (i32, [vp, vp, C.POINTER(vp), i32, vp, i32, i32, i32, vp]),
        "ca_peer_barrier": (i32, [C.POINTER(vp), i32, i32, C.c_uint32, i64, vp, vp]),
        "ca_attn_partials": (i32, [vp, vp, i32, i32, vp]),
        "ca_attn_merge": (i32, [vp, vp, i32, vp]),
        "ca_scatter_prefill": (i32, [vp, vp, vp, i64, i64, i32, i32, C.POINTER(C.c_int32), vp]),
        "ca_scatter_rows": (i32, [vp, vp, vp, i64, i64, i32, C.POINTER(C.c_int32), C.POINTER(C.c_int32), vp]),
        "ca_copy_chunks": (i32, [vp, C.POINTER(C.c_int32), C.POINTER(C.c_int32), i32, vp]),
        "ca_read_chunk": (i32, [vp, i32, i32, vp, vp, vp]),
        "ca_status_read": (i32, [vp, vp, C.POINTER(C.c_int32)]),
        "ca_status_clear": (i32, [vp, vp]),
        "ca_context_stats": (i32, [vp, C.POINTER(PlanStats)]),
        "ca_context_read_trace": (i32, [vp, C.POINTER(C.c_uint64), i32, C.POINTER(i32), vp]),
        "ca_plan_build": (i32, [C.POINTER(vp), C.POINTER(ChunkInfo), i32, i32, i32, i32, i32, i32, i64, i32, i32, i32]),
        "ca_plan_build_for_context": (i32, [vp, C.POINTER(vp), C.POINTER(ChunkInfo), i32, i32]),
        "ca_refresh_from_plan": (i32, [vp, vp, vp]),
        "ca_plan_array": (i32, [vp, i32, C.POINTER(C.POINTER(C.c_int32)), C.POINTER(i64)]),
        "ca_plan_stats_get": (i32, [vp, C.POINTER(PlanStats)]),
        "ca_plan_destroy": (None, [vp]),
        "ca_rms_norm": (i32, [vp, vp, vp, C.c_float, i64, i32, i32, vp]),
        "ca_fused_add_rms_norm": (i32, [vp, vp, vp, C.c_float, i64, i32, i32, vp]),
        "ca_rotary_embedding": (i32, [vp, vp, vp, vp, i32, i64, i64, i32, i32, i32, i64, i32, i32, i64, vp, vp]),
        "ca_attention_static": (i32, [vp, i32, vp, vp, i32, vp, i32, i32, vp, vp, i32, i32, vp, vp]),
        "ca_attention_static_status": (i32, [C.POINTER(C.c_int32), vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(rc):
    if rc != CA_OK:
        raise CAError(rc, (lib.ca_last_error() or b"").decode())
    return rc


def make_infos(infos):
    """infos: iterable of (chunk_id, n_tokens, seq_begin, seq_end) -> ctypes array."""
    infos = list(infos)
    arr = (ChunkInfo * max(1, len(infos)))()
    for i, (cid, nt, b, e) in enumerate(infos):
        arr[i] = ChunkInfo(cid, nt, b, e)
    return arr, len(infos)


def peer_barrier(flag_ptrs, rank, epoch, timeout_ns=2_000_000_000, status_ptr=None, stream=None):
    """Bounded barrier among the ranks whose flag arrays are flag_ptrs (device addresses), on `stream`."""
    import torch
    arr = (C.c_void_p * len(flag_ptrs))(*flag_ptrs)
    st = C.c_void_p(stream if stream is not None else torch.cuda.current_stream().cuda_stream)
    check(lib.ca_peer_barrier(arr, len(flag_ptrs), rank, epoch & 0xFFFFFFFF, timeout_ns, status_ptr, st))


class Plan:
    """Host-only work-list builder (no GPU needed)."""

    def __init__(self, infos, n_seqs, n_heads, chunk_size=64, tpp_threshold=1, n_ctas=296,
                 max_chunks=1 << 30, split_phases=False, seq_first_tensor=True, wide_runs=0):
        arr, n = make_infos(infos)
        self._h = C.c_void_p()
        check(lib.ca_plan_build(C.byref(self._h), arr, n, n_seqs, n_heads, chunk_size, tpp_threshold,
                                n_ctas, max_chunks, int(split_phases), int(seq_first_tensor), int(wide_runs)))

    def array(self, which):
        ptr, cnt = C.POINTER(C.c_int32)(), C.c_int64()
        check(lib.ca_plan_array(self._h, which, C.byref(ptr), C.byref(cnt)))
        if cnt.value == 0:
            return np.zeros(0, np.int32)
        return np.ctypeslib.as_array(ptr, shape=(cnt.value,)).copy()

    def items(self):
        return self.array(PLAN_ITEMS).reshape(-1, 16)

    def stats(self):
        st = PlanStats()
        check(lib.ca_plan_stats_get(self._h, C.byref(st)))
        return st.as_dict()

    def __del__(self):
        if getattr(self, "_h", None):
            lib.ca_plan_destroy(self._h)
            self._h = None


class Context:
    """A kernel context over a caller-owned pool (a torch uint8/any tensor on a CUDA device)."""

    def __init__(self, n_heads, d_head, chunk_size, dtype, pool_tensor, max_chunks, tpp_threshold=1, device=0):
        self.n_heads, self.d_head, self.chunk_size, self.dtype = n_heads, d_head, chunk_size, dtype
        self.pool = pool_tensor  # keep alive
        self.max_chunks = max_chunks
        self._h = C.c_void_p()
        ptr = pool_tensor.data_ptr() if pool_tensor is not None else None
        check(lib.ca_context_create(C.byref(self._h), device, n_heads, d_head, chunk_size, dtype, ptr,
                                    max_chunks, tpp_threshold))

    @staticmethod
    def _stream():
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def set_option(self, option, value):
        check(lib.ca_context_set_option(self._h, option, value))

    def refresh(self, infos, n_seqs):
        arr, n = make_infos(infos)
        check(lib.ca_refresh_kernel_context(self._h, arr, n, n_seqs, self._stream()))

    def append_kv(self, k, v):
        check(lib.ca_append_kv(self._h, k.data_ptr(), v.data_ptr(), k.shape[0], self._stream()))

    def attention(self, q, out, partition=0):
        check(lib.ca_attention(self._h, q.data_ptr(), out.data_ptr(), q.shape[0], partition, self._stream()))

    def attention_host(self, q_cpu, out_cpu, partition=0):
        """q_cpu, out_cpu: contiguous CPU tensors (pinned or not); returns when out_cpu holds the result."""
        assert not q_cpu.is_cuda and not out_cpu.is_cuda and q_cpu.is_contiguous() and out_cpu.is_contiguous()
        check(lib.ca_attention_host(self._h, q_cpu.data_ptr(), out_cpu.data_ptr(), q_cpu.shape[0], partition,
                                    self._stream()))

    def attention_to_peers(self, q, peer_ptrs, total_heads, head_offset, multicast_ptr=None):
        arr = (C.c_void_p * len(peer_ptrs))(*peer_ptrs)
        check(lib.ca_attention_to_peers(self._h, q.data_ptr(), arr, len(peer_ptrs), multicast_ptr, total_heads,
                                        head_offset, q.shape[0], self._stream()))

    def attn_partials(self, q, phases=3):
        check(lib.ca_attn_partials(self._h, q.data_ptr(), q.shape[0], phases, self._stream()))

    def attn_merge(self, out):
        check(lib.ca_attn_merge(self._h, out.data_ptr(), out.shape[0], self._stream()))

    def scatter_prefill(self, k, v, first_token, n_tokens, chunk_ids):
        assert k.stride(2) == 1 and v.stride(2) == 1 and k.stride() == v.stride()
        ids = (C.c_int32 * max(1, len(chunk_ids)))(*chunk_ids)
        check(lib.ca_scatter_prefill(self._h, k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
                                     first_token, n_tokens, ids, self._stream()))

    def scatter_rows(self, k, v, chunk_ids, rows):
        assert k.stride(2) == 1 and v.stride(2) == 1 and k.stride() == v.stride() and len(chunk_ids) == len(rows)
        ids = (C.c_int32 * max(1, len(chunk_ids)))(*chunk_ids)
        rr = (C.c_int32 * max(1, len(rows)))(*rows)
        check(lib.ca_scatter_rows(self._h, k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), len(chunk_ids),
                                  ids, rr, self._stream()))

    def copy_chunks(self, src, dst):
        s = (C.c_int32 * max(1, len(src)))(*src)
        d = (C.c_int32 * max(1, len(dst)))(*dst)
        check(lib.ca_copy_chunks(self._h, s, d, len(src), self._stream()))

    def read_chunk(self, chunk_id, n_tokens, k_out, v_out):
        check(lib.ca_read_chunk(self._h, chunk_id, n_tokens, k_out.data_ptr(), v_out.data_ptr(), self._stream()))

    def status(self):
        st = C.c_int32()
        check(lib.ca_status_read(self._h, self._stream(), C.byref(st)))
        return st.value

    def status_raw(self):
        """(return code, status word): CA_ERR_DEVICE_STATUS with the kernel's code when a kernel reported one."""
        st = C.c_int32()
        rc = lib.ca_status_read(self._h, self._stream(), C.byref(st))
        return rc, st.value

    def status_clear(self):
        check(lib.ca_status_clear(self._h, self._stream()))

    def stats(self):
        st = PlanStats()
        check(lib.ca_context_stats(self._h, C.byref(st)))
        return st.as_dict()

    def read_trace(self, max_ctas=4096):
        """[n_ctas, 8] uint64: ns of start, producer end, first / last consumer warp end; cycles of
        consumer warp 0 waiting for tiles, combining, producer waiting for free stages, warp 0 total."""
        buf = (C.c_uint64 * (8 * max_ctas))()
        n = C.c_int()
        check(lib.ca_context_read_trace(self._h, buf, max_ctas, C.byref(n), self._stream()))
        return np.ctypeslib.as_array(buf)[:8 * n.value].reshape(-1, 8).copy()

    def delta_tokens(self):
        return lib.ca_context_delta_tokens(self._h)

    def close(self):
        if getattr(self, "_h", None):
            lib.ca_context_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()
