"""The C-ABI library loads without a GPU, exports every symbol the public header declares, and its
GPU entry points fail loudly (never fall back) when no device is usable."""
import ctypes as C
import os
import re

import pytest
import torch

from chunk_attn import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "chunk_attn_b200.h")).read()
    return sorted(set(re.findall(r"CA_API\s+[\w\s\*]+?\b(ca_\w+)\s*\(", text)))


def test_header_and_library_agree():
    declared = declared_symbols()
    assert len(declared) >= 22
    assert declared == sorted(cabi.EXPORTED)
    for name in declared:
        assert hasattr(cabi.lib, name), name


def test_header_constants_match_the_ctypes_binding():
    # every CA_OPT_*, CA_ERR_*, CA_DTYPE_* and CA_PARTITION_* the header defines has the same value in cabi.py
    text = open(os.path.join(ROOT, "include", "chunk_attn_b200.h")).read()
    defines = dict(re.findall(r"^#define\s+(CA_(?:OPT|ERR|DTYPE|PARTITION)_\w+)\s+\(?(-?\d+)\)?\s*$", text, re.M))
    assert len([k for k in defines if k.startswith("CA_OPT_")]) >= 10
    for name, value in defines.items():
        if hasattr(cabi, name):
            assert getattr(cabi, name) == int(value), name
    for name in ("CA_OPT_WIDE_RUNS", "CA_OPT_WAIT_LIMIT_CYCLES", "CA_OPT_TRACE", "CA_OPT_FINISH_IN_TAILS", "CA_OPT_NUM_CTAS"):
        assert name in defines and hasattr(cabi, name), name


def test_host_only_entry_points():
    assert cabi.lib.ca_version() >= 100
    assert cabi.lib.ca_chunk_bytes(32, 128, 64, cabi.CA_DTYPE_F16) == 1 << 20
    assert cabi.lib.ca_chunk_bytes(32, 128, 64, 7) == -1
    # the tile layout: a permutation of the tile's elements; rows of a multiple of 128 bytes are stored as
    # 128-byte panels with the granules of a token's line XOR-swizzled by (token & 7), others row-major
    for d, C_, dt, es in ((128, 64, cabi.CA_DTYPE_F16, 2), (64, 32, cabi.CA_DTYPE_F32, 4), (4, 2, cabi.CA_DTYPE_F32, 4),
                          (20, 5, cabi.CA_DTYPE_F16, 2), (256, 16, cabi.CA_DTYPE_F16, 2)):
        per16 = 16 // es
        panelled = d % per16 == 0 and (d // per16) % 8 == 0
        offs = [[cabi.lib.ca_tile_elem_offset(d, C_, dt, t, e) for e in range(d)] for t in range(C_)]
        assert sorted(o for row in offs for o in row) == list(range(C_ * d))
        for t in range(C_):
            for e in range(d):
                if panelled:
                    gran, within = divmod(e, per16)
                    want = ((gran >> 3) * C_ + t) * 8 * per16 + ((gran & 7) ^ (t & 7)) * per16 + within
                else:
                    want = t * d + e
                assert offs[t][e] == want
    assert cabi.lib.ca_tile_elem_offset(128, 64, cabi.CA_DTYPE_F16, 64, 0) == -1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour without a device")
def test_gpu_entry_points_fail_loudly_without_a_device():
    h = C.c_void_p()
    rc = cabi.lib.ca_context_create(C.byref(h), 0, 2, 128, 64, cabi.CA_DTYPE_F16, None, 0, 1)
    assert rc == cabi.CA_ERR_CUDA and not h.value
    assert len(cabi.lib.ca_last_error()) > 0
    from chunk_attn import Attention
    with pytest.raises(RuntimeError, match="no CPU path"):
        Attention(n_heads=2, d_head=4, chunk_size=2, memory_mb=1, dtype=torch.float32, device=torch.device("cpu"))


def test_null_and_bad_arguments():
    assert cabi.lib.ca_context_create(None, 0, 2, 128, 64, 0, None, 0, 1) == cabi.CA_ERR_INVALID
    h = C.c_void_p()
    assert cabi.lib.ca_context_create(C.byref(h), 0, 2, 128, 64, 9, None, 0, 1) == cabi.CA_ERR_INVALID
    assert cabi.lib.ca_context_create(C.byref(h), 0, 2, 512, 64, 0, None, 0, 1) == cabi.CA_ERR_INVALID
    assert cabi.lib.ca_attention(None, None, None, 0, 0, None) == cabi.CA_ERR_INVALID
    assert cabi.lib.ca_append_kv(None, None, None, 0, None) == cabi.CA_ERR_INVALID
    assert cabi.lib.ca_context_delta_tokens(None) == -1
    cabi.lib.ca_context_destroy(None)
    cabi.lib.ca_plan_destroy(None)
