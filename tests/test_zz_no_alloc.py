"""ca_attention_static, the decode step for callers that cannot allocate device memory (a plugin in
a serving process whose framework owns all of the GPU's memory, a latency-critical loop that must
not hit cudaMalloc's device-wide synchronisation).  It keeps the partial results in a fixed array
inside the library instead of scratch grown with cudaMalloc, and reads its work list from device
arrays the caller owns.

Checked here through the C ABI against the ordinary entry point, ca_attention, on the same pool
and the same queries, twice in a row: the second call finds the first call's partial rows still in
the shared scratch and must not be disturbed by them.  Collected last on purpose (file name), so a
run that stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from chunk_attn import cabi, workloads as W
from gpu_helpers import CabiEngine

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3  # the tolerance of the other fp16 parity tests


def device_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def test_static_entry_point_matches_ca_attention_twice():
    H = 4
    w = W.single_level("noalloc", H, 128, 64, torch.float16, 9, 5 * 64, 2 * 64 + 11, 90, 0.5)
    eng = CabiEngine(H, 128, 64, torch.float16, max_chunks=128)
    rows = W.populate(eng, w)
    infos = eng.tree.get_chunks()

    # the caller's side of the allocation-free call: build the work list on the host and put it in
    # device memory of its own, once
    plan = cabi.Plan(infos, len(rows), H, chunk_size=64, n_ctas=296, max_chunks=128)
    st = plan.stats()
    assert 0 < st["n_slots"] <= cabi.CA_STATIC_MAX_SLOTS
    items = device_i32(plan.array(cabi.PLAN_ITEMS))
    merge_off = device_i32(plan.array(cabi.PLAN_MERGE_OFF))
    merge_slots = device_i32(plan.array(cabi.PLAN_MERGE_SLOTS))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    g = torch.Generator().manual_seed(91)
    for call in range(2):
        q = (torch.randn(len(rows), H, 128, generator=g) * (0.5 if call == 0 else 4.0)).to(torch.float16).cuda()
        expected = eng.forward(q)                     # ca_attention, scratch from cudaMalloc
        out = torch.full_like(q, float("nan"))
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        cabi.check(cabi.lib.ca_attention_static(
            eng.pool.data_ptr(), H, q.data_ptr(), out.data_ptr(), len(rows), items.data_ptr(), st["n_items"],
            st["n_ctas"], merge_off.data_ptr(), merge_slots.data_ptr(), st["n_slots"], 0, status.data_ptr(),
            stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.isfinite(out).all()
        assert (out.float() - expected.float()).abs().max().item() < TOL_F16, "call %d" % call

    # a work list that does not fit the fixed scratch is refused before anything is launched
    rc = cabi.lib.ca_attention_static(
        eng.pool.data_ptr(), H, q.data_ptr(), out.data_ptr(), len(rows), items.data_ptr(), st["n_items"],
        st["n_ctas"], merge_off.data_ptr(), merge_slots.data_ptr(), cabi.CA_STATIC_MAX_SLOTS + 1, 0, None, stream)
    assert rc == cabi.CA_ERR_INVALID
    assert b"CA_STATIC_MAX_SLOTS" in cabi.lib.ca_last_error()
