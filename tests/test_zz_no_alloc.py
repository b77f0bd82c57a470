"""ca_attention_static, the decode step for callers that cannot allocate device memory (a plugin in
a serving process whose framework owns all of the GPU's memory, a latency-critical loop that must
not hit cudaMalloc's device-wide synchronisation).  It keeps the partial results in a fixed array
inside the library instead of scratch grown with cudaMalloc, and reads its work list from device
arrays the caller owns.

Checked here through the C ABI against the ordinary entry point, ca_attention, AND against the CPU
oracle, on the same pool and the same queries, several calls in a row: every call finds the previous
call's partial rows still in the shared scratch and must not be disturbed by them.  Tokens are
appended between calls (delta_tokens 0, 1, 5), the work list is cut for a handful of CTAs so that the
kernel's self-scheduling counter is really drawn from, one call uses the library's own status word,
free device memory is watched across the calls, and a work list that names a partial row outside the
scratch must come back as a status code, not as a wrong answer or a stray write.  Collected last on
purpose (file name), so a run that stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from chunk_attn import cabi
import synthetic_workloads as W
from gpu_helpers import CabiEngine, max_abs, oracle_for, round_to

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3  # the tolerance of the other fp16 parity tests


def device_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def call_static(eng, H, q, out, n_rows, items, st, merge_off, merge_slots, delta, status, n_slots=None):
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the item array holds every item once for all heads; ca_plan_stats counts the (item, head) pieces
    return cabi.lib.ca_attention_static(
        eng.pool.data_ptr(), H, q.data_ptr(), out.data_ptr(), n_rows, items.data_ptr(), st["n_items"] // H, st["n_ctas"],
        merge_off.data_ptr(), merge_slots.data_ptr(), st["n_slots"] if n_slots is None else n_slots, delta,
        status.data_ptr() if status is not None else None, stream)


@pytest.mark.parametrize("n_ctas", [296, 4])
def test_static_entry_point_matches_ca_attention_and_the_oracle(n_ctas):
    H = 4
    w = W.single_level("noalloc", H, 128, 64, torch.float16, 9, 5 * 64, 2 * 64 + 11, 90, 0.5)
    eng = CabiEngine(H, 128, 64, torch.float16, max_chunks=128)
    ora, orows = oracle_for(w)
    rows = W.populate(eng, w)
    assert rows == orows
    n = len(rows)
    eng.refresh()
    infos = eng.tree.get_chunks()

    # the caller's side of the allocation-free call: build the work list on the host and put it in
    # device memory of its own, once
    plan = cabi.Plan(infos, n, H, chunk_size=64, n_ctas=n_ctas, max_chunks=128)
    st = plan.stats()
    assert 0 < st["n_slots"] <= cabi.CA_STATIC_MAX_SLOTS
    if n_ctas == 4:
        assert st["n_items"] > 2 * st["n_ctas"]   # items beyond the fixed ones are drawn from the device counter
    items = device_i32(plan.array(cabi.PLAN_ITEMS))
    merge_off = device_i32(plan.array(cabi.PLAN_MERGE_OFF))
    merge_slots = device_i32(plan.array(cabi.PLAN_MERGE_SLOTS))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    g = torch.Generator().manual_seed(91)
    free_before = None
    delta = 0
    for call, appended in enumerate([0, 1, 4, 0]):     # delta_tokens 0, 1, 5, 5
        for _ in range(appended):
            nk, nv = torch.randn(n, H, 128, generator=g), torch.randn(n, H, 128, generator=g)
            # straight through ca_append_kv (the work list on the device is not rebuilt: delta_tokens counts)
            eng.ctx.append_kv(nk.to("cuda", torch.float16), nv.to("cuda", torch.float16))
            eng.tree.append_token([7000 + delta] * n)
            ora.append_token([7000 + delta] * n, round_to(nk, torch.float16).numpy(), round_to(nv, torch.float16).numpy())
            delta += 1
        assert eng.ctx.delta_tokens() == delta
        qf = round_to(torch.randn(n, H, 128, generator=g) * (0.5 if call % 2 == 0 else 4.0), torch.float16)
        q = qf.to("cuda", torch.float16)
        expected = torch.empty_like(q)
        eng.ctx.attention(q, expected)                 # ca_attention, scratch from cudaMalloc
        out = torch.full_like(q, float("nan"))
        use_own_word = call == 2                       # one call leaves the status to the library's own word
        if call == 1:
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        cabi.check(call_static(eng, H, q, out, n, items, st, merge_off, merge_slots, delta,
                               None if use_own_word else status))
        torch.cuda.synchronize()
        if use_own_word:
            word = C.c_int32(-1)
            cabi.check(cabi.lib.ca_attention_static_status(C.byref(word), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            assert word.value == 0
        else:
            assert int(status.item()) == 0
        assert torch.isfinite(out).all()
        assert (out.float() - expected.float()).abs().max().item() < TOL_F16, "call %d" % call
        assert max_abs(out.float().cpu().numpy(), ora.forward(qf.numpy(), 0)) < TOL_F16, "call %d vs oracle" % call
    # nothing was allocated on the device by the second and later calls
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before

    # a work list that does not fit the fixed scratch is refused before anything is launched
    rc = call_static(eng, H, q, out, n, items, st, merge_off, merge_slots, delta, None, n_slots=cabi.CA_STATIC_MAX_SLOTS + 1)
    assert rc == cabi.CA_ERR_INVALID
    assert b"CA_STATIC_MAX_SLOTS" in cabi.lib.ca_last_error()

    # a work list naming partial rows outside [0, n_slots): the entries are skipped on the device and reported
    bad_items = plan.array(cabi.PLAN_ITEMS).reshape(-1, 16).copy()
    bad_items[0, 4] = st["n_slots"] // H + 7           # slot_base of the first item (numbered per item, not per head)
    bad_merge = plan.array(cabi.PLAN_MERGE_SLOTS).copy()
    bad_merge[-1] = cabi.CA_STATIC_MAX_SLOTS + 123
    for it_dev, ms_dev in ((device_i32(bad_items.reshape(-1)), merge_slots), (items, device_i32(bad_merge))):
        status.zero_()
        cabi.check(call_static(eng, H, q, out, n, it_dev, st, merge_off, ms_dev, delta, status))
        torch.cuda.synchronize()
        assert int(status.item()) == cabi.STATUS_BAD_WORK_LIST
    # and the next well-formed call is right again
    cabi.check(call_static(eng, H, q, out, n, items, st, merge_off, merge_slots, delta, status))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert (out.float() - expected.float()).abs().max().item() < TOL_F16
