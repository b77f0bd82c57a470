"""Failure paths of the attention kernels, exercised without faulting, trapping or hanging the GPU: every wait in
the kernels is bounded, and on expiry a kernel records a status code, unwinds and returns, leaving the context
usable.  The wait is made to run out by a test-only option that makes one CTA's producer stop feeding its
consumer warps (a flag that nothing sets), with the limit lowered to about a millisecond."""
import pytest
import torch

from chunk_attn import cabi
import synthetic_workloads as W
from gpu_helpers import CabiEngine, max_abs, oracle_for, round_to

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3


def test_wait_that_runs_out_is_reported_and_the_context_survives():
    w = W.single_level("failure", 4, 128, 64, torch.float16, 9, 5 * 64, 2 * 64 + 11, 77, 0.5)
    eng = CabiEngine(4, 128, 64, torch.float16, max_chunks=128)
    ora, orows = oracle_for(w)
    rows = W.populate(eng, w)
    assert rows == orows
    q = round_to(w.q[rows], torch.float16)
    ref = ora.forward(q.numpy(), 0)
    assert max_abs(eng.forward(q).float().cpu().numpy(), ref) < TOL_F16
    assert eng.ctx.status() == 0

    # one CTA's consumers are never handed their first item: their wait runs out after ~1 ms of SM clock
    eng.ctx.set_option(cabi.CA_OPT_WAIT_LIMIT_CYCLES, 2_000_000)
    eng.ctx.set_option(cabi.CA_OPT_TEST_WITHHOLD_ITEM, 0)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    eng.forward(q)
    t1.record()
    torch.cuda.synchronize()                      # the kernel returned by itself
    assert t0.elapsed_time(t1) < 500.0            # ms: nowhere near the default two-second limit
    rc, word = eng.ctx.status_raw()
    assert rc == cabi.CA_ERR_DEVICE_STATUS and word == cabi.STATUS_FULL_WAIT_TIMEOUT
    assert b"status 1" in cabi.lib.ca_last_error()

    # the same context, cleared, computes the next ordinary step correctly
    eng.ctx.set_option(cabi.CA_OPT_TEST_WITHHOLD_ITEM, -1)
    eng.ctx.set_option(cabi.CA_OPT_WAIT_LIMIT_CYCLES, 4_000_000_000)
    eng.ctx.status_clear()
    for _ in range(2):
        assert max_abs(eng.forward(q).float().cpu().numpy(), ref) < TOL_F16
    assert eng.ctx.status() == 0


def test_option_ranges():
    eng = CabiEngine(2, 128, 64, torch.float16, max_chunks=8)
    with pytest.raises(cabi.CAError):
        eng.ctx.set_option(cabi.CA_OPT_WAIT_LIMIT_CYCLES, 10)   # a limit this short would fail ordinary waits


def test_peer_barrier_gives_up_after_its_limit_and_passes_when_the_peer_arrives():
    # the barrier of the fused multi-GPU gather, on one GPU: two flag arrays stand in for two ranks.  Rank 0 signals
    # both arrays and waits for word 1 of its own, which nobody sets: after the 2 ms limit the kernel records status 6
    # and returns.  Once "rank 1" has arrived (its word written by hand) the same barrier passes.
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ptrs = [f.data_ptr() for f in flags]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    cabi.peer_barrier(ptrs, rank=0, epoch=1, timeout_ns=2_000_000, status_ptr=status.data_ptr())
    t1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == 6
    assert 1.5 < t0.elapsed_time(t1) < 200.0          # ms: the limit, not an endless spin
    assert flags[0][0].item() == 1 and flags[1][0].item() == 1   # rank 0's own arrival was published to both
    status.zero_()
    flags[0][1] = 1                                   # rank 1 arrives
    cabi.peer_barrier(ptrs, rank=0, epoch=1, timeout_ns=2_000_000, status_ptr=status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    flags[0][1] = 7                                   # a peer that is already further on does not hold anyone up
    cabi.peer_barrier(ptrs, rank=0, epoch=2, timeout_ns=2_000_000, status_ptr=status.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    with pytest.raises(cabi.CAError):
        cabi.peer_barrier(ptrs, rank=2, epoch=1)      # rank outside the group
