"""Runtime services on one GPU: the flag barrier of the push-style exchange (bounded wait and
its status path) and the per-record stream tickets."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _flag_arrays(n):
    """`n` peer-style flag arrays in this process's own device memory (as views and as a table)."""
    from mole_b200._lib import check, lib
    from mole_b200.core import _DeviceBytes
    ptrs, views = [], []
    for _ in range(n):
        p = C.c_void_p()
        check(lib.mole_peer_alloc(256, C.byref(p)))
        ptrs.append(p.value)
        views.append(torch.as_tensor(_DeviceBytes(p.value, 256), device="cuda").view(torch.int32))
    return ptrs, views, (C.c_void_p * n)(*ptrs)


def _free(ptrs):
    from mole_b200._lib import lib
    torch.cuda.synchronize()
    for p in ptrs:
        lib.mole_peer_free(C.c_void_p(p))


def test_flag_barrier_wait_runs_out_and_reports_the_missing_rank():
    """Rank 0 of 3 at a barrier that rank 2 never reaches (its flag is never set): the kernel
    gives up after the 5 ms limit, records 40 + 2 in the fault word and returns -- the stream and
    the context stay usable.  (The failure is a flag that nothing sets; no kernel is left waiting.)"""
    from mole_b200 import ops
    from mole_b200._lib import check, lib
    assert ops.device_fault() == 0
    ptrs, views, table = _flag_arrays(3)
    views[0][1] = 1                     # rank 1 has arrived at barrier 1; rank 2 has not
    torch.cuda.synchronize()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    check(lib.mole_peer_barrier(table, 3, 0, 1, 5_000_000, stream))
    t1.record()
    torch.cuda.synchronize()
    assert 4.0 < t0.elapsed_time(t1) < 200.0            # waited about the limit, not forever
    assert ops.device_fault() == 42                     # read and cleared
    assert ops.device_fault() == 0
    # this rank's own arrival was published to both peers before it started waiting
    assert int(views[1][0]) == 1 and int(views[2][0]) == 1
    # the context is intact: an ordinary kernel still runs
    assert float(torch.ones(8, device="cuda").sum()) == 8.0
    _free(ptrs)


def test_flag_barrier_passes_when_every_peer_has_arrived():
    from mole_b200 import ops
    from mole_b200._lib import check, lib
    ptrs, views, table = _flag_arrays(2)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for seq in (1, 2, 3):
        views[0][1] = seq + 1           # the peer may already be one barrier ahead
        torch.cuda.synchronize()
        check(lib.mole_peer_barrier(table, 2, 0, seq, 5_000_000, stream))
        torch.cuda.synchronize()
        assert ops.device_fault() == 0
        assert int(views[1][0]) == seq
    with pytest.raises(Exception):
        check(lib.mole_peer_barrier(table, 2, 0, 4, 0, stream))        # a wait without a limit is refused
    _free(ptrs)


def test_stream_tickets_order_only_what_they_name():
    """A ticket taken on stream A orders stream B behind the work A had been given up to the
    ticket, and an unknown or recycled ticket is refused."""
    from mole_b200._lib import MoleError
    from mole_b200.utils.Ustream import ExpertStreamCtx
    sctx = ExpertStreamCtx.get(torch.device("cuda", torch.cuda.current_device()))
    a, b = sctx.comm_stream(), sctx.tran_stream()
    x = torch.zeros(1 << 20, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(a):
        torch.cuda._sleep(20_000_000)           # ~10 ms
        x.add_(1.0)
        ticket = ExpertStreamCtx.record(a)
    ExpertStreamCtx.wait_ticket(b, ticket)
    with torch.cuda.stream(b):
        y = x.clone()                           # must see the add
    torch.cuda.synchronize()
    assert float(y.min()) == 1.0
    with pytest.raises(MoleError):
        ExpertStreamCtx.wait_ticket(b, ticket + 10_000)
