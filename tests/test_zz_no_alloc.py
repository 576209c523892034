"""The entry point that allocates nothing (``mole_gate_route_fwd_static``).

Some hosts of the library cannot give it a workspace: they handed all device memory to their own
pool at start-up, or must not trigger a driver allocation (and its implicit synchronisation)
where they call from.  For them the gate + routing build exists in a variant whose scratch is a
fixed 4 MiB array inside the library.  This test calls it through the C ABI twice in a row --
the second call sees the first call's leftovers in the shared scratch -- and requires the
results of the ordinary entry point, bit for bit.  It lives in a file of its own that sorts last
so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

FIELDS = ("scores", "idx", "slot", "gates", "counts", "offsets", "perm", "first_hist", "l_aux")


def _same(a, b):
    for f in FIELDS:
        assert torch.equal(getattr(a, f), getattr(b, f)), f"{f} differs from the workspace entry point"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_on_two_calls_in_a_row(dtype):
    from mole_b200 import ops
    g = torch.Generator().manual_seed(77)
    # two different problems, so that the second call meets scratch left by another shape
    shapes = [(4096, 512, 64, 2, 1.25), (1000, 256, 20, 3, 0.5)]
    for T, M, E, k, cf in shapes:
        x = torch.randn(T, M, generator=g).to(dtype).cuda()
        wg = (torch.randn(E, M, generator=g) * 0.05).to(dtype).cuda()
        bias = (torch.randn(E, generator=g) * 0.1).cuda()
        cap = ops.capacity(T, E, k, cf)
        want = ops.gate_route(x, wg, k, cap, bias)
        for _ in range(2):
            got = ops.gate_route_static(x, wg, k, cap, bias)
            _same(got, want)
        torch.cuda.synchronize()


def test_static_scratch_rejects_problems_beyond_its_size():
    from mole_b200 import _lib, ops
    T, M, E, k = 262144, 64, 256, 8          # (k + 1) * 4096 blocks * 256 experts * 4 B = 36 MiB
    x = torch.zeros(T, M, dtype=torch.bfloat16, device="cuda")
    wg = torch.zeros(E, M, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.MoleError) as e:
        ops.gate_route_static(x, wg, k, ops.capacity(T, E, k, 1.0))
    assert e.value.status == -4 and "built-in scratch" in str(e.value)


def test_static_entry_point_allocates_nothing():
    """With the outputs allocated beforehand, calls of the static entry point leave the device's
    memory use (driver view) and torch's allocator counters where they were."""
    from mole_b200 import ops
    T, M, E, k = 2048, 256, 32, 2
    x = torch.randn(T, M, device="cuda").bfloat16()
    wg = (torch.randn(E, M, device="cuda") * 0.05).bfloat16()
    cap = ops.capacity(T, E, k, 1.0)
    plan = ops.gate_route_static(x, wg, k, cap)          # first call on the device: set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    allocs0 = torch.cuda.memory_stats()["allocation.all.allocated"]
    for _ in range(3):
        ops.gate_route_static(x, wg, k, cap, plan=plan)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.cuda.memory_reserved() == reserved0
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocs0
