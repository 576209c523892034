"""(b) Dispatch / combine kernels against the oracle's encode / decode and their autograd."""
import pytest
import torch

from oracle import moe_ref as O
from util import assert_close

pytestmark = pytest.mark.gpu


def setup(T, M, E, k, cf, dtype, seed=0):
    from mole_b200 import ops
    g = torch.Generator().manual_seed(seed)
    scores = torch.softmax(torch.randn(T, E, generator=g), -1)
    x = torch.randn(T, M, generator=g).to(dtype)
    r = O.route(scores, k, cf)
    plan = ops.route_from_scores(scores.cuda(), k, ops.capacity(T, E, k, cf))
    return x, scores, r, plan, g


def strided(t, r, Cs):
    """Oracle [E, C, M] tensor placed into the capacity-strided layout [E, Cs, M]."""
    E, C, M = t.shape
    out = torch.zeros(E, Cs, M, dtype=t.dtype)
    out[:, :C] = t
    return out


CASES = [(1024, 256, 8, 2, 1.25), (600, 64, 16, 2, 0.5), (130, 512, 4, 1, 1.0), (2000, 128, 64, 3, 1.0)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,M,E,k,cf", CASES)
def test_dispatch_forward(dtype, T, M, E, k, cf):
    from mole_b200 import ops
    x, scores, r, plan, _ = setup(T, M, E, k, cf, dtype)
    rows = torch.full((E, plan.Cs, M), float("nan"), dtype=dtype, device="cuda")
    ops.dispatch(x.cuda(), plan, out=rows)
    rows = rows.cpu()
    ref = O.encode(x, r, E)
    for e in range(E):
        c = int(r.counts[e])
        pad = (c + 127) // 128 * 128
        assert torch.equal(rows[e, :c], ref[e, :c]), f"expert {e}: valid rows differ"
        assert (rows[e, c:pad] == 0).all(), f"expert {e}: pad rows not zero"
        assert torch.isnan(rows[e, pad:].float()).all(), f"expert {e}: wrote beyond the padded tile"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,M,E,k,cf", CASES)
def test_combine_forward_backward(dtype, T, M, E, k, cf):
    from mole_b200 import ops
    x, scores, r, plan, g = setup(T, M, E, k, cf, dtype, seed=1)
    C, Cs = r.capacity, plan.Cs
    out = torch.randn(E, C, M, generator=g).to(dtype)
    dy = torch.randn(T, M, generator=g).to(dtype)
    out_s = strided(out, r, Cs)
    # garbage beyond the padded tiles must never be read
    for e in range(E):
        pad = (int(r.counts[e]) + 127) // 128 * 128
        out_s[e, pad:] = float("nan")
    y = ops.combine(out_s.cuda(), plan, plan.gates)
    of = out.float().requires_grad_(True)
    gates = r.gates.detach().clone().requires_grad_(True)
    r2 = O.Routing(r.idx, r.slot, r.kept, gates, r.counts, r.offsets, r.perm, r.capacity, r.l_aux)
    yref = O.decode(of, r2)
    assert_close(y, yref, dtype, "combine forward")
    yref.backward(dy.float())
    drows, dgates = ops.combine_bwd(dy.cuda(), out_s.cuda(), plan, plan.gates)
    drows = drows.cpu()
    for e in range(E):
        c = int(r.counts[e])
        pad = (c + 127) // 128 * 128
        assert_close(drows[e, :c], of.grad[e, :c], dtype, f"combine backward rows, expert {e}")
        assert (drows[e, c:pad] == 0).all()
    kept = r.kept
    assert_close(dgates.cpu()[kept], gates.grad[kept], dtype, "combine backward gates",
                 scale=4.0 if dtype == torch.float32 else 1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,M,E,k,cf", CASES)
def test_dispatch_backward(dtype, T, M, E, k, cf):
    from mole_b200 import ops
    x, scores, r, plan, g = setup(T, M, E, k, cf, dtype, seed=2)
    C, Cs = r.capacity, plan.Cs
    ddisp = torch.randn(E, C, M, generator=g).to(dtype)
    xr = x.float().requires_grad_(True)
    O.encode(xr, r, E).backward(ddisp.float())
    dd = strided(ddisp, r, Cs)
    dd[:, C:] = float("nan")
    dx = ops.dispatch_bwd(dd.cuda(), plan, M, dtype, torch.device("cuda"))
    assert_close(dx, xr.grad, dtype, "dispatch backward")


def test_encode_decode_round_trip_full_size():
    """Size-independent property at the benchmark shape (16384 x 1024, 64 experts, top-2): with
    unit gates and no drops, combine(dispatch(x)) == k * x exactly in bf16 for k = 2."""
    from mole_b200 import ops
    T, M, E, k = 16384, 1024, 64, 2
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, M, generator=g).bfloat16().cuda()
    scores = torch.softmax(torch.randn(T, E, generator=g), -1).cuda()
    plan = ops.route_from_scores(scores, k, T)          # capacity = T: nothing dropped
    assert int(plan.counts.sum()) == T * k
    rows = ops.dispatch(x, plan)
    y = ops.combine(rows, plan, torch.ones_like(plan.gates))
    assert torch.equal(y, x * 2)
