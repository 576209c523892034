"""(a) Gate and routing-index build on the GPU against the oracle.  Integer outputs bit-exact."""
import numpy as np
import pytest
import torch

from oracle import moe_ref as O

pytestmark = pytest.mark.gpu


def make_scores(T, E, seed, kind):
    g = torch.Generator().manual_seed(seed)
    if kind == "uniform":
        return torch.softmax(torch.randn(T, E, generator=g) * 0.3, -1)
    if kind == "skew":                       # almost everything wants expert 0
        logits = torch.randn(T, E, generator=g)
        logits[:, 0] += 6.0
        return torch.softmax(logits, -1)
    if kind == "ties":                       # few distinct values: many exact ties
        return torch.randint(0, 3, (T, E), generator=g).float() / 4 + 0.125
    raise ValueError(kind)


def compare_plan(plan, r, gates_exact=True):
    assert plan.C == r.capacity
    for name in ("idx", "slot", "counts", "offsets", "perm"):
        got = getattr(plan, name).cpu()
        assert torch.equal(got, getattr(r, name)), f"{name} differs"
    if gates_exact:
        assert torch.equal(plan.gates.cpu(), r.gates.detach())
    else:
        torch.testing.assert_close(plan.gates.cpu(), r.gates.detach(), rtol=1e-6, atol=1e-9)
    torch.testing.assert_close(plan.l_aux.cpu().view(()), r.l_aux.detach(), rtol=1e-5, atol=1e-7)


CASES = [
    # T, E, k, capacity factor, kind
    (4096, 8, 2, 1.25, "uniform"),
    (1000, 64, 2, 1.25, "uniform"),        # T not a multiple of the 64-token block
    (777, 64, 2, 0.5, "skew"),             # heavy drops
    (5, 16, 2, 1.0, "uniform"),            # fewer tokens than experts
    (300, 7, 1, 1.0, "uniform"),           # top-1, odd expert count
    (256, 4, 4, 1.0, "ties"),              # k == E with exact ties
    (513, 256, 8, 2.0, "uniform"),         # the limits: 256 experts, top-8
    (2048, 32, 2, 0.01, "skew"),           # capacity 2
    (64, 1, 1, 1.0, "uniform"),            # one expert
]


@pytest.mark.parametrize("T,E,k,cf,kind", CASES)
def test_route_from_scores_bit_exact(T, E, k, cf, kind):
    from mole_b200 import ops
    scores = make_scores(T, E, 100 + T, kind)
    r = O.route(scores, k, cf)
    plan = ops.route_from_scores(scores.cuda(), k, ops.capacity(T, E, k, cf))
    compare_plan(plan, r)
    assert torch.equal(plan.first_hist.cpu().long(),
                       torch.bincount(r.idx[:, 0].long(), minlength=E))


def test_route_all_tokens_one_expert_capacity_one():
    from mole_b200 import ops
    T, E = 130, 8
    scores = torch.full((T, E), 0.01)
    scores[:, 3] = 0.93
    r = O.route(scores, 1, 0.0001)
    assert r.capacity == 1
    plan = ops.route_from_scores(scores.cuda(), 1, 1)
    compare_plan(plan, r)
    assert plan.counts.cpu().tolist() == [0, 0, 0, 1, 0, 0, 0, 0]


def test_route_normalized_gates():
    from mole_b200 import ops
    T, E, k = 900, 16, 2
    scores = make_scores(T, E, 3, "uniform")
    r = O.route(scores, k, 1.0, normalize_gate=True)
    plan = ops.route_from_scores(scores.cuda(), k, ops.capacity(T, E, k, 1.0), normalize=True)
    compare_plan(plan, r, gates_exact=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,M,E,k", [(4096, 512, 8, 2), (1500, 256, 64, 2), (333, 136, 20, 3)])
def test_gate_route_fused(dtype, T, M, E, k):
    """softmax(x @ Wg^T) and the routing built from it.  The integers must equal the oracle's on
    the GPU's own scores; against the oracle's scores only rounding-level ties may differ."""
    from mole_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, M, generator=g).to(dtype)
    wg = (torch.randn(E, M, generator=g) * 0.05).to(dtype)
    bias = torch.randn(E, generator=g) * 0.1
    cap = ops.capacity(T, E, k, 1.25)
    plan = ops.gate_route(x.cuda(), wg.cuda(), k, cap, bias.cuda())
    ref_scores = O.gate_scores(x.float(), wg.float(), bias)
    torch.testing.assert_close(plan.scores.cpu(), ref_scores, rtol=2e-5, atol=1e-7)
    compare_plan(plan, O.route(plan.scores.cpu(), k, 1.25))
    r = O.route(ref_scores, k, 1.25)
    flips = (plan.idx.cpu() != r.idx).any(dim=1)
    if flips.any():          # a flipped choice must sit on a rounding-level tie
        s = torch.sort(ref_scores[flips], dim=1, descending=True).values
        gap = (s[:, :k] - s[:, 1:k + 1]).min(dim=1).values / s[:, k - 1]
        assert gap.max() < 1e-5, f"top-k differs from the oracle with score gap {gap.max():.3g}"
    assert flips.float().mean() < 1e-3


def test_gate_backward_matches_autograd():
    from mole_b200 import ops
    T, M, E, k = 700, 128, 16, 2
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, M, generator=g)
    wg = torch.randn(E, M, generator=g) * 0.05
    cap = ops.capacity(T, E, k, 0.75)
    dgates = torch.randn(T, k, generator=g)
    dl = torch.tensor(0.37)
    for normalize in (False, True):
        xr, wr = x.clone().requires_grad_(True), wg.clone().requires_grad_(True)
        scores = O.gate_scores(xr, wr)
        r = O.route(scores, k, 0.75, normalize_gate=normalize)
        ((r.gates * dgates).sum() + dl * r.l_aux).backward()
        plan = ops.gate_route(x.cuda(), wg.cuda(), k, cap, None, normalize)
        assert torch.equal(plan.idx.cpu(), r.idx) and torch.equal(plan.slot.cpu(), r.slot)
        dlogits = ops.gate_bwd(plan, dgates.cuda(), dl.view(1).cuda())
        dwg = ops.gate_wgrad(dlogits, x.cuda())
        dx = ops.dispatch_bwd(None, plan, M, torch.float32, torch.device("cuda"), dlogits, wg.cuda())
        torch.testing.assert_close(dwg.cpu(), wr.grad, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dx.cpu(), xr.grad, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_weight_gradient_is_bit_reproducible(dtype):
    """dWg = dlogits^T x is summed over tokens in two stages with a fixed order (no atomics):
    repeated calls return identical bits, and the value matches a float64 product."""
    from mole_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, M, E = 4096 + 77, 256, 24
    x = torch.randn(T, M, generator=g).to(dtype).cuda()
    dl = (torch.randn(T, E, generator=g) * 1e-2).cuda()
    first = ops.gate_wgrad(dl, x)
    for _ in range(3):
        assert torch.equal(ops.gate_wgrad(dl, x), first)
    ref = (dl.double().t() @ x.double()).float()
    torch.testing.assert_close(first, ref, rtol=2e-4, atol=2e-4)
