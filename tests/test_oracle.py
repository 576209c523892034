"""CPU tests of the oracle: hand-computed cases, invariants, gradients, golden fixtures."""
from pathlib import Path

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from oracle import moe_ref as O

GOLDEN = Path(__file__).resolve().parent / "golden"


# ---- hand-computable micro cases -----------------------------------------------------------
def test_route_hand_case_k1_capacity1():
    # 4 tokens, 2 experts, top-1, capacity 1: tokens 0,2 prefer expert 0; 1,3 prefer expert 1
    scores = torch.tensor([[0.9, 0.1], [0.2, 0.8], [0.6, 0.4], [0.3, 0.7]])
    r = O.route(scores, k=1, capacity_factor=0.5)           # C = ceil(1*0.5*4/2) = 1
    assert r.capacity == 1
    assert r.idx.flatten().tolist() == [0, 1, 0, 1]
    assert r.slot.flatten().tolist() == [0, 0, 1, 1]
    assert r.kept.flatten().tolist() == [True, True, False, False]
    assert r.gates.flatten().tolist() == pytest.approx([0.9, 0.8, 0.0, 0.0])
    assert r.counts.tolist() == [1, 1] and r.offsets.tolist() == [0, 1, 2]
    assert r.perm.tolist() == [0, 1, -1, -1]
    # l_aux = E * sum_e mean(scores[:, e]) * mean(first choice == e) = 2 * (0.5*0.5 + 0.5*0.5)
    assert float(r.l_aux) == pytest.approx(1.0)


def test_route_hand_case_second_choices_after_first():
    # 3 tokens, 2 experts, top-2: every first choice takes a slot before any second choice
    scores = torch.tensor([[0.7, 0.3], [0.6, 0.4], [0.2, 0.8]])
    r = O.route(scores, k=2, capacity_factor=1.0)           # C = ceil(2*3/2) = 3
    assert r.idx.tolist() == [[0, 1], [0, 1], [1, 0]]
    # expert 0: first choices t0 -> 0, t1 -> 1; second choice t2 -> 2
    # expert 1: first choice t2 -> 0; second choices t0 -> 1, t1 -> 2
    assert r.slot.tolist() == [[0, 1], [1, 2], [0, 2]]
    assert r.counts.tolist() == [3, 3]
    assert r.perm.tolist() == [0, 2, 5, 4, 1, 3]


def test_topk_ties_go_to_lower_expert():
    scores = torch.tensor([[0.25, 0.25, 0.25, 0.25], [0.1, 0.4, 0.4, 0.1]])
    assert O.topk_lowest_index(scores, 2).tolist() == [[0, 1], [1, 2]]


def test_encode_decode_hand_case():
    x = torch.arange(8.0).view(4, 2)
    scores = torch.tensor([[0.9, 0.1], [0.2, 0.8], [0.6, 0.4], [0.3, 0.7]])
    r = O.route(scores, k=1, capacity_factor=0.5)
    disp = O.encode(x, r, 2)
    assert disp.tolist() == [[[0.0, 1.0]], [[2.0, 3.0]]]
    y = O.decode(disp, r)
    assert torch.allclose(y, torch.tensor([[0.0, 0.9], [1.6, 2.4], [0.0, 0.0], [0.0, 0.0]]))


# ---- invariants ---------------------------------------------------------------------------------
@settings(max_examples=40, deadline=None)
@given(T=st.integers(1, 70), E=st.integers(1, 9), k=st.integers(1, 3),
       cf=st.sampled_from([0.25, 0.5, 1.0, 1.25, 4.0]), seed=st.integers(0, 10_000),
       skew=st.booleans())
def test_routing_invariants(T, E, k, cf, seed, skew):
    k = min(k, E)
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g) * (3.0 if skew else 0.3)
    if skew:
        logits[:, 0] += 4.0                 # nearly everything wants expert 0
    scores = torch.softmax(logits, -1)
    r = O.route(scores, k, cf)
    C = r.capacity
    assert C == max(1, int(np.ceil(k * cf * T / E)))
    kept = r.kept
    # each token's experts are distinct
    for j in range(k):
        for j2 in range(j):
            assert (r.idx[:, j] != r.idx[:, j2]).all()
    # kept pairs occupy unique (expert, slot) cells below capacity
    cells = (r.idx.long() * (T * k + C) + r.slot.long())[kept]
    assert cells.unique().numel() == cells.numel()
    assert (r.slot[kept] < C).all() and (r.slot >= 0).all()
    hist = torch.bincount(r.idx.flatten().long(), minlength=E)
    assert r.counts.tolist() == torch.clamp(hist, max=C).tolist()
    assert r.offsets[-1].item() == int(kept.sum())
    # perm is a bijection from packed rows onto kept pairs, expert-major, slot order inside
    P = int(kept.sum())
    pairs = r.perm[:P].long()
    assert (r.perm[P:] == -1).all()
    assert sorted(pairs.tolist()) == sorted(torch.arange(T * k).view(T, k)[kept].tolist())
    flat_e = r.idx.flatten().long()[pairs]
    flat_s = r.slot.flatten().long()[pairs]
    assert (r.offsets.long()[flat_e] + flat_s == torch.arange(P)).all()
    # dropped pairs have gate 0; kept pairs carry the score
    assert (r.gates[~kept] == 0).all()
    assert torch.equal(r.gates[kept], torch.gather(scores, 1, r.idx.long())[kept])
    # slots are ordered by (choice, token)
    for e in range(E):
        order = [(j, t) for j in range(k) for t in range(T) if r.idx[t, j] == e]
        got = sorted(((int(r.slot[t, j]), (j, t)) for j, t in order))
        assert [p for _, p in got] == order


def test_encode_decode_identity_with_unit_gates():
    T, M, E, k = 50, 8, 4, 2
    x = torch.randn(T, M)
    r = O.route(torch.softmax(torch.randn(T, E), -1), k, 4.0)      # nothing dropped
    assert r.kept.all()
    r.gates = torch.ones_like(r.gates)
    y = O.decode(O.encode(x, r, E), r)
    assert torch.allclose(y, k * x)


def test_normalized_gates_sum_to_one_before_drops():
    scores = torch.softmax(torch.randn(40, 6), -1)
    r = O.route(scores, 2, 8.0, normalize_gate=True)
    assert torch.allclose(r.gates.sum(1), torch.ones(40), atol=1e-6)


# ---- gradients -----------------------------------------------------------------------------------
def test_layer_gradcheck_fp64():
    torch.manual_seed(3)
    T, M, E, F, k = 10, 4, 3, 6, 2
    x = torch.randn(T, M, dtype=torch.float64, requires_grad=True)
    w1 = (torch.randn(E, F, M, dtype=torch.float64) * 0.5).requires_grad_()
    b1 = (torch.randn(E, F, dtype=torch.float64) * 0.1).requires_grad_()
    w2 = (torch.randn(E, F, M, dtype=torch.float64) * 0.5).requires_grad_()
    b2 = (torch.randn(E, M, dtype=torch.float64) * 0.1).requires_grad_()
    scores = torch.softmax(torch.randn(T, E, dtype=torch.float64), -1).requires_grad_()

    def f(x, scores, w1, b1, w2, b2):
        r = O.route(scores, k, 1.0)
        out = O.expert_ffn(O.encode(x, r, E), w1, b1, w2, b2)
        return O.decode(out, r), r.l_aux

    assert torch.autograd.gradcheck(f, (x, scores, w1, b1, w2, b2), eps=1e-6, atol=1e-5)


def test_ffn_backward_matches_reference_formulas():
    """Autograd of the oracle FFN equals the reference's explicit backward
    (MOLE/cpp/core.cpp:388-412: gW2 = gelu(x1)^T dO, dX1 = gelu'(x1) * dO W2^T, ...)."""
    torch.manual_seed(0)
    B, R, M, F = 2, 7, 6, 10
    x = torch.randn(B, R, M, dtype=torch.float64, requires_grad=True)
    w1 = torch.randn(B, F, M, dtype=torch.float64, requires_grad=True)
    b1 = torch.randn(B, F, dtype=torch.float64, requires_grad=True)
    w2 = torch.randn(B, F, M, dtype=torch.float64, requires_grad=True)
    b2 = torch.randn(B, M, dtype=torch.float64, requires_grad=True)
    dO = torch.randn(B, R, M, dtype=torch.float64)
    O.expert_ffn(x, w1, b1, w2, b2).backward(dO)
    x1 = torch.baddbmm(b1.unsqueeze(1), x, w1.transpose(1, 2)).detach()
    h = torch.nn.functional.gelu(x1)
    cdf = 0.5 * (1 + torch.erf(x1 / 2 ** 0.5))
    pdf = torch.exp(-0.5 * x1 * x1) / (2 * torch.pi) ** 0.5
    dx1 = (dO @ w2.detach().transpose(1, 2)) * (cdf + x1 * pdf)
    assert torch.allclose(w2.grad, h.transpose(1, 2) @ dO)
    assert torch.allclose(b2.grad, dO.sum(1))
    assert torch.allclose(w1.grad, dx1.transpose(1, 2) @ x.detach())
    assert torch.allclose(b1.grad, dx1.sum(1))
    assert torch.allclose(x.grad, dx1 @ w1.detach())


def test_tanh_gelu_derivative_close_to_exact():
    x = torch.linspace(-6, 6, 1001, dtype=torch.float64)
    cdf = 0.5 * (1 + torch.erf(x / 2 ** 0.5))
    exact = cdf + x * torch.exp(-0.5 * x * x) / (2 * torch.pi) ** 0.5
    assert (O.gelu_tanh_derivative(x) - exact).abs().max() < 2e-3


# ---- golden fixtures -----------------------------------------------------------------------------
def test_golden_small_case():
    g = np.load(GOLDEN / "small.npz")
    t = {n: torch.from_numpy(g[n]) for n in ("x", "gy", "wg", "w1", "b1", "w2", "b2")}
    x = t["x"].clone().requires_grad_(True)
    ws = [t[n].clone().requires_grad_(True) for n in ("wg", "w1", "b1", "w2", "b2")]
    out = O.moe_layer(x, *ws, k=int(g["k"]), capacity_factor=float(g["cf"]))
    (out.y * t["gy"]).sum().backward()
    r = out.routing
    assert r.capacity == int(g["capacity"])
    for name in ("idx", "slot", "counts", "offsets", "perm"):
        assert np.array_equal(getattr(r, name).numpy(), g[name]), name
    assert not r.kept.all(), "the fixture is meant to drop pairs"
    np.testing.assert_allclose(out.y.detach().numpy(), g["y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(x.grad.numpy(), g["dx"], rtol=1e-5, atol=1e-6)
    for n, w in zip(("dwg", "dw1", "db1", "dw2", "db2"), ws):
        np.testing.assert_allclose(w.grad.numpy(), g[n], rtol=1e-5, atol=1e-6, err_msg=n)


def test_golden_c1_routing():
    g = np.load(GOLDEN / "c1_routing.npz")
    cfg = O.CONFIGS["c1"]
    inp = O.make_inputs(cfg["T"], cfg["M"], cfg["E"], cfg["F"], cfg["seed"])
    scores = O.gate_scores(inp["x"], inp["wg"])
    r = O.route(scores, cfg["k"], cfg["cf"])
    assert r.capacity == int(g["capacity"]) == 1280
    assert np.array_equal(r.idx.numpy(), g["idx"].astype(np.int32))
    assert np.array_equal(r.slot.numpy(), g["slot"].astype(np.int32))
    assert np.array_equal(r.counts.numpy(), g["counts"])
    assert np.array_equal(r.offsets.numpy(), g["offsets"])
    assert float(r.l_aux) == pytest.approx(float(g["l_aux"]), rel=1e-5)
