"""CPU oracle for the MOLE MoE-layer hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against.  It is imported
only by tests, by the smoke check and by the CPU-baseline / reference arms of
the benchmark; the product package never imports it and has no CPU fallback.

PARITY UNPINNED at the routing boundary: the reference (atc23-101/MOLE) holds no
tests, golden vectors or fixtures, does not build as shipped and calls its
routing / dispatch / combine out of an un-vendored, un-pinned third-party package
(``tutel.impls.fast_dispatch``; call sites MOLE/moe/layer.py:445-449,457-458,
declared in .gitmodules:4-6 with no recoverable version).  The routing below is
therefore this project's own GShard-style top-k-with-capacity specification,
constrained by what the reference's call sites require:

  * scores are a softmax over all experts of a bias-free linear gate
    (MOLE/utils/Ugate.py:5-14);
  * the dispatched tensor is expert-major ``[E_total, C, M]`` with global expert
    ``e`` at index ``e`` (MOLE/cpp/core.cpp:993-995, :158-161);
  * decode returns ``T*M`` elements (MOLE/moe/layer.py:460).

Everything inside the expert FFN follows the reference exactly:

  * forward  ``out = gelu(x @ W1^T + b1) @ W2 + b2`` on the capacity-padded
    tensor, ``W1`` and ``W2`` both stored ``[F, M]`` (MOLE/cpp/core.cpp:344-367,
    MOLE/moe/layer.py:89-96), exact (erf) GELU (``at::gelu``, core.cpp:351);
  * backward is autograd of the same expression, which equals the reference's
    ``bffn_bwd`` with exact GELU' (MOLE/cpp/core.cpp:381-414, the ``#else``
    branch of ``USE_MOLE_GELU``); ``gelu_bwd="tanh"`` switches to the
    tanh-approximation derivative the reference's own kernel uses
    (MOLE/cpp/gelu.cu:3-14);
  * experts are block-partitioned over ranks, expert ``e`` on rank ``e // (E/W)``,
    with an equal-split capacity-padded all-to-all either side of the FFN
    (MOLE/cpp/core.cpp:144-210, MOLE/cpp/communication.cpp:68-100).

Routing specification (integer outputs are compared bit-exact):

  1. ``logits = x.float() @ Wg.float().T (+ logit_bias)``; ``scores = softmax``.
  2. ``idx[t, j]`` = experts by descending score, ties to the lower expert id.
  3. ``g[t, j] = scores[t, idx[t, j]]``; with ``normalize_gate`` divided by
     ``max(sum_j g[t, j], eps)`` (sum over all k choices, before drops).
  4. ``C = max(1, ceil(k * capacity_factor * T / E))``.
  5. ``slot[t, j] = #{t' < t : idx[t', j] == e} + sum_{j' < j} hist_{j'}[e]`` with
     ``e = idx[t, j]``: every first choice is placed before any second choice,
     token order preserved inside a choice.
  6. A pair is kept iff ``slot < C``; dropped pairs have gate 0.
  7. ``counts[e] = min(sum_j hist_j[e], C)``; ``offsets = exclusive_scan(counts)``;
     ``perm[offsets[e] + slot] = t * k + j`` for kept pairs (token permutation).
  8. ``l_aux = E * sum_e mean_t(scores[t, e]) * mean_t(1[idx[t, 0] == e])``.
  9. ``disp[e, slot] = x[t]``; ``y[t] = sum_j kept * g[t, j] * out[e, slot]``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- #
# gate (MOLE/utils/Ugate.py:11-14)
# --------------------------------------------------------------------------- #
def gate_scores(x: torch.Tensor, wg: torch.Tensor,
                logit_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(x @ Wg^T)`` in fp32.  ``wg`` is ``[E, M]`` like ``Linear.weight``."""
    logits = x.float() @ wg.float().t()
    if logit_bias is not None:
        logits = logits + logit_bias.float()
    return torch.softmax(logits, dim=-1)


def capacity(T: int, E: int, k: int, capacity_factor: float) -> int:
    return max(1, int(math.ceil(k * capacity_factor * T / E)))


@dataclass
class Routing:
    idx: torch.Tensor      # [T, k] int32  chosen expert
    slot: torch.Tensor     # [T, k] int32  location inside the expert (may be >= C)
    kept: torch.Tensor     # [T, k] bool   slot < C
    gates: torch.Tensor    # [T, k] fp32   gate weight, 0 where dropped (differentiable)
    counts: torch.Tensor   # [E]   int32   min(hist, C)
    offsets: torch.Tensor  # [E+1] int32   exclusive scan of counts
    perm: torch.Tensor     # [T*k] int32   packed row -> pair id t*k+j, -1 beyond offsets[E]
    capacity: int
    l_aux: torch.Tensor    # scalar fp32 (differentiable)


def topk_lowest_index(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries per row, ties to the lower index."""
    work = scores.detach().clone()
    out = []
    rows = torch.arange(work.shape[0])
    for _ in range(k):
        j = torch.argmax(work, dim=-1)          # first maximal index
        out.append(j)
        work[rows, j] = -float("inf")
    return torch.stack(out, dim=1)


def route(scores: torch.Tensor, k: int, capacity_factor: float,
          normalize_gate: bool = False, eps: float = 1e-9,
          capacity_override: Optional[int] = None) -> Routing:
    """Top-k selection, capacity and slot assignment (spec items 2-8)."""
    T, E = scores.shape
    C = capacity_override if capacity_override is not None else capacity(T, E, k, capacity_factor)
    idx = topk_lowest_index(scores, k)                       # [T, k] int64
    g = torch.gather(scores, 1, idx)                         # differentiable
    if normalize_gate:
        g = g / g.sum(dim=1, keepdim=True).clamp_min(eps)
    slot = torch.empty(T, k, dtype=torch.int64)
    base = torch.zeros(E, dtype=torch.int64)
    for j in range(k):
        onehot = F.one_hot(idx[:, j], E)                     # [T, E] int64
        loc = torch.cumsum(onehot, dim=0) - 1 + base         # [T, E]
        slot[:, j] = torch.gather(loc, 1, idx[:, j:j + 1]).squeeze(1)
        base = base + onehot.sum(dim=0)
    kept = slot < C
    gates = g * kept.to(g.dtype)
    counts = torch.clamp(base, max=C)
    offsets = torch.zeros(E + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    perm = torch.full((T * k,), -1, dtype=torch.int64)
    pair = torch.arange(T * k).view(T, k)
    rows = offsets[idx] + slot
    perm[rows[kept]] = pair[kept]
    me = scores.mean(dim=0)
    ce = F.one_hot(idx[:, 0], E).to(scores.dtype).mean(dim=0)
    l_aux = E * torch.sum(me * ce)
    return Routing(idx.int(), slot.int(), kept, gates, counts.int(), offsets.int(),
                   perm.int(), C, l_aux)


# --------------------------------------------------------------------------- #
# dispatch / combine (reference call sites MOLE/moe/layer.py:448-449, 457-458)
# --------------------------------------------------------------------------- #
def encode(x: torch.Tensor, r: Routing, E: int) -> torch.Tensor:
    """``disp[e, slot] = x[t]`` into a zero ``[E, C, M]`` tensor."""
    T, M = x.shape
    k = r.idx.shape[1]
    flat = (r.idx.long() * r.capacity + r.slot.long())[r.kept]        # [P]
    tok = torch.arange(T).view(T, 1).expand(T, k)[r.kept]
    disp = torch.zeros(E * r.capacity, M, dtype=x.dtype)
    disp = disp.index_put((flat,), x[tok])
    return disp.view(E, r.capacity, M)


def decode(out: torch.Tensor, r: Routing) -> torch.Tensor:
    """``y[t] = sum_j g[t, j] * out[idx, slot]`` over kept pairs."""
    E, C, M = out.shape
    T, k = r.idx.shape
    flat = (r.idx.long() * C + r.slot.long()).clamp(max=E * C - 1)    # dropped -> any row
    rows = out.reshape(E * C, M)[flat.view(-1)].view(T, k, M)
    w = r.gates.to(out.dtype).unsqueeze(-1)                           # 0 where dropped
    return (rows * w).sum(dim=1)


# --------------------------------------------------------------------------- #
# expert FFN (MOLE/cpp/core.cpp:344-367 forward, :381-414 backward)
# --------------------------------------------------------------------------- #
class _GeluTanhBwd(torch.autograd.Function):
    """Exact GELU forward with the reference kernel's tanh-approximation derivative
    (MOLE/cpp/gelu.cu:3-14), selected by ``gelu_bwd="tanh"``."""

    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return F.gelu(x)

    @staticmethod
    def backward(ctx, gy):
        (x,) = ctx.saved_tensors
        return gy * gelu_tanh_derivative(x)


def gelu_tanh_derivative(x: torch.Tensor) -> torch.Tensor:
    c = 0.7978845608028654      # sqrt(2/pi)
    a = 0.044715
    inner = c * (x + a * x * x * x)
    t = torch.tanh(inner)
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * c * (1.0 + 3.0 * a * x * x)


def expert_ffn(disp: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor,
               w2: torch.Tensor, b2: torch.Tensor, act: str = "gelu",
               gelu_bwd: str = "exact") -> torch.Tensor:
    """``[B, R, M] -> [B, R, M]``; w1, w2 ``[B, F, M]``, b1 ``[B, F]``, b2 ``[B, M]``."""
    x1 = torch.baddbmm(b1.unsqueeze(1), disp, w1.transpose(1, 2))
    if act == "gelu":
        x2 = _GeluTanhBwd.apply(x1) if gelu_bwd == "tanh" else F.gelu(x1)
    elif act == "relu":
        x2 = torch.relu(x1)
    else:
        raise ValueError(f"unsupported activation {act!r}")
    return torch.baddbmm(b2.unsqueeze(1), x2, w2)


# --------------------------------------------------------------------------- #
# whole layer (MOLE/moe/layer.py:429-476)
# --------------------------------------------------------------------------- #
@dataclass
class LayerOut:
    y: torch.Tensor
    routing: Routing
    scores: torch.Tensor


def moe_layer(x: torch.Tensor, wg: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor,
              w2: torch.Tensor, b2: torch.Tensor, k: int, capacity_factor: float,
              logit_bias: Optional[torch.Tensor] = None, normalize_gate: bool = False,
              act: str = "gelu", gelu_bwd: str = "exact",
              scores_override: Optional[torch.Tensor] = None) -> LayerOut:
    """Single-process layer.  ``x`` is ``[..., M]``; returns ``y`` of the same shape and dtype.

    ``scores_override`` replaces the gate's scores *values used for routing decisions and
    gate weights* (tests use it to re-run the oracle on GPU-produced scores when a top-k
    choice sits on a rounding-level tie)."""
    shape, dtype = x.shape, x.dtype
    E, _, M = w1.shape
    xt = x.reshape(-1, M)
    scores = gate_scores(xt, wg, logit_bias) if scores_override is None else scores_override
    r = route(scores, k, capacity_factor, normalize_gate)
    disp = encode(xt, r, E)
    out = expert_ffn(disp, w1, b1, w2, b2, act, gelu_bwd)
    y = decode(out, r).reshape(shape).to(dtype)
    return LayerOut(y, r, scores)


def moe_layer_ep(x: torch.Tensor, wg: torch.Tensor, w1_local: torch.Tensor,
                 b1_local: torch.Tensor, w2_local: torch.Tensor, b2_local: torch.Tensor,
                 k: int, capacity_factor: float, group=None,
                 logit_bias: Optional[torch.Tensor] = None,
                 normalize_gate: bool = False) -> LayerOut:
    """Expert-parallel layer over a ``torch.distributed`` group (gloo on CPU).

    Rank ``r`` holds experts ``[r*L, (r+1)*L)``.  The exchange is the reference's
    equal-split, capacity-padded all-to-all (MOLE/cpp/core.cpp:144-210) including its
    ``[W, L, C, M] -> [L, W*C, M]`` re-layouts (core.cpp:233, :240)."""
    import torch.distributed as dist
    from torch.distributed.nn.functional import all_to_all_single

    W = dist.get_world_size(group)
    L, _, M = w1_local.shape
    E = L * W
    shape, dtype = x.shape, x.dtype
    xt = x.reshape(-1, M)
    scores = gate_scores(xt, wg, logit_bias)
    r = route(scores, k, capacity_factor, normalize_gate)
    C = r.capacity
    disp = encode(xt, r, E)                                   # [E, C, M] = [W, L, C, M]
    recv = all_to_all_single(torch.empty_like(disp), disp.contiguous(), group=group)
    local = recv.view(W, L, C, M).permute(1, 0, 2, 3).reshape(L, W * C, M)
    out = expert_ffn(local, w1_local, b1_local, w2_local, b2_local)
    back = out.view(L, W, C, M).permute(1, 0, 2, 3).contiguous().view(E, C, M)
    ret = all_to_all_single(torch.empty_like(back), back, group=group)
    y = decode(ret.view(E, C, M), r).reshape(shape).to(dtype)
    return LayerOut(y, r, scores)


# --------------------------------------------------------------------------- #
# seeded synthetic workloads (shapes and distributions of the benchmark configs)
# --------------------------------------------------------------------------- #
CONFIGS = {
    # name: T (tokens per rank), M, E, k, F, capacity factor, seed
    "c1": dict(T=4096, M=512, E=8, k=2, F=2048, cf=1.25, seed=0),
    "c2": dict(T=16384, M=1024, E=64, k=2, F=4096, cf=1.25, seed=1),
    "c3": dict(T=8192, M=2048, E=64, k=2, F=8192, cf=1.25, seed=0),
    "c4": dict(T=16384, M=1024, E=64, k=2, F=4096, cf=1.25, seed=2, zipf=1.2),
    "c5": dict(T=32768, M=2048, E=128, k=1, F=8192, cf=1.25, seed=3),
}


def make_inputs(T: int, M: int, E: int, F: int, seed: int, zipf: float = 0.0,
                experts: Optional[range] = None, token_seed: Optional[int] = None):
    """Seeded synthetic layer: weights ~ N(0, 0.02), zero biases, x and upstream grad ~ N(0, 1).

    Expert weights are seeded by global expert id so that any sharding reproduces the same
    model; ``experts`` selects the ids to materialise.  ``zipf > 0`` adds the fixed logit
    bias ``-zipf * ln(rank_e)`` over a seeded permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    wg = torch.randn(E, M, generator=g) * 0.02
    ids = list(experts) if experts is not None else list(range(E))
    w1 = torch.empty(len(ids), F, M)
    w2 = torch.empty(len(ids), F, M)
    for n, e in enumerate(ids):
        ge = torch.Generator().manual_seed(1_000_003 * (seed + 1) + e)
        w1[n] = torch.randn(F, M, generator=ge) * 0.02
        w2[n] = torch.randn(F, M, generator=ge) * 0.02
    b1 = torch.zeros(len(ids), F)
    b2 = torch.zeros(len(ids), M)
    gt = torch.Generator().manual_seed(seed if token_seed is None else 7_000_001 + token_seed)
    if token_seed is None:
        gt = g
    x = torch.randn(T, M, generator=gt)
    gy = torch.randn(T, M, generator=gt)
    bias = None
    if zipf > 0:
        ranks = torch.randperm(E, generator=torch.Generator().manual_seed(seed + 99)) + 1
        bias = -zipf * torch.log(ranks.float())
    return dict(x=x, gy=gy, wg=wg, w1=w1, b1=b1, w2=w2, b2=b2, logit_bias=bias)


# --------------------------------------------------------------------------- #
# explicit forward + backward with the layer's storage dtype
# --------------------------------------------------------------------------- #
# When the reference's op sequence runs on tensors of dtype D, every at::Tensor it
# materialises (x1, gelu(x1), the FFN output, the activation gradient, every weight gradient;
# MOLE/cpp/core.cpp:350-353, 388-412) holds values rounded to D, while each matmul accumulates in
# fp32.  The functions below restate that: fp32 arithmetic with a rounding to D wherever a
# tensor is stored.  For D = float32 they coincide with autograd of ``expert_ffn``.

def _act_and_grad(x1: torch.Tensor, act: str, gelu_bwd: str):
    if act == "relu":
        return torch.relu(x1), (x1 > 0).to(x1.dtype)
    h = F.gelu(x1)
    if gelu_bwd == "tanh":
        return h, gelu_tanh_derivative(x1)
    cdf = 0.5 * (1.0 + torch.erf(x1 * 0.7071067811865476))
    pdf = torch.exp(-0.5 * x1 * x1) * 0.3989422804014327
    return h, cdf + x1 * pdf


def ffn_explicit(x, w1, b1, w2, b2, dout, dtype, act="gelu", gelu_bwd="exact"):
    """One expert on its rows ``x [n, M]`` with upstream gradient ``dout [n, M]`` (fp32 tensors
    holding dtype-representable values).  Returns out, dx and the four parameter gradients,
    following MOLE/cpp/core.cpp:350-353 (forward) and :388-412 (backward)."""
    rd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).float())
    x1 = rd(x @ w1.t() + b1)
    h_full, dact = _act_and_grad(x1, act, gelu_bwd)
    h = rd(h_full)
    out = rd(h @ w2 + b2)
    gw2 = rd(h.t() @ dout)
    dx1 = rd((dout @ w2.t()) * dact)
    gb2 = rd(dout.sum(0))
    gw1 = rd(dx1.t() @ x)
    gb1 = rd(dx1.sum(0))
    dx = rd(dx1 @ w1)
    return dict(out=out, dx=dx, gw1=gw1, gb1=gb1, gw2=gw2, gb2=gb2)


def layer_explicit(x, gy, wg, w1, b1, w2, b2, k, capacity_factor, dtype,
                   scores=None, logit_bias=None, normalize_gate=False, l_aux_weight=0.0,
                   act="gelu", gelu_bwd="exact"):
    """Whole layer forward + backward with storage dtype ``dtype``.  All inputs are fp32 tensors
    holding dtype-representable values.  ``scores`` (optional) supplies the scores the routing
    *decisions* are taken from (a GPU run's own scores, so that rounding-level ties do not
    flip choices); gate values and their gradients always come from this function's scores."""
    rd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).float())
    T, M = x.shape
    E = w1.shape[0]
    xg = x.clone().requires_grad_(True)
    wgg = wg.clone().requires_grad_(True)
    own = gate_scores(xg, wgg, logit_bias)
    r = route(own.detach() if scores is None else scores, k, capacity_factor, normalize_gate)
    # differentiable gates / l_aux from this function's own scores on the decided routing
    g = torch.gather(own, 1, r.idx.long())
    if normalize_gate:
        g = g / g.sum(dim=1, keepdim=True).clamp_min(1e-9)
    g = g * r.kept.to(g.dtype)
    me = own.mean(dim=0)
    ce = F.one_hot(r.idx[:, 0].long(), E).to(own.dtype).mean(dim=0)
    l_aux = E * torch.sum(me * ce)
    C = r.capacity
    gates = g.detach()
    disp = encode(x, r, E)                                        # exact copies
    pair_t = torch.arange(T).view(T, 1).expand(T, k)
    out = torch.zeros(E, C, M)
    ddisp = torch.zeros(E, C, M)
    drows = torch.zeros(E, C, M)
    grads = dict(gw1=torch.zeros_like(w1), gb1=torch.zeros_like(b1),
                 gw2=torch.zeros_like(w2), gb2=torch.zeros_like(b2))
    # combine backward needs the expert outputs, which need the forward of every expert first
    for e in range(E):
        n = int(r.counts[e])
        res = ffn_explicit(disp[e, :n], w1[e], b1[e], w2[e], b2[e], torch.zeros(n, M), dtype, act,
                           gelu_bwd)
        out[e, :n] = res["out"]
    rr = Routing(r.idx, r.slot, r.kept, gates, r.counts, r.offsets, r.perm, C, l_aux.detach())
    y = rd(decode(out, rr))
    # backward of combine: drows = g * dy, dgates = <dy, out row>
    flat = (r.idx.long() * C + r.slot.long()).clamp(max=E * C - 1)
    rows_of_pair = out.reshape(E * C, M)[flat.view(-1)].view(T, k, M)
    dgates = (rows_of_pair * gy.unsqueeze(1)).sum(-1) * r.kept
    kept = r.kept
    drows.view(E * C, M)[flat[kept]] = rd(gates[kept].unsqueeze(-1) * gy[pair_t[kept]])
    for e in range(E):
        n = int(r.counts[e])
        res = ffn_explicit(disp[e, :n], w1[e], b1[e], w2[e], b2[e], drows[e, :n], dtype, act,
                           gelu_bwd)
        ddisp[e, :n] = res["dx"]
        for name in grads:
            grads[name][e] = res[name]
    dx_disp = torch.zeros(T, M)
    dx_disp.index_add_(0, pair_t[kept], ddisp.view(E * C, M)[flat[kept]])
    dx_disp = rd(dx_disp)
    ((g * dgates).sum() + l_aux_weight * l_aux).backward()
    dx = rd(dx_disp + rd(xg.grad))
    return dict(y=y, dx=dx, dwg=rd(wgg.grad), routing=rr, scores=own.detach(), dgates=dgates,
                l_aux=l_aux.detach(), **grads)
