"""The whole layer (``MOLEModule`` forward + backward through the C ABI) against the oracle."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe_ref as O
from util import assert_close

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
DIST1 = {"local_rank": 0, "world_size": 1, "rank": 0}


def build_module(inp, E, M, F, k, dtype, d_experts=0, pool_size=-1, ebatch=64, **kw):
    from mole_b200 import MOLEModule
    m = MOLEModule(d_experts, E - d_experts, M, F, pool_size, k, ebatch, DIST1, "gelu", 1, False,
                   pool_size != -1, dtype=dtype, **kw)
    state = {"gate": [inp["wg"], None],
             "experts": [[inp["w1"][e], inp["b1"][e], inp["w2"][e], inp["b2"][e]] for e in range(E)]}
    m.set_layer_state(state, grad=False)
    return m


def run_module(m, inp, cf, dtype, l_aux_weight=0.0):
    x = inp["x"].to(dtype).cuda().requires_grad_(True)
    y = m(x, capacity_factor=cf)
    loss = (y.float() * inp["gy"].cuda()).sum() + l_aux_weight * m.l_aux
    loss.backward()
    torch.cuda.synchronize()
    return x, y


def run_oracle(inp, k, cf, dtype, scores=None, l_aux_weight=0.0, logit_bias=None):
    """The oracle's explicit forward + backward on the values the GPU sees, with every stored
    tensor rounded to ``dtype``; routing decisions from the GPU's scores when given."""
    rd = lambda t: t.to(dtype).float()
    return O.layer_explicit(rd(inp["x"]), rd(inp["gy"]), rd(inp["wg"]), rd(inp["w1"]), rd(inp["b1"]),
                            rd(inp["w2"]), rd(inp["b2"]), k, cf, dtype, scores=scores,
                            logit_bias=logit_bias, l_aux_weight=l_aux_weight)


def compare(m, x, y, ref, dtype):
    plan = m.last_plan
    r = ref["routing"]
    for name in ("idx", "slot", "counts", "offsets", "perm"):
        assert torch.equal(getattr(plan, name).cpu(), getattr(r, name)), name
    assert_close(y, ref["y"], dtype, "y")
    assert_close(x.grad, ref["dx"], dtype, "dx")
    assert_close(m.gate[0].linear.weight.grad, ref["dwg"], dtype, "dWg", scale=4.0)
    got = [m.FC1_W_GPU.grad_tensors, m.FC1_B_GPU.grad_tensors, m.FC2_W_GPU.grad_tensors,
           m.FC2_B_GPU.grad_tensors]
    for name, g in zip(("gw1", "gb1", "gw2", "gb2"), got):
        assert_close(g, ref[name], dtype, name, scale=4.0 if dtype == torch.float32 else 1.0)
    torch.testing.assert_close(m.l_aux.detach().cpu(), ref["l_aux"], rtol=1e-4, atol=1e-6)


def test_layer_fp32_config1_matches_oracle_and_golden():
    """Benchmark config 1: 4096 x 512, 8 experts, top-2, d_ffn 2048, cf 1.25, fp32, seed 0."""
    cfg = O.CONFIGS["c1"]
    inp = O.make_inputs(cfg["T"], cfg["M"], cfg["E"], cfg["F"], cfg["seed"])
    m = build_module(inp, cfg["E"], cfg["M"], cfg["F"], cfg["k"], torch.float32)
    x, y = run_module(m, inp, cfg["cf"], torch.float32, l_aux_weight=0.01)
    ref = run_oracle(inp, cfg["k"], cfg["cf"], torch.float32, l_aux_weight=0.01)
    compare(m, x, y, ref, torch.float32)
    g = np.load(GOLDEN / "c1_routing.npz")
    assert np.array_equal(m.last_plan.idx.cpu().numpy(), g["idx"].astype(np.int32))
    assert np.array_equal(m.last_plan.slot.cpu().numpy(), g["slot"].astype(np.int32))
    assert np.array_equal(m.last_plan.counts.cpu().numpy(), g["counts"])
    assert float(y.detach().double().sum()) == pytest.approx(float(g["y"]), abs=1e-4 * float(g["y_abs"]))


def test_layer_fp32_golden_small_with_drops():
    g = np.load(GOLDEN / "small.npz")
    inp = {n: torch.from_numpy(g[n]) for n in ("x", "gy", "wg", "w1", "b1", "w2", "b2")}
    E, M, F, k = int(g["E"]), int(g["M"]), int(g["F"]), int(g["k"])
    m = build_module(inp, E, M, F, k, torch.float32)
    x, y = run_module(m, inp, float(g["cf"]), torch.float32)
    plan = m.last_plan
    for name in ("idx", "slot", "counts", "offsets", "perm"):
        assert np.array_equal(getattr(plan, name).cpu().numpy(), g[name]), name
    assert_close(y, torch.from_numpy(g["y"]), torch.float32, "y")
    assert_close(x.grad, torch.from_numpy(g["dx"]), torch.float32, "dx", scale=4.0)
    assert_close(m.FC1_W_GPU.grad_tensors, torch.from_numpy(g["dw1"]), torch.float32, "gW1", scale=4.0)
    assert_close(m.FC2_B_GPU.grad_tensors, torch.from_numpy(g["db2"]), torch.float32, "gb2", scale=4.0)
    assert_close(m.gate[0].linear.weight.grad, torch.from_numpy(g["dwg"]), torch.float32, "dWg", scale=4.0)


@pytest.mark.parametrize("backend", [1, 2, 3], ids=["cuda_cores", "tcgen05_one_cta", "tcgen05_cta_pair"])
@pytest.mark.parametrize("cf", [1.25, 0.5])
def test_layer_bf16_matches_oracle(backend, cf):
    T, M, E, F, k = 2048, 256, 16, 512, 2
    inp = O.make_inputs(T, M, E, F, seed=21)
    inp["wg"] = inp["wg"] * 5
    inp["b1"] = torch.randn(E, F, generator=torch.Generator().manual_seed(1)) * 0.05
    inp["b2"] = torch.randn(E, M, generator=torch.Generator().manual_seed(2)) * 0.05
    m = build_module(inp, E, M, F, k, torch.bfloat16, ffn_backend=backend)
    x, y = run_module(m, inp, cf, torch.bfloat16)
    ref = run_oracle(inp, k, cf, torch.bfloat16, scores=m.last_plan.scores.cpu())
    compare(m, x, y, ref, torch.bfloat16)


def test_layer_bf16_skewed_routing():
    """Zipf-biased gate logits: expert loads from 0 to capacity, heavy drops."""
    T, M, E, F, k = 4096, 256, 32, 256, 2
    inp = O.make_inputs(T, M, E, F, seed=2, zipf=1.2)
    m = build_module(inp, E, M, F, k, torch.bfloat16)
    m.gate[0].logit_bias = (inp["logit_bias"] * 4).cuda()
    x, y = run_module(m, inp, 1.25, torch.bfloat16)
    counts = m.last_plan.counts.cpu()
    assert counts.max() == m.last_plan.C and counts.min() < 64
    ref = run_oracle(inp, k, 1.25, torch.bfloat16, scores=m.last_plan.scores.cpu(),
                     logit_bias=inp["logit_bias"] * 4)
    compare(m, x, y, ref, torch.bfloat16)


def test_offloaded_experts_match_resident():
    """Same weights once GPU-resident and once streamed from pinned host memory through a
    4-slot pool in batches of 2: identical kernels in identical order, so identical bits."""
    T, M, E, F, k = 1024, 256, 8, 512, 1
    inp = O.make_inputs(T, M, E, F, seed=8)
    from mole_b200 import core as mcore
    res = build_module(inp, E, M, F, k, torch.bfloat16, ebatch=2)
    x1, y1 = run_module(res, inp, 1.25, torch.bfloat16)
    mcore.UniMem._instance = None
    off = build_module(inp, E, M, F, k, torch.bfloat16, d_experts=E, pool_size=4, ebatch=2)
    off.prefetch_fwd(2)
    x2, y2 = run_module(off, inp, 1.25, torch.bfloat16)
    assert torch.equal(y1, y2)
    assert torch.equal(x1.grad, x2.grad)
    assert torch.equal(res.FC1_W_GPU.grad_tensors.cpu(), off.FC1_W_CPU.all_tensors.grad_)
    assert torch.equal(res.FC2_W_GPU.grad_tensors.cpu(), off.FC2_W_CPU.all_tensors.grad_)
    assert torch.equal(res.FC1_B_GPU.grad_tensors.cpu(), off.FC1_B_CPU.all_tensors.grad_)
    assert torch.equal(res.FC2_B_GPU.grad_tensors.cpu(), off.FC2_B_CPU.all_tensors.grad_)
    mcore.UniMem._instance = None


def test_layer_bf16_gradient_accumulation_two_micro_batches():
    """``acc_step = 2``: every backward adds to the GPU-resident experts' gradient tensors
    (``acc = acc_step > 1``, MOLE/cpp/define.hpp:657; ``+=`` at MOLE/cpp/core.cpp:295-316) and
    zeroing is the optimizer's job.  Two micro-batches must leave the sum of their gradients, and
    after zeroing a third backward leaves just its own."""
    from mole_b200 import MOLEModule
    T, M, E, F, k = 1024, 256, 8, 512, 2
    a = O.make_inputs(T, M, E, F, seed=41)
    b = O.make_inputs(T, M, E, F, seed=41, token_seed=5)
    m = MOLEModule(0, E, M, F, -1, k, E, DIST1, "gelu", 2, False, False, dtype=torch.bfloat16)
    m.set_layer_state({"gate": [a["wg"], None],
                       "experts": [[a["w1"][e], a["b1"][e], a["w2"][e], a["b2"][e]] for e in range(E)]},
                      grad=False)
    refs = []
    for inp in (a, b):
        x, y = run_module(m, inp, 1.25, torch.bfloat16)
        refs.append(run_oracle(inp, k, 1.25, torch.bfloat16, scores=m.last_plan.scores.cpu()))
    for name, got in (("gw1", m.FC1_W_GPU.grad_tensors), ("gb1", m.FC1_B_GPU.grad_tensors),
                      ("gw2", m.FC2_W_GPU.grad_tensors), ("gb2", m.FC2_B_GPU.grad_tensors)):
        # the second backward adds to a bf16-rounded first gradient: one more rounding than the sum
        assert_close(got, refs[0][name] + refs[1][name], torch.bfloat16, name, scale=2.0)
    for p in (m.FC1_W_GPU, m.FC1_B_GPU, m.FC2_W_GPU, m.FC2_B_GPU):
        p.grad_tensors.zero_()
    x, y = run_module(m, a, 1.25, torch.bfloat16)
    assert_close(m.FC1_W_GPU.grad_tensors, refs[0]["gw1"], torch.bfloat16, "gw1 after zeroing")
    assert_close(m.FC2_W_GPU.grad_tensors, refs[0]["gw2"], torch.bfloat16, "gw2 after zeroing")


@pytest.mark.parametrize("k", [1, 2])
def test_layer_bf16_combine_fused_into_second_gemm(k):
    """The gate-weighted combine as part of the FC2 epilogue (bf16 reductions into y, MOLE/cpp/core.cpp:353
    followed by MOLE/moe/layer.py:456-458 in one kernel) against the oracle and against the layer with
    the separate combine kernel: same routing, y within tolerance, identical backward (it reads the
    same stored expert rows).  Ragged expert loads, so that rows carried along as a short last tile
    take part."""
    T, M, E, F = 2048 + 40, 256, 8, 512
    inp = O.make_inputs(T, M, E, F, seed=23)
    inp["wg"] = inp["wg"] * 5
    inp["b2"] = torch.randn(E, M, generator=torch.Generator().manual_seed(2)) * 0.05
    from mole_b200.moe.layer import MOLEModule
    res = {}
    for fused in (True, False):
        MOLEModule._instance.clear()
        m = build_module(inp, E, M, F, k, torch.bfloat16, fuse_combine=fused)
        x, y = run_module(m, inp, 1.25, torch.bfloat16)
        res[fused] = (m, x, y)
    m, x, y = res[True]
    ref = run_oracle(inp, k, 1.25, torch.bfloat16, scores=m.last_plan.scores.cpu())
    for name in ("idx", "slot", "counts", "offsets", "perm"):
        assert torch.equal(getattr(m.last_plan, name).cpu(), getattr(ref["routing"], name)), name
    assert_close(y, ref["y"], torch.bfloat16, "y with the fused combine")
    m0, x0, y0 = res[False]
    assert_close(y, y0.float(), torch.bfloat16, "fused vs separate combine")
    assert torch.equal(x.grad, x0.grad)
    assert torch.equal(m.FC1_W_GPU.grad_tensors, m0.FC1_W_GPU.grad_tensors)
    # the fused path really ran: a second forward without the fusion differs in rounding somewhere
    assert not torch.equal(y, y0) or k == 1


def test_layer_step_replayed_from_a_cuda_graph():
    """Forward + backward of a layer captured once in a CUDA graph and replayed: the replay gives
    the eager step's bits -- on the inputs of the capture and on new ones copied into the same
    tensors -- and leaves one graph launch per step on the host side."""
    from mole_b200.utils.Ugraph import GraphedStep
    T, M, E, F, k, cf = 2048, 256, 16, 512, 2, 1.25
    inp = O.make_inputs(T, M, E, F, seed=31)
    inp["wg"] = inp["wg"] * 5
    g = torch.Generator().manual_seed(5)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):          # leaves are created on the stream the step will be captured on
        m = build_module(inp, E, M, F, k, torch.bfloat16)
        x = inp["x"].to(torch.bfloat16).cuda().requires_grad_(True)
        gy = inp["gy"].to(torch.bfloat16).cuda()
        x2 = torch.randn(T, M, generator=g).to(torch.bfloat16).cuda()
    torch.cuda.synchronize()

    def step():
        x.grad = None
        m.gate[0].linear.weight.grad = None
        y = m(x, capacity_factor=cf)
        y.backward(gy)
        return y

    def snapshot(y):
        torch.cuda.synchronize()
        return [t.detach().clone() for t in (y, x.grad, m.gate[0].linear.weight.grad,
                                              m.FC1_W_GPU.grad_tensors, m.FC1_B_GPU.grad_tensors,
                                              m.FC2_W_GPU.grad_tensors, m.FC2_B_GPU.grad_tensors)]

    with torch.cuda.stream(s):
        eager1 = snapshot(step())
        with torch.no_grad():
            x_saved = x.detach().clone()
            x.copy_(x2)
        eager2 = snapshot(step())
        with torch.no_grad():
            x.copy_(x_saved)
    torch.cuda.synchronize()

    # the layer keeps l_aux (and with it the autograd graph of the last eager forward, whose leaf
    # nodes are tied to the stream of that forward): let it go before the capture
    m.l_aux = None
    graphed = GraphedStep(step, s)
    got1 = snapshot(graphed())
    with torch.no_grad():
        x.copy_(x2)
    got2 = snapshot(graphed())
    torch.cuda.synchronize()
    for name, a, b in zip(("y", "dx", "dWg", "gW1", "gb1", "gW2", "gb2"), eager1, got1):
        assert torch.equal(a, b), f"{name}: replay differs from the eager step"
    for name, a, b in zip(("y", "dx", "dWg", "gW1", "gb1", "gW2", "gb2"), eager2, got2):
        assert torch.equal(a, b), f"{name}: replay on new inputs differs from the eager step"
    assert not torch.equal(eager1[0], eager2[0])
