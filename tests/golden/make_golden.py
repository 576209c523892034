"""Generates the golden fixtures in this directory from the CPU oracle (oracle/moe_ref.py).

    python tests/golden/make_golden.py

The reference (atc23-101/MOLE) holds no tests or known-answer vectors and cannot be imported
or built, so these fixtures pin the oracle against itself: a change in the oracle's routing or
arithmetic shows up as a diff here.  ``small.npz`` holds a complete small case (inputs, routing
integers, outputs and gradients); ``c1_routing.npz`` holds the routing integers and float64
checksums of outputs / gradients for benchmark config 1 (4096 x 512, 8 experts, top-2, fp32,
seed 0).
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import moe_ref as O  # noqa: E402

HERE = Path(__file__).resolve().parent


def run(inp, k, cf):
    x = inp["x"].clone().requires_grad_(True)
    names = ("wg", "w1", "b1", "w2", "b2")
    ws = [inp[n].clone().requires_grad_(True) for n in names]
    out = O.moe_layer(x, *ws, k=k, capacity_factor=cf, logit_bias=inp["logit_bias"])
    (out.y * inp["gy"]).sum().backward()
    grads = {"dx": x.grad, **{"d" + n: w.grad for n, w in zip(names, ws)}}
    return out, grads


def small():
    T, M, E, F, k, cf = 96, 64, 8, 128, 2, 0.75          # capacity 18: some pairs are dropped
    inp = O.make_inputs(T, M, E, F, seed=11)
    inp["x"] = inp["x"] * 2.0
    inp["wg"] = inp["wg"] * 10.0                          # spread the scores
    inp["b1"] = torch.randn(E, F, generator=torch.Generator().manual_seed(5)) * 0.1
    inp["b2"] = torch.randn(E, M, generator=torch.Generator().manual_seed(6)) * 0.1
    out, grads = run(inp, k, cf)
    r = out.routing
    np.savez_compressed(
        HERE / "small.npz", T=T, M=M, E=E, F=F, k=k, cf=cf,
        **{n: inp[n].numpy() for n in ("x", "gy", "wg", "w1", "b1", "w2", "b2")},
        scores=out.scores.detach().numpy(), idx=r.idx.numpy(), slot=r.slot.numpy(),
        gates=r.gates.detach().numpy(), counts=r.counts.numpy(), offsets=r.offsets.numpy(),
        perm=r.perm.numpy(), capacity=r.capacity, l_aux=float(r.l_aux.detach()),
        y=out.y.detach().numpy(), **{n: g.numpy() for n, g in grads.items()})
    print("small: capacity", r.capacity, "kept", int(r.kept.sum()), "of", T * k)


def c1():
    cfg = O.CONFIGS["c1"]
    inp = O.make_inputs(cfg["T"], cfg["M"], cfg["E"], cfg["F"], cfg["seed"])
    out, grads = run(inp, cfg["k"], cfg["cf"])
    r = out.routing
    sums = {n: float(g.double().sum()) for n, g in grads.items()}
    sums["y"] = float(out.y.detach().double().sum())
    abs_sums = {n + "_abs": float(g.double().abs().sum()) for n, g in grads.items()}
    abs_sums["y_abs"] = float(out.y.detach().double().abs().sum())
    np.savez_compressed(
        HERE / "c1_routing.npz", idx=r.idx.numpy().astype(np.int8), slot=r.slot.numpy().astype(np.int16),
        counts=r.counts.numpy(), offsets=r.offsets.numpy(), capacity=r.capacity,
        l_aux=float(r.l_aux.detach()), **sums, **abs_sums)
    print("c1: counts", r.counts.tolist())


if __name__ == "__main__":
    torch.manual_seed(0)
    small()
    c1()
