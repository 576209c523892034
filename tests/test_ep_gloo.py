"""Expert-parallel layout of the oracle on 2 CPU ranks (gloo): with experts block-partitioned
and the reference's capacity-padded all-to-all, every rank gets what the single-process layer
gives for that rank's tokens, forward and backward."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_ref as O

T, M, E, F, K, CF = 48, 16, 4, 32, 2, 1.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        L = E // world
        full = O.make_inputs(T, M, E, F, seed=5, token_seed=rank)
        full["b1"] = torch.randn(E, F, generator=torch.Generator().manual_seed(1)) * 0.1
        x = full["x"].clone().requires_grad_(True)
        sl = slice(rank * L, (rank + 1) * L)
        loc = [full[n][sl].clone().requires_grad_(True) for n in ("w1", "b1", "w2", "b2")]
        wg = full["wg"].clone().requires_grad_(True)
        out = O.moe_layer_ep(x, wg, *loc, k=K, capacity_factor=CF)
        (out.y * full["gy"]).sum().backward()

        # single-process layer on this rank's tokens with all experts
        x2 = full["x"].clone().requires_grad_(True)
        ws = [full[n].clone().requires_grad_(True) for n in ("wg", "w1", "b1", "w2", "b2")]
        ref = O.moe_layer(x2, *ws, k=K, capacity_factor=CF)
        (ref.y * full["gy"]).sum().backward()
        ok = torch.allclose(out.y, ref.y, atol=1e-5) and torch.allclose(x.grad, x2.grad, atol=1e-5)
        ok = ok and torch.equal(out.routing.slot, ref.routing.slot)
        ok = ok and torch.allclose(wg.grad, ws[0].grad, atol=1e-5)
        # expert gradients: a rank's experts collect the contributions of every rank's tokens
        contrib = torch.zeros(world, E, F, M)
        contrib[rank] = ws[1].grad
        dist.all_reduce(contrib)
        ok = ok and torch.allclose(loc[0].grad, contrib.sum(0)[sl], atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_oracle_ep_two_ranks_matches_single_process():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
