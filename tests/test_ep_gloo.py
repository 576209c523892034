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


# --------------------------------------------------------------------------------------------
# host side of the product's exchange: records -> byte geometry of each all-to-all
# --------------------------------------------------------------------------------------------
def _all2all_bytes(recv, send, bytes_per_peer, peer_stride, offset, rank, world):
    """What the library's exchange does with these arguments, on CPU tensors through gloo: block
    ``q`` of ``send`` (``bytes_per_peer`` bytes at ``offset + q * peer_stride``) goes to rank
    ``q`` and lands in block ``rank`` of its ``recv``."""
    sb, rb = send.view(torch.uint8).view(-1), recv.view(torch.uint8).view(-1)
    outs = [sb[offset + q * peer_stride: offset + q * peer_stride + bytes_per_peer].clone()
            for q in range(world)]
    ins = [torch.empty(bytes_per_peer, dtype=torch.uint8) for _ in range(world)]
    ins[rank].copy_(outs[rank])
    reqs = [dist.isend(outs[q], q) for q in range(world) if q != rank]
    reqs += [dist.irecv(ins[q], q) for q in range(world) if q != rank]
    for r in reqs:
        r.wait()
    for r in range(world):
        rb[offset + r * peer_stride: offset + r * peer_stride + bytes_per_peer] = ins[r]


def _geometry_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mole_b200.core import build_records, exchange_geometry
        L, Cs, Md = 6, 4, 8                        # 6 local experts in records of 4 and 2
        E_total = L * world
        # element (e, s, m) of rank r's dispatched buffer carries its own coordinates
        disp = torch.empty(E_total, Cs, Md)
        for e in range(E_total):
            disp[e] = rank * 1000 + e * 10 + torch.arange(Cs)[:, None] + torch.zeros(Md)
        records, groups = build_records(L, 0, 4, False, 0, 0)
        assert [(r.base_in_all, r.batch_size) for r in records] == [(0, 4), (4, 2)]
        chunk_bytes = Cs * Md * disp.element_size()
        x0 = torch.full((world, L, Cs, Md), -1.0)
        for rec in records:
            _all2all_bytes(x0, disp, *exchange_geometry(rec, L, chunk_bytes), rank, world)
        # rank `rank` owns global experts [rank * L, (rank + 1) * L): chunk [w][l] must be what
        # source rank w dispatched to global expert rank * L + l
        ok = True
        for w in range(world):
            for l in range(L):
                want = w * 1000 + (rank * L + l) * 10 + torch.arange(Cs)[:, None] + torch.zeros(Md)
                ok = ok and torch.equal(x0[w, l], want)
        # the return exchange with the same geometry brings every chunk back to its source
        back = torch.full_like(disp, -1.0)
        for rec in records:
            _all2all_bytes(back, x0, *exchange_geometry(rec, L, chunk_bytes), rank, world)
        ok = ok and torch.equal(back, disp)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_record_exchange_geometry_two_ranks():
    """The byte ranges the pipeline hands to the exchange, record by record, reproduce the
    expert-parallel layout ([source rank][local expert] chunks) and its inverse."""
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_geometry_worker, args=(world, port, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world)), dict(ret)

