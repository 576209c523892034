"""Worker of the expert-parallel GPU test: one process per GPU (launched by
``torch.distributed.run``).  Every rank runs the layer on its own tokens with its shard of the
experts and checks output, input gradient, gate gradient and its experts' gradients against the
oracle's explicit forward + backward, which needs no communication: a rank's tokens see all
experts, and an expert's gradient is the sum of what every rank's tokens contribute."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oracle import moe_ref as O  # noqa: E402
from util import assert_close  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mole_b200 import MOLEModule

    T, M, E, F, k, cf = 1024, 256, 8, 512, 2, 1.0
    dtype = torch.bfloat16
    L = E // world
    per_rank = [O.make_inputs(T, M, E, F, seed=31, token_seed=r) for r in range(world)]
    for inp in per_rank:
        inp["wg"] = inp["wg"] * 5
        inp["b1"] = torch.randn(E, F, generator=torch.Generator().manual_seed(1)) * 0.05
        inp["b2"] = torch.randn(E, M, generator=torch.Generator().manual_seed(2)) * 0.05
    mine = per_rank[rank]
    # "records": two records per rank, NCCL all-to-all per record.  "push": one record, rows
    # stored straight into the consuming rank's memory (dispatch / FC2 / combine bwd / dX).
    # "push_pair": the same with the CTA-pair kernel forced, so that its row map / peer scatter runs
    # on several ranks (by default this small shape picks the one-CTA kernel).
    mode = sys.argv[1] if len(sys.argv) > 1 else "records"
    push = mode.startswith("push")
    ebatch = L if push else max(1, L // 2)
    m = MOLEModule(0, E, M, F, -1, k, ebatch, {"local_rank": local, "world_size": world, "rank": rank},
                   "gelu", 1, False, False, dtype=dtype, ffn_backend=3 if mode == "push_pair" else 0)
    sl = slice(rank * L, (rank + 1) * L)
    m.set_layer_state({"gate": [mine["wg"], None],
                       "experts": [[mine["w1"][e], mine["b1"][e], mine["w2"][e], mine["b2"][e]]
                                   for e in range(rank * L, (rank + 1) * L)]}, grad=False)
    x = mine["x"].to(dtype).cuda().requires_grad_(True)
    for _ in range(2 if push else 1):      # twice: the push buffers are reused per step
        x.grad = None
        m.gate[0].linear.weight.grad = None
        y = m(x, capacity_factor=cf)
        (y.float() * mine["gy"].cuda()).sum().backward()
    torch.cuda.synchronize()
    if push:
        assert m.MOLECore._peer is not None, "the push-style exchange was not taken"
    else:
        assert m.MOLECore._peer is None

    # every rank's routing decisions come from that rank's GPU scores
    scores = [torch.empty(T, E, device="cuda") for _ in range(world)]
    dist.all_gather(scores, m.last_plan.scores)
    rd = lambda t: t.to(dtype).float()
    refs = []
    for r, inp in enumerate(per_rank):
        refs.append(O.layer_explicit(rd(inp["x"]), rd(inp["gy"]), rd(inp["wg"]), rd(inp["w1"]),
                                     rd(inp["b1"]), rd(inp["w2"]), rd(inp["b2"]), k, cf, dtype,
                                     scores=scores[r].cpu()))
    ref = refs[rank]
    for name in ("idx", "slot", "counts", "perm"):
        assert torch.equal(getattr(m.last_plan, name).cpu(), getattr(ref["routing"], name)), name
    assert_close(y, ref["y"], dtype, f"rank {rank} y")
    assert_close(x.grad, ref["dx"], dtype, f"rank {rank} dx")
    assert_close(m.gate[0].linear.weight.grad, ref["dwg"], dtype, f"rank {rank} dWg", scale=4.0)
    got = {"gw1": m.FC1_W_GPU.grad_tensors, "gb1": m.FC1_B_GPU.grad_tensors,
           "gw2": m.FC2_W_GPU.grad_tensors, "gb2": m.FC2_B_GPU.grad_tensors}
    for name, g in got.items():
        # the GPU sums all ranks' rows in one fp32 accumulation; the per-rank references were each
        # rounded to bf16 before this sum, hence the wider tolerance
        want = sum(r[name][sl] for r in refs)
        assert_close(g, want, dtype, f"rank {rank} {name}", scale=2.0)
    m.MOLECore.close_peer_exchange()
    dist.barrier()
    if rank == 0:
        print("EP_OK", world, mode)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
