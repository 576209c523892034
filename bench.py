"""Benchmark of the MoE-layer hot path: forward + backward tokens/s of one ``MOLEModule``.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c3] [--impl ours|reference]

For N > 1 launch under ``python -m torch.distributed.run`` (one rank per GPU, NCCL).  Rank 0
prints one JSON line.  Workload (synthetic, seeded): the expert-parallel GPT-MoE block of the
benchmark configs -- 64 experts sharded over the ranks, 8192 tokens per rank x d_model 2048,
top-2 gate, d_ffn 8192, capacity factor 1.25, bf16 -- the config the headline metric
("MoE layer fwd+bwd tokens/s at 1/2/4/8 B200") is quoted on; it fits one GPU, so N = 1 runs it
with all 64 experts local.  ``--config c2|c4|c5`` select the other single-GPU configs; at N = 1
the default run also measures them for a few steps each (``other_configs``).

After the timed regions the last step's results are checked against the CPU oracle on a sample
(``parity``): routing integers bit-exact, two local experts' FFN outputs and gradients, the
layer output and input gradient of 64 tokens; a mismatch makes the run fail.

``--impl reference`` times the reference's algorithm on the host CPU: the reference ships no
CPU path and cannot be built or imported, so this arm runs the CPU oracle (a PyTorch
restatement, ``oracle/moe_ref.py``) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "moe_layer_fwd_bwd_tokens_per_s"
CONFIGS = {
    # tokens per rank, d_model, experts (total), top-k, d_ffn, capacity factor, seed
    "c1": dict(T=4096, M=512, E=8, k=2, F=2048, cf=1.25, seed=0,
               name="c1: 4096 tok x 512, 8 experts, top-2, d_ffn 2048, cf 1.25, fp32 (the CPU config)"),
    "c2": dict(T=16384, M=1024, E=64, k=2, F=4096, cf=1.25, seed=1,
               name="c2: 16384 tok x 1024, 64 experts, top-2, d_ffn 4096, cf 1.25, bf16, 1 GPU"),
    "c3": dict(T=8192, M=2048, E=64, k=2, F=8192, cf=1.25, seed=0,
               name="c3: expert-parallel block, 64 experts sharded, 8192 tok/rank x 2048, top-2, "
                    "d_ffn 8192, cf 1.25, bf16"),
    "c4": dict(T=16384, M=1024, E=64, k=2, F=4096, cf=1.25, seed=2, zipf=1.2,
               name="c4: c2 shape with Zipf(1.2) expert popularity"),
    "c5": dict(T=32768, M=2048, E=128, k=1, F=8192, cf=1.25, seed=3, offload=True, pool=16,
               name="c5: 128 offloaded experts (16 pool slots), 32768 tok x 2048, top-1, d_ffn 8192"),
}
RTOL_BF16 = 1e-2


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c3", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per rank (debugging)")
    ap.add_argument("--ffn-backend", type=int, default=0,
                    help="0 default, 1 CUDA cores, 2 one-CTA tcgen05, 3 CTA pairs (for comparisons)")
    ap.add_argument("--host-profile", action="store_true",
                    help="cProfile of the host side of a few steps on rank 0, printed to stderr")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="one GPU, GPU-resident experts: capture the step in a CUDA graph "
                         "(mole_b200.utils.Ugraph.GraphedStep) and time its replays")
    ap.add_argument("--timeline", default="",
                    help="write rank 0's kernel timeline of a few running steps (start, duration, gap "
                         "to the previous kernel; CUPTI through torch.profiler) to this file and exit")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernel-report", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    return ap.parse_args()


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"],
                    source="MEASURED_PEAKS.json (of measured)")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="recipe fallback (of fallback)")


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons through NVML (read-only) in a thread
    while the timed region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.sm, self.mask, self.max_mhz, self.error = [], 0, None, None
        self._stop = threading.Event()
        self.thread = None

    def _handle(self):
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(self.index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        try:
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid)

    def _run(self, pynvml, h):
        get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons",
                              getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons", None))
        while not self._stop.is_set():
            try:
                self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                if get_reasons:
                    self.mask |= int(get_reasons(h))
            except Exception as e:          # keep the benchmark running without clock data
                self.error = repr(e)
                return
            time.sleep(self.period)

    def __enter__(self):
        try:
            pynvml, h = self._handle()
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._run, args=(pynvml, h), daemon=True)
            self.thread.start()
        except Exception as e:
            self.error = repr(e)
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self.thread:
            self.thread.join(timeout=2)

    def summary(self):
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(n for bit, n in self.REASONS.items() if self.mask & bit),
               "samples": len(self.sm)}
        if self.error:
            out["error"] = self.error
        return out


# --------------------------------------------------------------------------------------------
# the layer under test
# --------------------------------------------------------------------------------------------
def init_weights(m, cfg, rank, L, dtype, device):
    """N(0, 0.02) weights seeded by global expert id, zero biases, N(0, 0.02) gate."""
    with torch.no_grad():
        g = torch.Generator(device=device).manual_seed(cfg["seed"])
        wg = torch.randn(cfg["E"], cfg["M"], generator=g, device=device) * 0.02
        m.gate[0].linear.weight.copy_(wg)
        offloaded = m.d_experts > 0
        for l in range(L):
            e = rank * L + l
            ge = torch.Generator(device=device).manual_seed(1_000_003 * (cfg["seed"] + 1) + e)
            w1 = torch.randn(cfg["F"], cfg["M"], generator=ge, device=device) * 0.02
            w2 = torch.randn(cfg["F"], cfg["M"], generator=ge, device=device) * 0.02
            kinds = ((m.FC1_W_CPU, m.FC1_B_CPU, m.FC2_W_CPU, m.FC2_B_CPU) if offloaded else
                     (m.FC1_W_GPU, m.FC1_B_GPU, m.FC2_W_GPU, m.FC2_B_GPU))
            kinds[0].fetch_single(l).copy_(w1)
            kinds[2].fetch_single(l).copy_(w2)
            kinds[1].fetch_single(l).zero_()
            kinds[3].fetch_single(l).zero_()
        if cfg.get("zipf"):
            # Gumbel-max construction: with logit noise of scale beta, P(expert is the top choice) is
            # proportional to rank^-s when the bias is -s * beta * ln(rank).  The gate's logits
            # are Gaussian with std 0.02 * sqrt(M); beta is the Gumbel scale of equal variance.
            ranks = torch.randperm(cfg["E"], generator=torch.Generator().manual_seed(cfg["seed"] + 99)) + 1
            beta = 0.02 * (cfg["M"] ** 0.5) * (6 ** 0.5) / 3.141592653589793
            m.gate[0].logit_bias = (-cfg["zipf"] * beta * torch.log(ranks.float())).to(device)


def build_layer(cfg, world, rank, local, dtype, ffn_backend):
    """A fresh ``MOLEModule`` for ``cfg`` with its seeded weights, tokens and upstream gradient."""
    from mole_b200 import MOLEModule
    from mole_b200 import core as mcore
    device = torch.device("cuda", local)
    T, M, E, F, k = (cfg[n] for n in ("T", "M", "E", "F", "k"))
    L = E // world
    dist_info = {"local_rank": local, "world_size": world, "rank": rank}
    MOLEModule._instance.clear()
    mcore.UniMem._instance = None
    if cfg.get("offload"):
        m = MOLEModule(E, 0, M, F, cfg["pool"], k, 8, dist_info, "gelu", 1, False, True, dtype=dtype,
                       ffn_backend=ffn_backend)
    else:
        m = MOLEModule(0, E, M, F, -1, k, max(L, 1), dist_info, "gelu", 1, False, False, dtype=dtype,
                       ffn_backend=ffn_backend)
    init_weights(m, cfg, rank, L, dtype, device)
    gt = torch.Generator(device=device).manual_seed(7_000_001 + rank)
    x = torch.randn(T, M, generator=gt, device=device).to(dtype).requires_grad_(True)
    gy = torch.randn(T, M, generator=gt, device=device).to(dtype)
    return m, x, gy


def bind_to_gpu_cores(index):
    """Several ranks on one host: keep this process (and with it the pinned host buffers it
    touches first) on the CPU cores next to its GPU, as NVML reports them.  A host-process
    setting only; returns the number of cores kept, or None when nothing was changed."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        near = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        keep = near & os.sched_getaffinity(0)
        if keep:
            os.sched_setaffinity(0, keep)
            return len(keep)
    except Exception:
        pass
    return None


class Harness:
    """Barrier, all-reduce and launch counting shared by the timed regions."""

    def __init__(self, world, device):
        self.world, self.device = world, device

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], device=self.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    @staticmethod
    def launches() -> int:
        from mole_b200 import _lib
        n = C.c_int64()
        _lib.check(_lib.lib.mole_launch_count(C.byref(n)))
        return n.value

    def timed(self, step, steps):
        """CUDA events around `steps` calls on the launching stream, max over ranks (ms in total).
        A ~25 ms GPU spin queued in front of the first event lets the host enqueue ahead, as it
        does in a steady training loop; it is not part of the timing."""
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        torch.cuda._sleep(50_000_000)
        ev0.record()
        h0 = time.perf_counter()
        for _ in range(steps):
            step()
        host_ms = (time.perf_counter() - h0) * 1e3 / steps     # enqueue time, no sync inside
        ev1.record()
        self.barrier()
        return self.max_over_ranks(ev0.elapsed_time(ev1)), host_ms


def make_step(m, x, gy, cf):
    def step():
        x.grad = None
        m.gate[0].linear.weight.grad = None
        y = m(x, capacity_factor=cf)
        y.backward(gy)
        return y
    return step


def warm_up(step, hs: Harness, warmup: int):
    """`warmup` steps, then keep warming (untimed, at most 60 more steps) until a synchronised
    step is within 15 % of the best one seen: a freshly started box can spend its first seconds
    paging the image in.  Every rank runs the same count."""
    for _ in range(max(warmup, 3)):
        step()
    hs.barrier()
    best, extra = float("inf"), 0
    while extra < 60:
        t0 = time.perf_counter()
        step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        extra += 1
        settled = dt <= 1.15 * best and extra >= 3
        best = min(best, dt)
        if hs.world > 1:
            import torch.distributed as dist
            flag = torch.tensor([0 if settled else 1], device=hs.device)
            dist.all_reduce(flag)
            settled = flag.item() == 0
        if settled:
            break
    hs.barrier()
    return extra


def write_timeline(step, hs: Harness, rank, path, steps=6):
    """Kernels of `steps` running layer steps in the order the GPU ran them, with the idle time
    in front of each: what the per-kernel events of `gemm_roofline` cannot show (the small
    kernels, the gaps, the waits of the expert-parallel barriers).  Per-step totals at the end."""
    from torch.profiler import ProfilerActivity, profile
    hs.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    hs.barrier()
    if rank != 0:
        return
    evs = sorted((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                 if e.device_type == torch.autograd.DeviceType.CUDA)
    first = [i for i, e in enumerate(evs) if "gate_topk" in e[2]]
    with open(path, "w") as out:
        prev_end = None
        for s0, s1, name in evs:
            gap = 0.0 if prev_end is None else s0 - prev_end
            out.write("%12.1f us  dur %8.1f  gap %7.1f  %s\n" % (s0 - evs[0][0], s1 - s0, gap, name[:100]))
            prev_end = s1 if prev_end is None else max(prev_end, s1)
        for a, b in zip(first, first[1:]):
            busy = sum(e[1] - e[0] for e in evs[a:b])
            gemm = sum(e[1] - e[0] for e in evs[a:b] if "gemm" in e[2] or "wgrad_resident" in e[2])
            out.write("step: %.1f us from its first kernel to the next step's; kernels %.1f us, of them "
                      "grouped GEMMs %.1f us; %d launches\n" % (evs[b][0] - evs[a][0], busy, gemm, b - a))
    print(json.dumps({"timeline": path, "kernels": len(evs), "steps": steps}))


def check_fault(where):
    from mole_b200 import ops
    fault = ops.device_fault()
    if fault:
        raise RuntimeError(f"device fault word = {fault} {where}: a kernel's bounded wait ran out")


# --------------------------------------------------------------------------------------------
# end to end: host buffers in, host buffers out, copies inside the timed region
# --------------------------------------------------------------------------------------------
class EndToEnd:
    """Every step copies its x and upstream gradient from pinned host memory and copies y and dx
    back.  The copies are double-buffered on two side streams (what an input pipeline does):
    step i+1's inputs travel while step i computes, step i's results travel while step i+1
    computes; everything is ordered by events and has landed when the region ends.  With
    ``compute=False`` only the copies run: the host-link roofline of the same traffic."""

    def __init__(self, m, x, gy, cf):
        self.m, self.cf = m, cf
        self.xh = x.detach().cpu().pin_memory()
        self.gyh = gy.cpu().pin_memory()
        self.yh = [torch.empty_like(self.xh).pin_memory() for _ in range(2)]
        self.dxh = [torch.empty_like(self.xh).pin_memory() for _ in range(2)]
        self.xd = [torch.empty_like(x, requires_grad=True) for _ in range(2)]
        self.gyd = [torch.empty_like(gy) for _ in range(2)]
        self.yd = torch.empty_like(gy)
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.in_ready = [torch.cuda.Event() for _ in range(2)]
        self.comp_done = [torch.cuda.Event() for _ in range(2)]
        self.out_done = [torch.cuda.Event() for _ in range(2)]
        self.bytes_in = 2 * x.numel() * x.element_size()
        self.bytes_out = 2 * x.numel() * x.element_size()

    def upload(self, buf):
        with torch.cuda.stream(self.s_in), torch.no_grad():
            self.s_in.wait_event(self.comp_done[buf])          # the buffers' previous step has finished
            self.xd[buf].copy_(self.xh, non_blocking=True)
            self.gyd[buf].copy_(self.gyh, non_blocking=True)
            self.in_ready[buf].record(self.s_in)

    def run(self, n, compute=True):
        cur = torch.cuda.current_stream()
        keep = []
        for b in range(2):
            self.comp_done[b].record(cur)
            self.out_done[b].record(cur)
        self.upload(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                self.upload(b ^ 1)
            cur.wait_event(self.in_ready[b])
            cur.wait_event(self.out_done[b])       # results of step i-2 have left this slot
            if compute:
                self.xd[b].grad = None
                self.m.gate[0].linear.weight.grad = None
                y = self.m(self.xd[b], capacity_factor=self.cf)
                y.backward(self.gyd[b])
                dx = self.xd[b].grad
                y = y.detach()
            else:
                y, dx = self.yd, self.gyd[b]
            self.comp_done[b].record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.comp_done[b])
                self.yh[b].copy_(y, non_blocking=True)
                self.dxh[b].copy_(dx, non_blocking=True)
                self.out_done[b].record(self.s_out)
            keep = keep[-2:] + [(y, dx)]       # alive until their copies are done
        cur.wait_event(self.out_done[0])
        cur.wait_event(self.out_done[1])


# --------------------------------------------------------------------------------------------
# parity of what was timed
# --------------------------------------------------------------------------------------------
def _err_over_scale(actual, expected, whole=False):
    """max |a - e| / (|e| + rms): the quantity the parity tests bound by rtol.  The rms is that of
    e's row for activations (rows differ in scale with their gate weight) and of the whole matrix
    for an expert's weight gradient (`whole`): a gradient row whose activations are all small
    sums rounding differences of bf16 pre-activations that are not small against that row."""
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    rms = e.pow(2).mean().sqrt() if whole else e.pow(2).mean(dim=-1, keepdim=True).sqrt()
    return float(((a - e).abs() / (e.abs() + rms).clamp_min(1e-30)).max()) if e.numel() else 0.0


def _rel_fro(actual, expected):
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    return float((a - e).norm() / e.norm().clamp_min(1e-30))


def parity_check(m, cfg, x, gy, y, world, rank, device, dtype):
    """The last step's results against the CPU oracle, on a sample sized for seconds of host
    work: (1) routing integers bit-exact against ``oracle.route`` on the GPU's own scores;
    (2) for sampled local experts (one whose last 128-row tile is ragged, and at 1-2 ranks the
    fullest one too) out, dx, gW1, gW2 against ``oracle.ffn_explicit`` on that expert's rows
    gathered from every rank's tokens; (3) y and x.grad of 64 tokens from the expert rows;
    (4) with several ranks, the pushed dispatch rows bit-exact.  Collective: every rank calls it."""
    import torch.distributed as dist
    from oracle import moe_ref as O
    plan, tap = m.last_plan, m.parity_tap
    T, M = x.shape
    E, k, Cap, Cs = plan.E, plan.k, plan.C, plan.Cs
    L = E // world
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(max(1, cores // world))
    out = {"rtol": RTOL_BF16, "checked_on": "last step of the timed regions"}

    # (1) routing
    r = O.route(plan.scores.cpu(), k, cfg["cf"])
    names = ("idx", "slot", "counts", "offsets", "perm")
    bad = [n for n in names if not torch.equal(getattr(plan, n).cpu(), getattr(r, n))]
    if r.capacity != Cap:
        bad.append("capacity")
    out["routing"] = "exact" if not bad else "MISMATCH in " + ",".join(bad)

    def gather(t):
        if world == 1:
            return [t]
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return parts

    xs, gys = gather(x.detach()), gather(gy)
    idxs, slots, gates = gather(plan.idx), gather(plan.slot), gather(plan.gates.detach())
    cnt = torch.stack(gather(plan.counts)).cpu()                    # [W, E]
    per_expert = cnt.sum(0)                                         # rows of every global expert
    n_samp = 2 if world <= 2 else 1
    sampled = []                                                    # global expert ids, same on every rank
    for q in range(world):
        loc = per_expert[q * L:(q + 1) * L]
        rag = loc % 128
        rag = torch.where(rag == 0, torch.full_like(rag, 1 << 20), rag)
        picks = [int(rag.argmin())]
        if n_samp > 1:
            order = torch.argsort(loc, descending=True).tolist()
            picks.append(next(o for o in order if o != picks[0]) if L > 1 else picks[0])
        sampled += [q * L + l for l in dict.fromkeys(picks)]
    rows_tap, dx_tap = tap["rows"].detach(), tap["dx_rows"].detach()
    mine_rows = torch.stack([rows_tap[e] for e in sampled])         # [S, Cs, M]
    mine_dx = torch.stack([dx_tap[e] for e in sampled])
    all_rows, all_dx = gather(mine_rows), gather(mine_dx)

    # (2) expert FFN of my sampled experts
    rd = lambda t: t.to(dtype).float()
    worst, worst_gw_elem, experts_checked, x0_exact = 0.0, 0.0, [], True
    peer = m.MOLECore._peer
    for si, e in enumerate(sampled):
        if e // L != rank:
            continue
        l = e - rank * L
        X, DO, OUT, DX = [], [], [], []
        packed_base = 0
        for w in range(world):
            sel = (idxs[w] == e) & (slots[w] < Cap)
            tok, j = sel.nonzero(as_tuple=True)
            order = torch.argsort(slots[w][tok, j])
            tok, j = tok[order], j[order]
            xr = xs[w][tok]
            X.append(xr.float().cpu())
            DO.append(rd(gates[w][tok, j].unsqueeze(1) * gys[w][tok].float()).cpu())
            n = int(cnt[w, e])
            assert n == tok.numel()
            OUT.append(all_rows[w][si, :n].float().cpu())
            DX.append(all_dx[w][si, :n].float().cpu())
            if peer is not None and peer.packed:      # one run per expert, sources in rank order
                run = peer.x0.view(L, world * Cs, M)[l]
                x0_exact = x0_exact and torch.equal(run[packed_base:packed_base + n], xr)
                packed_base += n
            elif peer is not None:
                x0_exact = x0_exact and torch.equal(peer.x0[w, l, :n], xr)
        X, DO, OUT, DX = (torch.cat(t) for t in (X, DO, OUT, DX))
        w1, b1, w2, b2 = (p.fetch_single(l).float().cpu()
                          for p in (m.FC1_W_GPU, m.FC1_B_GPU, m.FC2_W_GPU, m.FC2_B_GPU))
        ref = O.ffn_explicit(X, w1, b1, w2, b2, DO, dtype)
        gw1, gw2 = m.FC1_W_GPU.fetch_single_grad(l), m.FC2_W_GPU.fetch_single_grad(l)
        errs = {"out": _err_over_scale(OUT, ref["out"]), "dx": _err_over_scale(DX, ref["dx"]),
                "gW1_fro": _rel_fro(gw1, ref["gw1"]), "gW2_fro": _rel_fro(gw2, ref["gw2"])}
        worst = max(worst, *errs.values())
        # single elements of a weight gradient: reported, bounded by 4 x rtol (see the note)
        errs["gW1_max"] = _err_over_scale(gw1, ref["gw1"], whole=True)
        errs["gW2_max"] = _err_over_scale(gw2, ref["gw2"], whole=True)
        worst_gw_elem = max(worst_gw_elem, errs["gW1_max"], errs["gW2_max"])
        experts_checked.append({"expert": e, "rows": int(X.shape[0]), **errs})

    # (3) layer output and input gradient of 64 tokens, from the expert rows of this rank
    gtok = torch.Generator().manual_seed(1234 + rank)
    toks = torch.randperm(T, generator=gtok)[:64].to(device)
    ti, si_, ga = plan.idx[toks].long(), plan.slot[toks].long(), plan.gates.detach()[toks]
    kept = (si_ < Cap)
    flat = (ti * Cs + si_.clamp(max=Cs - 1))
    prow = rows_tap.reshape(E * Cs, M)[flat.view(-1)].view(64, k, M).float() * kept.unsqueeze(-1)
    y_ref = rd((prow * ga.unsqueeze(-1)).sum(1))
    dxrow = dx_tap.reshape(E * Cs, M)[flat.view(-1)].view(64, k, M).float() * kept.unsqueeze(-1)
    xg = x.detach()[toks].float().cpu().requires_grad_(True)
    lb = getattr(m.gate[0], "logit_bias", None)
    own = O.gate_scores(xg, m.gate[0].linear.weight.detach().float().cpu(),
                        lb.cpu() if lb is not None else None)
    g = torch.gather(own, 1, ti.cpu()) * kept.cpu()
    dgates = (prow * gy[toks].float().unsqueeze(1)).sum(-1).cpu()
    (g * dgates).sum().backward()
    dx_ref = rd(dxrow.sum(1).cpu() + xg.grad)
    e_y = _err_over_scale(y.detach()[toks], y_ref)
    e_dx = _err_over_scale(x.grad[toks], dx_ref)
    worst = max(worst, e_y, e_dx)
    out.update({"experts": experts_checked, "y_64_tokens": e_y, "dx_64_tokens": e_dx,
                "max_rel_err": worst})
    if peer is not None:
        out["pushed_dispatch_rows"] = "exact" if x0_exact else "MISMATCH"
    ok = (not bad) and worst <= RTOL_BF16 and worst_gw_elem <= 4 * RTOL_BF16 and x0_exact
    # every rank's verdict
    if world > 1:
        flag = torch.tensor([0 if ok else 1, 0], device=device, dtype=torch.float64)
        flag[1] = worst
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        out["max_rel_err_all_ranks"] = float(flag[1])
        ok = flag[0].item() == 0
    out["ok"] = bool(ok)
    out["note"] = ("max_rel_err = the largest of: max |actual - oracle| / (|oracle| + rms of the oracle's "
                   "row) for out / dx / y, and the relative Frobenius error of each weight gradient; "
                   "bound: rtol.  Single elements of a weight gradient (gW*_max, against |oracle| + rms "
                   "of the matrix) are bounded by 4 x rtol: a gradient element sums ~256 products of "
                   "bf16 activations, and where the GPU's accumulation order rounds a pre-activation to "
                   "the neighbouring bf16 value (0.1 % of them) one product moves by an ulp of a large "
                   "activation -- for a few of the 16.7 M elements that is 1-2 % of the matrix's rms.  "
                   "oracle = oracle/moe_ref.py on the host CPU in fp32 with bf16-rounded stored tensors")
    torch.set_num_threads(cores)
    return out


# --------------------------------------------------------------------------------------------
# rooflines
# --------------------------------------------------------------------------------------------
KINDS = {0: "FC1", 1: "FC2", 2: "dX2", 3: "dX", 4: "dW"}

# DRAM traffic of the six grouped-GEMM launches over their algorithmic bytes, measured once with
# ncu (dram__bytes_read.sum + dram__bytes_write.sum) on the config-2 shape at 8192 tokens:
# 4601 MB measured, 4498 MB algorithmic.
NCU_TRAFFIC_OVER_ALGORITHMIC = 1.02


def gemm_roofline(step, pairs, M, F, n_experts, pk, hs: Harness, reps=5):
    """Per-launch durations of the tensor-core grouped GEMM: CUDA events on its own stream around
    every launch, over `reps` layer steps after one discarded.  Algorithmic work of every one of
    the six launches is 2*P*M*F flops (P = kept pairs); padding rows, empty tiles and
    recomputation do not count."""
    from mole_b200 import _lib
    lib = _lib.lib
    cap = 8192
    ms = (C.c_float * cap)()
    kind = (C.c_int32 * cap)()
    n = C.c_int32()
    hs.barrier()
    _lib.check(lib.mole_profile_gemm(1))
    step()                                        # discarded: first step with the events in place
    hs.barrier()
    _lib.check(lib.mole_profile_read(ms, kind, cap, C.byref(n)))
    for _ in range(reps):
        step()
    hs.barrier()
    _lib.check(lib.mole_profile_gemm(0))
    _lib.check(lib.mole_profile_read(ms, kind, cap, C.byref(n)))
    per = {}
    for i in range(min(n.value, cap)):
        per.setdefault(KINDS.get(kind[i], str(kind[i])), []).append(ms[i])
    flops = 2.0 * pairs * M * F
    launches = {}
    total_ms = 0.0
    for name, v in per.items():
        per_step = sum(v) / reps
        total_ms += per_step
        launches[name] = {"launches_per_step": len(v) / reps, "ms_per_step": per_step,
                          "tflops": flops * (2 if name == "dW" else 1) / (per_step * 1e-3) / 1e12
                          if per_step > 0 else None}
    achieved = 6 * flops / (total_ms * 1e-3) / 1e12 if total_ms > 0 else 0.0
    # HBM side of the same launches (bf16): every launch moves the local experts' weights or
    # weight gradients once (n_experts * M * F elements) plus its row operands and outputs.
    wbytes = 2.0 * n_experts * M * F
    rows_m, rows_f = 2.0 * pairs * M, 2.0 * pairs * F
    alg_bytes = {"FC1": wbytes + rows_m + 2 * rows_f, "FC2": wbytes + rows_f + rows_m,
                 "dX2": wbytes + rows_m + 2 * rows_f, "dX": wbytes + rows_f + rows_m,
                 "dW": 2 * wbytes + 2 * (rows_f + rows_m)}
    total_bytes = sum(alg_bytes.values())
    roof = {"bound": "tensor", "kernel": "tc_gemm_kernel (6 launches per step: FC1, FC2, dW2, dX2, dW1, dX)",
            "achieved": achieved, "peak": pk["tf_burst"], "unit": "TFLOP/s",
            "frac": achieved / pk["tf_burst"],
            "frac_of_sustained_peak": achieved / pk["tf_sustained"], "peak_sustained": pk["tf_sustained"],
            "traffic": total_bytes * NCU_TRAFFIC_OVER_ALGORITHMIC / 6,
            "traffic_note": "bytes per launch, mean of the six: algorithmic bytes x the DRAM-traffic / "
                            "algorithmic ratio ncu measured on a smaller case of the same kernels "
                            "(traffic grows with the weights and rows like the algorithmic bytes do)",
            "peak_source": pk["source"] + "; frac is against the burst figure (the step is a few ms "
                           "at full clocks), frac_of_sustained_peak against the power-capped one",
            "algorithmic_flops_per_launch": flops, "ms_per_step_all_launches": total_ms,
            "profiled_steps": reps,
            "hbm_side": {"algorithmic_bytes_per_step": total_bytes,
                         "achieved_gbs": total_bytes / (total_ms * 1e-3) / 1e9 if total_ms > 0 else None,
                         "peak_gbs": pk["hbm"],
                         "frac": total_bytes / (total_ms * 1e-3) / 1e9 / pk["hbm"] if total_ms > 0 else None,
                         "note": "few rows per expert put these GEMMs at the ridge: the same launches "
                                 "read against the measured copy bandwidth"}}
    return roof, launches


def cublas_padded_gemm(L, R, M, F, device, reps=5):
    """The kernel to beat, alone: the reference's six batched GEMMs (MOLE/cpp/core.cpp:350-353,
    389-412) as stock PyTorch calls (cuBLAS strided-batched) on capacity-padded bf16 tensors
    [L, R, .], R = capacity x source ranks, every one timed with CUDA events."""
    bf = dict(dtype=torch.bfloat16, device=device)
    x = torch.randn(L, R, M, **bf)
    do = torch.randn(L, R, M, **bf)
    w1 = torch.randn(L, F, M, **bf) * 0.02
    w2 = torch.randn(L, F, M, **bf) * 0.02
    b1, b2 = torch.zeros(L, 1, F, **bf), torch.zeros(L, 1, M, **bf)
    h = torch.randn(L, R, F, **bf)
    dx1 = torch.randn(L, R, F, **bf)
    gw = torch.empty(L, F, M, **bf)
    ops = {
        "FC1": lambda: torch.baddbmm(b1, x, w1.transpose(1, 2)),
        "FC2": lambda: torch.baddbmm(b2, h, w2),
        "dW2": lambda: torch.matmul(h.transpose(1, 2), do, out=gw),
        "dX2": lambda: torch.matmul(do, w2.transpose(1, 2)),
        "dW1": lambda: torch.matmul(dx1.transpose(1, 2), x, out=gw),
        "dX": lambda: torch.matmul(dx1, w1),
    }
    res, total = {}, 0.0
    for name, fn in ops.items():
        fn()
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        b.synchronize()
        res[name] = a.elapsed_time(b) / reps
        total += res[name]
    del x, do, w1, w2, h, dx1, gw
    torch.cuda.empty_cache()
    return {"ms_sum_of_six": total, "ms": res, "padded_rows_per_expert": R,
            "tflops_on_padded_rows": 6 * 2.0 * L * R * M * F / (total * 1e-3) / 1e12,
            "note": "torch.baddbmm / torch.matmul (cuBLAS strided-batched, bf16) on the capacity-"
                    "padded [L, R, .] tensors, GEMMs only: no gelu, gelu', bias sums or re-layouts"}


def stock_torch_gpu(m, x, gy, k, cf, steps=5):
    """The reference's own GPU arithmetic restated with stock PyTorch on this GPU, whole layer:
    softmax gate, top-k routing with capacity (one-hot cumsum), capacity-padded [E, C, M]
    buffer, torch.baddbmm -> gelu -> torch.baddbmm over ALL padded rows (MOLE/cpp/core.cpp:350-353),
    weighted combine; backward by autograd.  Same weights, tokens and upstream gradient as the
    measured step; cuBLAS strided-batched GEMMs.  Device-resident, one GPU."""
    import torch.nn.functional as Fn
    T, M = x.shape
    wg = m.gate[0].linear.weight.detach().clone().requires_grad_(True)
    params = [p.all_tensors.detach().clone().requires_grad_(True)
              for p in (m.FC1_W_GPU, m.FC1_B_GPU, m.FC2_W_GPU, m.FC2_B_GPU)]
    w1, b1, w2, b2 = params
    E = w1.shape[0]
    cap = max(1, math.ceil(k * cf * T / E))
    xin = x.detach().clone().requires_grad_(True)
    tok = torch.arange(T, device=x.device).repeat(k)

    def one():
        for t in (xin, wg, *params):
            t.grad = None
        scores = torch.softmax(xin.float() @ wg.float().t(), -1)
        gates, idx = torch.topk(scores, k, dim=-1)
        flat = idx.t().reshape(-1)                                   # all first choices, then second
        pos = (Fn.one_hot(flat, E).cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1)
        keep = pos < cap
        disp = xin.new_zeros(E, cap, M)
        disp = disp.index_put((flat[keep], pos[keep]), xin[tok[keep]])
        h = Fn.gelu(torch.baddbmm(b1.view(E, 1, -1), disp, w1.transpose(1, 2)))
        o = torch.baddbmm(b2.view(E, 1, -1), h, w2)
        g = (gates.t().reshape(-1) * keep).to(o.dtype)
        rows = o[flat, pos.clamp(max=cap - 1)] * g[:, None]
        y = torch.zeros_like(xin).index_add_(0, tok, rows)
        y.backward(gy)

    for _ in range(2):
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    del params, wg, xin
    torch.cuda.empty_cache()
    return {"value": T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "note": "stock PyTorch on the same GPU (cuBLAS strided-batched baddbmm over the "
                    "capacity-padded [E, C, M] buffer, autograd backward, whole layer incl. a "
                    "one-hot-cumsum router): the reference's GPU arithmetic, not this library"}


def hbm_kernel_report(m, x, gy, cf, pk):
    """Achieved HBM bandwidth of the gate / dispatch / combine kernels on the benchmark shape
    (algorithmic bytes / CUDA-event time, 5 launches each after a warm-up)."""
    from mole_b200 import ops
    plan = m.last_plan
    T, M = x.shape
    E, k = plan.E, plan.k
    es = x.element_size()
    P = int(plan.counts.sum().item())
    xd = x.detach()
    wg = m.gate[0].linear.weight.detach()
    rows = ops.dispatch(xd, plan)
    # L2 flush by READING a 256 MiB buffer that is never written: afterwards L2 holds clean lines
    # only.  (A memset flush leaves 126 MB of dirty lines whose write-back then competes with the
    # timed kernel: the ~20 us launches here read 8-10 us longer after one.)
    big = torch.zeros(64 << 20, dtype=torch.int32, device=x.device)

    def timeit(fn):
        fn()
        ts = []
        for _ in range(5):
            big.sum()
            torch.cuda._sleep(400_000)      # ~0.2 ms of GPU spin: the host enqueues the rest meanwhile
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    rep = {}

    def add(name, fn, nbytes):
        t = timeit(fn)
        gbs = nbytes / (t * 1e-3) / 1e9
        rep[name] = {"ms": t, "algorithmic_bytes": nbytes, "gbs": gbs, "frac_of_hbm_peak": gbs / pk["hbm"]}

    add("gate_route", lambda: ops.gate_route(xd, wg, k, plan.C, getattr(m.gate[0], "logit_bias", None)),
        T * M * es + T * E * 4)
    add("dispatch_fwd", lambda: ops.dispatch(xd, plan, out=rows), 2 * P * M * es)
    add("combine_fwd", lambda: ops.combine(rows, plan, plan.gates), (P + T) * M * es)
    add("combine_bwd", lambda: ops.combine_bwd(gy, rows, plan, plan.gates), 3 * P * M * es + P * 4)
    add("dispatch_bwd", lambda: ops.dispatch_bwd(rows, plan, M, x.dtype, x.device), (P + T) * M * es)
    dlogits = torch.randn(T, E, device=x.device) * 1e-3
    add("dispatch_bwd_with_gate_dx (the launch the layer uses: + dlogits @ Wg)",
        lambda: ops.dispatch_bwd(rows, plan, M, x.dtype, x.device, dlogits, wg),
        (P + T) * M * es + T * E * 4 + E * M * es)
    fill = torch.empty(1 << 30, dtype=torch.uint8, device=x.device)
    add("memset_1GiB (write-only reference)", lambda: fill.zero_(), fill.numel())
    src = torch.empty(1 << 30, dtype=torch.uint8, device=x.device)
    add("copy_1GiB (read+write reference)", lambda: fill.copy_(src), 2 * fill.numel())
    rep["peak_gbs"] = pk["hbm"]
    rep["note"] = "L2 flushed (a 256 MiB read-only buffer is summed) before every timed launch"
    return rep


def pinned_copy_peak(device, nbytes=1 << 30, reps=3):
    """Pinned host <-> device copy bandwidth of this GPU's host link, each direction alone and
    both at once (GB/s)."""
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h2 = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d2 = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s2 = torch.cuda.Stream()

    def t(fn):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return nbytes * reps / (a.elapsed_time(b) * 1e-3) / 1e9

    h2d = t(lambda: d.copy_(h, non_blocking=True))
    d2h = t(lambda: h.copy_(d, non_blocking=True))

    def both():
        cur = torch.cuda.current_stream()
        s2.wait_stream(cur)
        d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            h2.copy_(d2, non_blocking=True)
        cur.wait_stream(s2)

    duplex = t(both)
    return {"h2d_gbs": h2d, "d2h_gbs": d2h, "duplex_gbs_per_direction": duplex}


# --------------------------------------------------------------------------------------------
# one configuration, a few steps (the other single-GPU configs)
# --------------------------------------------------------------------------------------------
def run_small_config(key, local, ffn_backend, pk, steps):
    """c2 / c4 / c5 on one GPU for a few steps: tokens/s and the grouped GEMM's roofline; for the
    offloaded config also the host-link side (bytes, achieved GB/s, overlap)."""
    cfg = dict(CONFIGS[key])
    device = torch.device("cuda", local)
    dtype = torch.bfloat16
    hs = Harness(1, device)
    m, x, gy = build_layer(cfg, 1, 0, local, dtype, ffn_backend)
    step = make_step(m, x, gy, cfg["cf"])
    for _ in range(3):
        step()
    hs.barrier()
    ms, _ = hs.timed(step, steps)
    ms_per_step = ms / steps
    plan = m.last_plan
    pairs = int(plan.counts.sum().item())
    T, M, E, F, k = (cfg[n] for n in ("T", "M", "E", "F", "k"))
    res = {"workload": cfg["name"], "value": T / (ms_per_step * 1e-3), "unit": "tokens/s",
           "ms_per_step": ms_per_step, "steps": steps, "kept_pairs": pairs,
           "drop_rate": 1.0 - pairs / (T * k)}
    roof, launches = gemm_roofline(step, pairs, M, F, E, pk, hs, reps=3)
    res["roofline"] = {n: roof[n] for n in ("bound", "achieved", "peak", "unit", "frac",
                                            "frac_of_sustained_peak", "ms_per_step_all_launches")}
    res["gemm_launches"] = launches
    if cfg.get("offload"):
        es = 2
        per_expert = (2 * F * M + F + M) * es
        h2d = 2 * E * per_expert            # weights fetched for forward and again for backward
        d2h = E * per_expert                # weight gradients
        link = pinned_copy_peak(device)
        t_copy = max(h2d / (link["h2d_gbs"] * 1e9), d2h / (link["d2h_gbs"] * 1e9)) * 1e3
        t_comp = roof["ms_per_step_all_launches"]
        res["offload"] = {
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "h2d_achieved_gbs": h2d / (ms_per_step * 1e-3) / 1e9,
            "d2h_achieved_gbs": d2h / (ms_per_step * 1e-3) / 1e9,
            "pinned_copy_peak": link,
            "roofline": {"bound": "host link", "ms_copy_alone_at_peak": t_copy,
                         "ms_gemm_alone": t_comp, "ms_per_step": ms_per_step,
                         "frac": t_copy / ms_per_step,
                         "overlap_fraction": max(0.0, min(1.0, (t_copy + t_comp - ms_per_step) /
                                                          max(min(t_copy, t_comp), 1e-9)))},
            "note": "config 5 is bound by the host link, not by the tensor cores: frac = time the "
                    "step's H2D bytes need at the measured pinned-copy bandwidth / step time; "
                    "overlap_fraction = share of the shorter of (copies, GEMMs) hidden behind the other"}
    check_fault(f"after {key}")
    del m, x, gy, step
    from mole_b200 import MOLEModule, core as mcore
    MOLEModule._instance.clear()
    mcore.UniMem._instance = None
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from mole_b200.utils.Udist import MOLEDist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    near_cores = bind_to_gpu_cores(local) if world > 1 else None
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    cfg = dict(CONFIGS[args.config])
    if args.tokens:
        cfg["T"] = args.tokens
    dtype = torch.bfloat16
    T, M, E, F, k, cf = (cfg[n] for n in ("T", "M", "E", "F", "k", "cf"))
    L = E // world
    MOLEDist(local_rank=local)
    hs = Harness(world, device)
    # --cuda-graph: the layer and its inputs are created on the stream the step is captured on
    # (autograd ties the accumulation into a leaf's .grad to the stream of its creation)
    use_graph = bool(args.cuda_graph) and world == 1 and not cfg.get("offload")
    gstream = torch.cuda.Stream() if use_graph else None
    if use_graph:
        with torch.cuda.stream(gstream):
            m, x, gy = build_layer(cfg, world, rank, local, dtype, args.ffn_backend)
        torch.cuda.synchronize()
    else:
        m, x, gy = build_layer(cfg, world, rank, local, dtype, args.ffn_backend)
    want_parity = not args.no_parity and not cfg.get("offload")
    if want_parity:
        m.parity_tap = {}
    step = make_step(m, x, gy, cf)
    if use_graph:
        # eager runs of the step (warm-up, GEMM timing, parity) stay on the capture stream as well
        raw_step = step

        def step():
            with torch.cuda.stream(gstream):
                return raw_step()

    extra = warm_up(step, hs, args.warmup)
    check_fault("after the warm-up")

    if args.timeline:
        write_timeline(step, hs, rank, args.timeline)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.host_profile and rank == 0:
        import cProfile
        import pstats
        prof = cProfile.Profile()
        prof.enable()
        for _ in range(5):
            step()
        prof.disable()
        torch.cuda.synchronize()
        pstats.Stats(prof, stream=sys.stderr).sort_stats("cumulative").print_stats(45)
    elif args.host_profile:
        for _ in range(5):
            step()
    hs.barrier()

    # ---- device-resident timed region --------------------------------------------------------
    # A region in which the host needed nearly as long to enqueue a step as the GPU to run it
    # (another tenant's job on the host's cores) measures the host, not the kernels: it is taken
    # again, at most twice, and the count is reported.
    timed_step, launches_per_step = step, None
    if use_graph:
        from mole_b200.utils.Ugraph import GraphedStep
        m.l_aux = None                        # lets the eager steps' autograd graph go
        if want_parity:
            m.parity_tap = {}
        torch.cuda.synchronize()
        c0 = hs.launches()
        timed_step = GraphedStep(raw_step, gstream, warmup=3)
        launches_per_step = (hs.launches() - c0) // 4      # three warm-up runs and the captured one
        for _ in range(3):
            timed_step()
        hs.barrier()
    host_bound_retries = 0
    while True:
        with ClockSampler(local) as clocks:
            n0 = hs.launches()
            ms, host_ms = hs.timed(timed_step, args.steps)
            n1 = hs.launches()
        host_bound = hs.max_over_ranks(1.0 if host_ms >= 0.85 * ms / args.steps else 0.0) > 0
        if not host_bound or host_bound_retries >= 2:
            break
        host_bound_retries += 1
    ms_per_step = ms / args.steps
    value = world * T / (ms_per_step * 1e-3)
    check_fault("after the timed region")

    # ---- end to end ------------------------------------------------------------------------
    e2e_run = EndToEnd(m, x, gy, cf)
    e2e_run.run(2)
    hs.barrier()
    torch.cuda._sleep(50_000_000)       # same queue-ahead spin; the first upload waits behind it
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    e2e_run.run(args.steps)
    ev1.record()
    hs.barrier()
    ms2 = hs.max_over_ranks(ev0.elapsed_time(ev1))
    e2e_value = world * T / (ms2 / args.steps * 1e-3)
    # host-link roofline of the same traffic: every rank does only the copies, no compute
    link_steps = min(args.steps, 50)
    e2e_run.run(2, compute=False)
    hs.barrier()
    ev0.record()
    e2e_run.run(link_steps, compute=False)
    ev1.record()
    hs.barrier()
    ms3 = hs.max_over_ranks(ev0.elapsed_time(ev1)) / link_steps
    e2e = {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": e2e_run.bytes_in,
           "d2h_bytes_per_step": e2e_run.bytes_out, "ms_per_step": ms2 / args.steps,
           "host_link_roofline": {
               "ms_per_step_copies_only": ms3,
               "gbs_per_direction_per_gpu": e2e_run.bytes_in / (ms3 * 1e-3) / 1e9,
               "tokens_per_s_if_copy_bound": world * T / (ms3 * 1e-3),
               "e2e_frac_of_copy_bound": (ms3 / (ms2 / args.steps)),
               "e2e_frac_of_device_resident": e2e_value / value,
               "note": "the same double-buffered pinned copies on every rank at once with no compute "
                       "between them; e2e cannot be faster than max(this, the device-resident step)"},
           "note": "x and upstream grad copied from pinned host memory, y and dx copied back, every step; "
                   "copies double-buffered on side streams, all landed inside the timed region"}
    check_fault("after the end-to-end region")

    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["name"], "tokens_per_rank": T, "d_model": M, "experts": E,
                   "top_k": k, "d_ffn": F, "capacity_factor": cf, "local_experts": L,
                   "parallelism": f"ep{world}",
                   "l2": "per-step working set (weights, gradients, activations) is >10 GB, far above "
                         "the 126 MB L2, so no flush is needed between iterations",
                   "timing": "CUDA events around the K steps on the launching stream; a ~25 ms GPU spin "
                             "queued before the first event lets the host enqueue ahead"},
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": (n1 - n0) if launches_per_step is None else launches_per_step * args.steps,
        "cuda_graph": use_graph,
        "host_enqueue_ms_per_step": host_ms, "host_bound_retries": host_bound_retries,
        "warmup_settling_steps": extra,
    }
    if near_cores:
        out["host_cores_near_gpu"] = near_cores
    plan = m.last_plan
    pairs = int(plan.counts.sum().item())
    out["config"]["kept_pairs_rank0"] = pairs
    out["config"]["drop_rate_rank0"] = 1.0 - pairs / (T * k)

    # ---- parity of the last step -------------------------------------------------------------
    if want_parity:
        y = step()
        torch.cuda.synchronize()
        out["parity"] = parity_check(m, cfg, x, gy, y, world, rank, device, dtype)
        m.parity_tap = None
        check_fault("after the parity step")

    pk = peaks()
    # at N > 1 a rank's local experts see the pairs every rank routed to them
    local_pairs = pairs
    if world > 1:
        cnt = plan.counts.clone()
        dist.all_reduce(cnt)
        local_pairs = int(cnt[rank * L:(rank + 1) * L].sum().item())
    out["roofline"], out["gemm_launches"] = gemm_roofline(step, local_pairs, M, F, L, pk, hs)
    if rank == 0 and not args.no_kernel_report and not cfg.get("offload"):
        R = world * math.ceil(k * cf * T / E)
        out["cublas_padded_gemm"] = cublas_padded_gemm(L, R, M, F, device)
        ours = out["roofline"]["ms_per_step_all_launches"]
        out["cublas_padded_gemm"]["ours_ms_sum_of_six"] = ours
        out["cublas_padded_gemm"]["speedup_over_cublas"] = out["cublas_padded_gemm"]["ms_sum_of_six"] / ours
    if rank == 0 and not args.no_kernel_report and not cfg.get("offload"):
        out["hbm_kernels"] = hbm_kernel_report(m, x, gy, cf, pk)
    if rank == 0 and world == 1 and not args.no_kernel_report and not cfg.get("offload"):
        out["stock_torch_gpu"] = stock_torch_gpu(m, x, gy, k, cf)
    if world == 1 and not args.no_kernel_report and not cfg.get("offload"):
        # the combine fused into the FC2 epilogue against the separate combine kernel, same box,
        # alternating (device-resident steps)
        keep = m.fuse_combine
        ab = {True: [], False: []}
        for _ in range(3):
            for fused in (True, False):
                m.fuse_combine = fused
                for _ in range(3):
                    step()
                t, _ = hs.timed(step, 20)
                ab[fused].append(t / 20)
        m.fuse_combine = keep
        out["combine_fusion"] = {"fused_ms_per_step": statistics.median(ab[True]),
                                 "separate_ms_per_step": statistics.median(ab[False]),
                                 "default": "separate kernel (fuse_combine=True selects the fused epilogue)",
                                 "note": "whole fwd+bwd step, 3 x 20 steps each way, alternating"}
    check_fault("after the kernel reports")
    hs.barrier()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_full_c1(steps=3, warmup=1)
        out["cpu_baseline_sample_of_workload"] = cpu_sample(cfg, steps=3, warmup=1)
    if rank == 0 and world == 1 and not args.no_other_configs and args.config == "c3":
        del step, e2e_run
        m.MOLECore.close_peer_exchange()
        del m, x, gy
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        out["other_configs"] = {key: run_small_config(key, local, args.ffn_backend, pk, steps)
                                for key, steps in (("c2", 20), ("c4", 20), ("c5", 3))}
    hs.barrier()
    if rank == 0:
        print(json.dumps(out))
    ok = out.get("parity", {}).get("ok", True)
    if world > 1:
        dist.destroy_process_group()
    if not ok:
        print("parity check FAILED: " + json.dumps(out.get("parity")), file=sys.stderr)
        sys.exit(3)


# --------------------------------------------------------------------------------------------
# CPU arms: the oracle
# --------------------------------------------------------------------------------------------
def _cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return ""


def _time_oracle(T, M, E, F, k, cf, seed, steps, warmup):
    from oracle import moe_ref as O
    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    wg = torch.randn(E, M, generator=g) * 0.02
    w1 = torch.empty(E, F, M).normal_(0, 0.02, generator=g)
    w2 = torch.empty(E, F, M).normal_(0, 0.02, generator=g)
    b1, b2 = torch.zeros(E, F), torch.zeros(E, M)
    x = torch.randn(T, M, generator=g)
    gy = torch.randn(T, M, generator=g)
    params = [t.requires_grad_(True) for t in (wg, w1, b1, w2, b2)]
    xr = x.requires_grad_(True)

    def one():
        for t in params + [xr]:
            t.grad = None
        t0 = time.perf_counter()
        out = O.moe_layer(xr, *params, k=k, capacity_factor=cf)
        out.y.backward(gy)
        return time.perf_counter() - t0

    for _ in range(warmup):
        one()
    times = [one() for _ in range(steps)]
    return statistics.median(times), threads


def cpu_full_c1(steps, warmup):
    """The CPU oracle on config 1 at full size (4096 x 512, 8 experts, top-2, d_ffn 2048, fp32,
    autograd backward, capacity-padded baddbmm like MOLE/cpp/core.cpp:350-353), all host threads:
    the configuration the CPU baseline is defined on."""
    c = CONFIGS["c1"]
    med, threads = _time_oracle(c["T"], c["M"], c["E"], c["F"], c["k"], c["cf"], c["seed"], steps, warmup)
    return {"value": c["T"] / med, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"config 1 at full size ({c['name']}); fp32 oracle, median of {steps} fwd+bwd "
                      f"after {warmup} warm-up",
            "seconds_per_step": med, "cpu": _cpu_model()}


def cpu_sample(cfg, steps, warmup, fraction=8):
    """1/fraction sample of the workload: E/fraction experts and T/fraction tokens with the same
    d_model, d_ffn, top-k and capacity factor, so every expert sees the same number of rows and
    the work per token is that of the full layer.  fp32, autograd backward, all host threads."""
    E = max(cfg["k"], cfg["E"] // fraction)
    T = max(64, cfg["T"] // fraction)
    med, threads = _time_oracle(T, cfg["M"], E, cfg["F"], cfg["k"], cfg["cf"], cfg["seed"], steps, warmup)
    return {"value": T / med, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"1/{fraction} of the workload: {E} of {cfg['E']} experts, {T} of {cfg['T']} tokens, "
                      f"same d_model/d_ffn/top-k/capacity factor; fp32 oracle, median of {steps} fwd+bwd",
            "tokens_run": T, "experts_run": E,
            "seconds_per_step": med, "cpu": _cpu_model()}


def run_reference(args):
    """The reference's algorithm on the host cores.  The reference itself cannot run here (it has no
    CPU path, does not build as shipped and calls an un-vendored routing package), so this is the
    CPU oracle; under torchrun only rank 0 works.  Each step is a bounded sample of the workload
    (1/8 of the experts and of the tokens, same work per token: about a quarter of a second), so
    that K steps and W warm-up steps as given end within minutes (K is capped at 300)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = dict(CONFIGS[args.config])
    if args.tokens:
        cfg["T"] = args.tokens
    world = int(os.environ.get("WORLD_SIZE", "1"))
    steps = max(1, min(args.steps, 300))
    warmup = max(1, min(args.warmup, 10))
    b = cpu_sample(cfg, steps=steps, warmup=warmup)
    ms = b["seconds_per_step"] * 1e3
    out = {
        "impl": "reference", "metric": METRIC, "value": b["value"], "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"] + " -- CPU arm: a 1/8 sample of it per step",
                   "tokens_per_rank": b["tokens_run"], "d_model": cfg["M"],
                   "experts": b["experts_run"], "top_k": cfg["k"], "d_ffn": cfg["F"],
                   "capacity_factor": cfg["cf"], "parallelism": "cpu",
                   "full_workload": {"tokens_per_rank": cfg["T"], "experts": cfg["E"]}},
        "cpu_baseline": b,
        "cpu_baseline_config1": cpu_full_c1(steps=3, warmup=1),
        "e2e": {"value": b["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
