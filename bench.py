"""Benchmark of the MoE-layer hot path: forward + backward tokens/s of one ``MOLEModule``.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c3] [--impl ours|reference]

For N > 1 launch under ``python -m torch.distributed.run`` (one rank per GPU, NCCL).  Rank 0
prints one JSON line.  Workload (synthetic, seeded): the expert-parallel GPT-MoE block of the
benchmark configs -- 64 experts sharded over the ranks, 8192 tokens per rank x d_model 2048,
top-2 gate, d_ffn 8192, capacity factor 1.25, bf16 -- the config the headline metric
("MoE layer fwd+bwd tokens/s at 1/2/4/8 B200") is quoted on; it fits one GPU, so N = 1 runs it
with all 64 experts local.  ``--config c2|c4|c5`` select the other single-GPU configs.

``--impl reference`` times the reference's algorithm on the host CPU: the reference ships no
CPU path and cannot be built or imported, so this arm runs the CPU oracle (a PyTorch
restatement, ``oracle/moe_ref.py``) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per rank (debugging)")
    ap.add_argument("--ffn-backend", type=int, default=0,
                    help="0 default (CTA pairs), 1 CUDA cores, 2 one-CTA tcgen05 (for comparisons)")
    ap.add_argument("--host-profile", action="store_true",
                    help="cProfile of the host side of a few steps on rank 0, printed to stderr")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernel-report", action="store_true")
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
# our arm
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


def run_ours(args):
    import torch.distributed as dist
    from mole_b200 import MOLEModule, _lib, ops
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
    dist_info = {"local_rank": local, "world_size": world, "rank": rank}
    if cfg.get("offload"):
        m = MOLEModule(E, 0, M, F, cfg["pool"], k, 8, dist_info, "gelu", 1, False, True, dtype=dtype,
                       ffn_backend=args.ffn_backend)
    else:
        m = MOLEModule(0, E, M, F, -1, k, max(L, 1), dist_info, "gelu", 1, False, False, dtype=dtype,
                       ffn_backend=args.ffn_backend)
    init_weights(m, cfg, rank, L, dtype, device)

    gt = torch.Generator(device=device).manual_seed(7_000_001 + rank)
    x = torch.randn(T, M, generator=gt, device=device).to(dtype).requires_grad_(True)
    gy = torch.randn(T, M, generator=gt, device=device).to(dtype)

    def step():
        x.grad = None
        m.gate[0].linear.weight.grad = None
        y = m(x, capacity_factor=cf)
        y.backward(gy)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def launches():
        n = C.c_int64()
        _lib.check(_lib.lib.mole_launch_count(C.byref(n)))
        return n.value

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # A freshly started box can spend its first seconds paging the image in, and the host then
    # enqueues slower than the GPU executes.  Keep warming (untimed, at most 60 more steps) until
    # a synchronised step is within 15 % of the best one seen; every rank runs the same count.
    best, extra = float("inf"), 0
    while extra < 60:
        t0 = time.perf_counter()
        step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        extra += 1
        settled = dt <= 1.15 * best and extra >= 3
        best = min(best, dt)
        if world > 1:
            flag = torch.tensor([0 if settled else 1], device=device)
            dist.all_reduce(flag)
            settled = flag.item() == 0
        if settled:
            break
    barrier()
    fault = ops.device_fault()
    if fault:
        raise RuntimeError(f"device fault word = {fault}: a kernel's bounded wait ran out")

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
    barrier()

    # ---- device-resident timed region --------------------------------------------------------
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        n0 = launches()
        # ~25 ms of GPU spin in front of the first event: the host enqueues several steps ahead
        # while it runs, as it does in a steady training loop, so a host-side hiccup on a shared
        # machine does not leave the GPU idle inside the timed region.  Not part of the timing.
        torch.cuda._sleep(50_000_000)
        ev0.record()
        h0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        host_ms = (time.perf_counter() - h0) * 1e3 / args.steps     # enqueue time, no sync inside
        ev1.record()
        barrier()
        n1 = launches()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_per_step = ms / args.steps
    value = world * T / (ms_per_step * 1e-3)

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region ------
    # Every step copies its x and upstream gradient from pinned host memory and copies y and dx
    # back.  The copies are double-buffered on two side streams (what an input pipeline does):
    # step i+1's inputs travel while step i computes, step i's results travel while step i+1
    # computes; everything is ordered by events and has landed when the region ends.
    xh = x.detach().cpu().pin_memory()
    gyh = gy.cpu().pin_memory()
    yh = [torch.empty_like(xh).pin_memory() for _ in range(2)]
    dxh = [torch.empty_like(xh).pin_memory() for _ in range(2)]
    xd = [torch.empty_like(x, requires_grad=True) for _ in range(2)]
    gyd = [torch.empty_like(gy) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_ready = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def upload(buf):
        with torch.cuda.stream(s_in), torch.no_grad():
            s_in.wait_event(comp_done[buf])          # the buffers' previous step has finished
            xd[buf].copy_(xh, non_blocking=True)
            gyd[buf].copy_(gyh, non_blocking=True)
            in_ready[buf].record(s_in)

    def run_e2e(n):
        cur_stream = torch.cuda.current_stream()
        keep = []
        for b in range(2):
            comp_done[b].record(cur_stream)
            out_done[b].record(cur_stream)
        upload(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                upload(b ^ 1)
            cur_stream.wait_event(in_ready[b])
            cur_stream.wait_event(out_done[b])       # results of step i-2 have left this slot
            xd[b].grad = None
            m.gate[0].linear.weight.grad = None
            y = m(xd[b], capacity_factor=cf)
            y.backward(gyd[b])
            comp_done[b].record(cur_stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                yh[b].copy_(y.detach(), non_blocking=True)
                dxh[b].copy_(xd[b].grad, non_blocking=True)
                out_done[b].record(s_out)
            keep = keep[-2:] + [(y, xd[b].grad)]       # alive until their copies are done
        cur_stream.wait_event(out_done[0])
        cur_stream.wait_event(out_done[1])

    run_e2e(2)
    barrier()
    # same queue-ahead spin as above; the first upload waits on an event recorded behind it, so
    # no copy of the timed steps starts before the first event
    torch.cuda._sleep(50_000_000)
    ev0.record()
    run_e2e(args.steps)
    ev1.record()
    barrier()
    ms2 = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms2], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms2 = t.item()
    e2e_value = world * T / (ms2 / args.steps * 1e-3)
    es = x.element_size()
    e2e = {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * M * es,
           "d2h_bytes_per_step": 2 * T * M * es,
           "note": "x and upstream grad copied from pinned host memory, y and dx copied back, every step; "
                   "copies double-buffered on side streams, all landed inside the timed region"}

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
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": n1 - n0,
        "host_enqueue_ms_per_step": host_ms, "warmup_settling_steps": extra,
    }
    if near_cores:
        out["host_cores_near_gpu"] = near_cores
    plan = m.last_plan
    pairs = int(plan.counts.sum().item())
    out["config"]["kept_pairs_rank0"] = pairs
    out["config"]["drop_rate_rank0"] = 1.0 - pairs / (T * k)

    pk = peaks()
    if rank == 0 or world > 1:
        out["roofline"], out["gemm_launches"] = gemm_roofline(step, pairs, M, F, L, pk, barrier)
    if rank == 0 and not args.no_kernel_report and not cfg.get("offload"):
        out["hbm_kernels"] = hbm_kernel_report(m, x, gy, cf, pk)
    if rank == 0 and world == 1 and not args.no_kernel_report and not cfg.get("offload"):
        out["stock_torch_gpu"] = stock_torch_gpu(m, x, gy, k, cf)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_sample(cfg, steps=3, warmup=1)
    barrier()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


KINDS = {0: "FC1", 1: "FC2", 2: "dX2", 3: "dX", 4: "dW"}


# DRAM traffic of the six grouped-GEMM launches over their algorithmic bytes, from one ncu capture
# (profiles/tc_gemm_c2_tokens8192_ncu_full.md: 4601 MB measured, 4498 MB algorithmic).
NCU_TRAFFIC_OVER_ALGORITHMIC = 1.02


def gemm_roofline(step, pairs, M, F, n_experts, pk, barrier):
    """Per-launch durations of the tensor-core grouped GEMM (CUDA events on its own stream, inside
    two extra layer steps).  Algorithmic work of every one of the six launches is 2*P*M*F flops
    (P = kept pairs); padding rows, empty tiles and recomputation do not count."""
    from mole_b200 import _lib
    lib = _lib.lib
    barrier()
    _lib.check(lib.mole_profile_gemm(1))
    reps = 2
    for _ in range(reps):
        step()
    barrier()
    _lib.check(lib.mole_profile_gemm(0))
    n = C.c_int32()
    cap = 4096
    ms = (C.c_float * cap)()
    kind = (C.c_int32 * cap)()
    _lib.check(lib.mole_profile_read(ms, kind, cap, C.byref(n)))
    per = {}
    for i in range(min(n.value, cap)):
        per.setdefault(KINDS.get(kind[i], str(kind[i])), []).append(ms[i])
    flops = 2.0 * pairs * M * F
    launches = {}
    total_ms = 0.0
    for name, v in per.items():
        per_step = sum(v) / reps
        n_launch = len(v) / reps
        total_ms += per_step
        launches[name] = {"launches_per_step": n_launch, "ms_per_step": per_step,
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
    # ncu, dram__bytes_read.sum + dram__bytes_write.sum of the six launches over their algorithmic
    # bytes, from the capture summarised in profiles/ (measured once, not live)
    traffic_ratio = NCU_TRAFFIC_OVER_ALGORITHMIC
    roof = {"bound": "tensor", "kernel": "tc_gemm_kernel (6 launches per step: FC1, FC2, dW2, dX2, dW1, dX)",
            "achieved": achieved, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
            "frac": achieved / pk["tf_sustained"],
            "traffic": total_bytes * traffic_ratio / 6 if traffic_ratio else None,
            "traffic_note": "bytes per launch, mean of the six: algorithmic bytes x the DRAM-traffic / "
                            "algorithmic ratio ncu measured on a smaller case of the same kernels "
                            "(traffic grows with the weights and rows like the algorithmic bytes do)",
            "peak_source": pk["source"] + ", sustained figure: the kernel is timed inside a long step",
            "algorithmic_flops_per_launch": flops, "ms_per_step_all_launches": total_ms,
            "hbm_side": {"algorithmic_bytes_per_step": total_bytes,
                         "achieved_gbs": total_bytes / (total_ms * 1e-3) / 1e9 if total_ms > 0 else None,
                         "peak_gbs": pk["hbm"],
                         "frac": total_bytes / (total_ms * 1e-3) / 1e9 / pk["hbm"] if total_ms > 0 else None,
                         "note": "few rows per expert put these GEMMs at the ridge: the same launches "
                                 "read against the measured copy bandwidth"}}
    return roof, launches


def stock_torch_gpu(m, x, gy, k, cf, steps=5):
    """The reference's own GPU arithmetic restated with stock PyTorch on this GPU, as the kernel to
    beat: softmax gate, top-k routing with capacity (one-hot cumsum), capacity-padded [E, C, M]
    buffer, torch.baddbmm -> gelu -> torch.baddbmm over ALL padded rows (MOLE/cpp/core.cpp:350-353),
    weighted combine; backward by autograd.  Same weights, tokens and upstream gradient as the
    measured step; cuBLAS strided-batched GEMMs.  Device-resident, one GPU."""
    import math
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
                    "capacity-padded [E, C, M] buffer, autograd backward): the reference's GPU "
                    "arithmetic, not this library"}


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
    drows = torch.empty_like(rows)
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


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle on a bounded sample of the workload
# --------------------------------------------------------------------------------------------
def cpu_sample(cfg, steps, warmup, fraction=8):
    """1/fraction sample of the workload: E/fraction experts and T/fraction tokens with the same
    d_model, d_ffn, top-k and capacity factor, so every expert sees the same number of rows and
    the work per token is that of the full layer.  fp32, autograd backward, all host threads."""
    from oracle import moe_ref as O
    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    E = max(cfg["k"], cfg["E"] // fraction)
    T = max(64, cfg["T"] // fraction)
    M, F, k, cf = cfg["M"], cfg["F"], cfg["k"], cfg["cf"]
    g = torch.Generator().manual_seed(cfg["seed"])
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
    med = statistics.median(times)
    model = ""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                model = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    return {"value": T / med, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"1/{fraction} of the workload: {E} of {cfg['E']} experts, {T} of {cfg['T']} tokens, "
                      f"same d_model/d_ffn/top-k/capacity factor; fp32 oracle, median of {steps} fwd+bwd",
            "seconds_per_step": med, "cpu": model}


def run_reference(args):
    """The reference's algorithm on the host cores.  The reference itself cannot run here (it has no
    CPU path, does not build as shipped and calls an un-vendored routing package), so this is the
    CPU oracle; under torchrun only rank 0 works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = dict(CONFIGS[args.config])
    if args.tokens:
        cfg["T"] = args.tokens
    world = int(os.environ.get("WORLD_SIZE", "1"))
    b = cpu_sample(cfg, steps=max(1, args.steps), warmup=max(1, min(args.warmup, 2)))
    ms = b["seconds_per_step"] * 1e3
    out = {
        "impl": "reference", "metric": METRIC, "value": b["value"], "unit": "tokens/s",
        "n_gpus": world, "steps": max(1, args.steps), "warmup": max(1, min(args.warmup, 2)),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "tokens_per_rank": cfg["T"], "d_model": cfg["M"],
                   "experts": cfg["E"], "top_k": cfg["k"], "d_ffn": cfg["F"],
                   "capacity_factor": cfg["cf"], "parallelism": "cpu"},
        "cpu_baseline": b,
        "e2e": {"value": b["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
