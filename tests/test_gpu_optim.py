"""The optimizer step fused behind backward for offloaded experts ("instant Adam",
MOLE/cpp/core.cpp:848-943, 1216-1227), the mixed optimizer and checkpoint file
(MOLE/optim/mixed_optim.py:155-343, MOLE/utils/Uscheduler.py:66-92) and the scheduler's profiling /
prefetch policy on a two-layer stack (MOLE/utils/Uscheduler.py:228-349)."""
import pytest
import torch

from oracle import moe_ref as O

pytestmark = pytest.mark.gpu
DIST1 = {"local_rank": 0, "world_size": 1, "rank": 0}


def _fresh():
    from mole_b200 import MOLEModule
    from mole_b200 import core as mcore
    from mole_b200.utils.Uscheduler import UniScheduler
    MOLEModule._instance.clear()
    MOLEModule._cpu_optimizer = None
    mcore.UniMem._instance = None
    UniScheduler._instance = None
    UniScheduler._optimizer = None


def _layer(inp, E, M, F, k, dtype, offload, adv_adam=False, acc_step=1, pool=4, ebatch=2):
    from mole_b200 import MOLEModule
    if offload:
        m = MOLEModule(E, 0, M, F, pool, k, ebatch, DIST1, "gelu", acc_step, adv_adam, True, dtype=dtype)
    else:
        m = MOLEModule(0, E, M, F, -1, k, ebatch, DIST1, "gelu", acc_step, False, False, dtype=dtype)
    m.set_layer_state({"gate": [inp["wg"], None],
                       "experts": [[inp["w1"][e], inp["b1"][e], inp["w2"][e], inp["b2"][e]]
                                   for e in range(E)]}, grad=False)
    return m


def _run(m, inp, dtype):
    x = inp["x"].to(dtype).cuda().requires_grad_(True)
    y = m(x, capacity_factor=1.25)
    (y.float() * inp["gy"].cuda()).sum().backward()
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("adamw", [False, True])
def test_instant_adam_matches_torch_adam_on_resident_experts(adamw):
    """fp32 layer, all experts offloaded, the Adam step taken on the GPU behind each expert
    batch's backward -- against the same layer with GPU-resident experts stepped by
    ``torch.optim.Adam`` / ``AdamW``: parameters and both moments within fp32 rtol 1e-5 after
    three steps."""
    from mole_b200.utils.Uscheduler import UniScheduler
    T, M, E, F, k = 512, 128, 8, 256, 1
    dtype = torch.float32
    inp = O.make_inputs(T, M, E, F, seed=12)
    inp["b1"] = torch.randn(E, F, generator=torch.Generator().manual_seed(1)) * 0.05
    hp = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.05)

    _fresh()
    res = _layer(inp, E, M, F, k, dtype, offload=False, ebatch=E)
    kinds = (res.FC1_W_GPU, res.FC1_B_GPU, res.FC2_W_GPU, res.FC2_B_GPU)
    params = [p.fetch_all_with_grad() for p in kinds]
    opt = (torch.optim.AdamW if adamw else torch.optim.Adam)(params, **hp)
    outs_ref, want_first = [], None
    for i in range(3):
        outs_ref.append(_run(res, inp, dtype).detach().cpu())
        opt.step()
        if i == 0:
            want_first = [p.detach().cpu().clone() for p in params]
    want = [p.detach().cpu().clone() for p in params]
    want_m = [opt.state[p]["exp_avg"].cpu() for p in params]
    want_v = [opt.state[p]["exp_avg_sq"].cpu() for p in params]

    _fresh()
    UniScheduler(local_rank=0, disable_overlap=False, adv_adam=True, gate_control_by_MOLE=False)
    off = _layer(inp, E, M, F, k, dtype, offload=True, adv_adam=True)
    mixed = UniScheduler.build_optimizer(adamW=adamw, **hp)
    assert mixed.hasCPU and not mixed.hasGPU
    for step in range(3):
        UniScheduler.set_step(step)
        UniScheduler.adam_set()                      # step count for the bias correction
        y = _run(off, inp, dtype)
        torch.testing.assert_close(y.detach().cpu(), outs_ref[step], rtol=1e-5, atol=1e-6)
        mixed.step()                                 # offloaded experts: only counts the step
        mixed.zero_grad()
        UniScheduler.zero_grad()
        if step == 0:
            # same parameters and (bit-identical) gradients went into both first steps: only the
            # order of the update's fp32 operations differs
            for name, p, w in zip(("W1", "b1", "W2", "b2"),
                                  (off.FC1_W_CPU, off.FC1_B_CPU, off.FC2_W_CPU, off.FC2_B_CPU), want_first):
                torch.testing.assert_close(p.all_tensors, w, rtol=1e-5, atol=1e-8,
                                           msg=lambda s: f"first step {name}: {s}")
    got = [p.all_tensors for p in (off.FC1_W_CPU, off.FC1_B_CPU, off.FC2_W_CPU, off.FC2_B_CPU)]
    # Later steps see gradients that differ in their last bits (the parameters do); where an
    # element's gradient changes sign between steps the normalised update amplifies that, hence an
    # absolute term of 5e-4 of the distance the three steps can move a parameter (3 lr).
    atol = 5e-4 * 3 * hp["lr"]
    for name, g, w, wm, wv in zip(("W1", "b1", "W2", "b2"), got, want, want_m, want_v):
        torch.testing.assert_close(g, w, rtol=1e-5, atol=atol, msg=lambda s: f"{name}: {s}")
        # moments of elements whose gradient nearly cancels over the steps: absolute term at 1e-4
        # of the largest moment
        torch.testing.assert_close(g.momentum, wm, rtol=1e-4, atol=1e-4 * float(wm.abs().max()),
                                   msg=lambda s: f"m {name}: {s}")
        torch.testing.assert_close(g.variance, wv, rtol=1e-4, atol=1e-4 * float(wv.abs().max()),
                                   msg=lambda s: f"v {name}: {s}")
    _fresh()


def test_instant_adam_bf16_hybrid_split():
    """bf16, six offloaded experts of which the first four are stepped on the GPU and the last two
    by the host optimizer from their stored gradients: every expert must move, with one formula."""
    from mole_b200.utils.Uscheduler import UniScheduler
    T, M, E, F, k = 512, 128, 6, 256, 1
    dtype = torch.bfloat16
    inp = O.make_inputs(T, M, E, F, seed=13)
    _fresh()
    sched = UniScheduler(local_rank=0, disable_overlap=False, adv_adam=True, hybrid_adam=True,
                         gate_control_by_MOLE=False)
    off = _layer(inp, E, M, F, k, dtype, offload=True, adv_adam=True, pool=4, ebatch=2)
    mixed = UniScheduler.build_optimizer(lr=1e-2)
    UniScheduler.set_hybrid(4)
    before = off.FC1_W_CPU.all_tensors.clone()
    UniScheduler.set_step(0)
    UniScheduler.adam_set()
    _run(off, inp, dtype)
    after_gpu = off.FC1_W_CPU.all_tensors.clone()
    assert not torch.equal(after_gpu[:4], before[:4])          # stepped on the GPU
    assert torch.equal(after_gpu[4:], before[4:])              # still waiting for the host step
    g = off.FC1_W_CPU.all_tensors.grad_.float()
    assert g[4:].abs().sum() > 0                               # their gradients came back
    mixed.step()
    after = off.FC1_W_CPU.all_tensors
    assert torch.equal(after[:4], after_gpu[:4]) and not torch.equal(after[4:], before[4:])
    # first Adam step with zero moments: |delta| = lr wherever the gradient is not tiny
    big = g.abs() > 1e-3
    delta = (after.float() - before.float()).abs()
    assert ((delta[big] - 1e-2).abs() < 2e-3).all()
    _fresh()


def test_mixed_optimizer_and_checkpoint_round_trip(tmp_path):
    """Two layers with GPU-resident and offloaded experts under ``MOLEMixedAdam``; ``save_states``
    after two steps, two more steps, ``load_states`` into a fresh model + optimizer, the same two
    steps again: identical parameters (checkpoint = parameters, gradients, moments, step counts)."""
    from mole_b200 import MOLEModule
    from mole_b200.utils.Uscheduler import UniScheduler
    T, M, F, k = 256, 128, 256, 2
    dtype = torch.float32
    inps = [O.make_inputs(T, M, 8, F, seed=20 + i) for i in range(2)]

    def build():
        _fresh()
        UniScheduler(local_rank=0, disable_overlap=False, adv_adam=False, gate_control_by_MOLE=True)
        layers = []
        for inp in inps:
            m = MOLEModule(4, 4, M, F, 4, k, 2, DIST1, "gelu", 1, False, True, dtype=dtype)
            m.set_layer_state({"gate": [inp["wg"], None],
                               "experts": [[inp["w1"][e], inp["b1"][e], inp["w2"][e], inp["b2"][e]]
                                           for e in range(8)]}, grad=False)
            layers.append(m)
        opt = UniScheduler.build_optimizer(lr=1e-2)
        assert opt.hasCPU and opt.hasGPU and opt.hasGate
        return layers, opt

    def step(layers, opt, s):
        UniScheduler.set_step(s)
        x = inps[0]["x"].cuda().requires_grad_(True)
        h = x
        for m in layers:
            h = h + m(h, capacity_factor=1.25)
        (h * inps[0]["gy"].cuda()).sum().backward()
        torch.cuda.synchronize()
        opt.step(AllreduceGate=False)
        opt.zero_grad()
        UniScheduler.zero_grad()

    def snapshot(layers):
        return [m.get_layer_state(False) for m in layers]

    layers, opt = build()
    for s in range(2):
        step(layers, opt, s)
    UniScheduler.save_states(str(tmp_path / "ckpt"), grad=False)
    for s in range(2, 4):
        step(layers, opt, s)
    want = snapshot(layers)

    layers2, opt2 = build()
    UniScheduler.load_states(str(tmp_path / "ckpt"), grad=False)
    for s in range(2, 4):
        step(layers2, opt2, s)
    got = snapshot(layers2)
    for a, b in zip(got, want):
        torch.testing.assert_close(a["gate"][0], b["gate"][0], rtol=1e-6, atol=1e-7)
        for ea, eb in zip(a["experts"], b["experts"]):
            for ta, tb in zip(ea, eb):
                torch.testing.assert_close(ta, tb, rtol=1e-6, atol=1e-7)
    _fresh()


def test_scheduler_profiles_gaps_and_prefetches():
    """Two layers of offloaded experts driven as a training loop drives the reference: profiling
    steps measure the gaps in front of each layer and one expert's fetch time, the scheduler sets
    per-layer prefetch counts, and the steps that then run with prefetching produce the same
    output as the steps before."""
    from mole_b200 import MOLEModule
    from mole_b200.utils.Uscheduler import UniScheduler
    T, M, F, k, E = 256, 128, 256, 1, 4
    dtype = torch.bfloat16
    inps = [O.make_inputs(T, M, E, F, seed=30 + i) for i in range(2)]
    _fresh()
    sched = UniScheduler(local_rank=0, disable_overlap=False, adv_adam=False, gate_control_by_MOLE=True)
    layers = []
    for inp in inps:
        m = MOLEModule(E, 0, M, F, 6, k, 2, DIST1, "gelu", 1, False, True, dtype=dtype)
        m.set_layer_state({"gate": [inp["wg"], None],
                           "experts": [[inp["w1"][e], inp["b1"][e], inp["w2"][e], inp["b2"][e]]
                                       for e in range(E)]}, grad=False)
        layers.append(m)
    UniScheduler.schedule_policy(profile_step=4, prefetch_on=True)
    x = inps[0]["x"].to(dtype).cuda()
    outs = []
    for s in range(8):
        UniScheduler.set_step(s)
        UniScheduler.prefetch_fwd()
        xs = x.clone().requires_grad_(True)
        h = xs
        for m in layers:
            # some work between the MoE layers, so that there is a gap to fill
            h = torch.tanh(h @ torch.eye(M, device="cuda", dtype=dtype))
            h = m(h, capacity_factor=1.25, time_it=UniScheduler.time_it(),
                  prefetch=UniScheduler.prefetch_it())
        h.float().sum().backward()
        torch.cuda.synchronize()
        UniScheduler.profile_prefetch("")
        outs.append(h.detach().float().cpu())
    assert sched.ftime is not None and sched.ftime > 0
    assert len(sched.fwd_stat) == 2 and len(sched.bwd_stat) == 2
    assert len(sched.fwd_pf) == 2 and sched.fwd_pf[0] == 0          # first layer's is switched off
    assert layers[1].local_prefetch_fwd_count >= 1                  # a gap of any length hides >= 1 fetch
    assert all(0 <= m.local_prefetch_bwd_count <= E for m in layers)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])                              # prefetching changes no result
    _fresh()
