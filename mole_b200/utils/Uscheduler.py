"""``UniScheduler``: the per-process policy object above the MoE layers (interface of
MOLE/utils/Uscheduler.py).

It owns what spans layers: the step counter, the profiling of the first steps (how long the
model runs between consecutive MoE layers, how long one expert takes to fetch), the prefetch
counts derived from that ratio (Uscheduler.py:228-343) -- per layer ("local") or, with
``global_prefetch``, spread over the pool by ``fast_assign_prefetch`` (MOLE/cpp/core.cpp:1302-1345)
so that a layer with time to spare fetches for later ones -- the optimizer factory
(Uscheduler.py:94-130) and the checkpoint file (Uscheduler.py:66-92).

A training loop uses it as the reference's does::

    UniScheduler(local_rank=0, disable_overlap=False, adv_adam=False, gate_control_by_MOLE=True)
    layers = [MOLEModule(...), ...]
    UniScheduler.schedule_policy(profile_step=6, prefetch_on=True)
    opt = UniScheduler.build_optimizer(lr=1e-3)
    for step in range(n):
        UniScheduler.set_step(step)
        UniScheduler.prefetch_fwd()
        loss = model(batch, time_it=UniScheduler.time_it(), prefetch=UniScheduler.prefetch_it())
        loss.backward()
        UniScheduler.profile_prefetch("")
        opt.step(); opt.zero_grad(); UniScheduler.zero_grad()
"""
from __future__ import annotations

import ast
import math

import torch

from .. import core as MOLE_util
from ..moe import layer as MOLE
from ..optim import mixed_optim
from . import Udist, Ustream, Utimer
from .Uparam import UnifiedCPUTensor


class UniScheduler:
    _instance = None
    _optimizer = None

    def __new__(cls, *args, **kw):
        if cls._instance is None:
            inst = object.__new__(cls)
            local_rank = kw.get("local_rank", 0)
            if torch.cuda.is_available():
                Ustream.ExpertStreamCtx(device=f"cuda:{local_rank}",
                                        disable=kw.get("disable_overlap", False), set_current=False)
                Udist.MOLEDist(local_rank=local_rank)
            inst.device = f"cuda:{local_rank}"
            inst.adv_adam = kw.get("adv_adam", False)
            inst.hybrid_adam = kw.get("hybrid_adam", False)
            if inst.hybrid_adam:
                inst.adv_adam = True
                inst.hybrid_adam_extra = []
            inst.hybrid_adam_count = -1 if inst.adv_adam else 0
            inst.gate_control_by_MOLE = kw.get("gate_control_by_MOLE", True)
            inst.ftime = None
            inst.fwd_stat = None
            inst.bwd_stat = None
            inst.cur_step = -1
            inst.prefetch_on = False
            inst.profile_step = -1
            inst.global_prefetch = False
            inst.deactivate_first_prefetch = True
            inst.schedule_hybrid = False
            inst.prefetch_floor = False
            inst.adamW = False
            inst.fwd_pf, inst.bwd_pf = [], []
            inst.device_s_experts = kw.get("device_s_experts", -1)
            assert not inst.hybrid_adam or inst.device_s_experts == -1, \
                "hybrid Adam and one contiguous host block cannot be combined"
            cls._instance = inst
        return cls._instance

    def __init__(self, *args, **kw):
        pass

    @staticmethod
    def schedule_policy(profile_step, prefetch_on, deactivate_first_prefetch=True, prefetch_floor=False,
                        global_prefetch=False, schedule_hybrid=False):
        inst = UniScheduler._instance
        inst.profile_step = profile_step
        inst.prefetch_on = prefetch_on
        inst.deactivate_first_prefetch = deactivate_first_prefetch
        inst.global_prefetch = global_prefetch
        inst.schedule_hybrid = schedule_hybrid
        inst.prefetch_floor = prefetch_floor

    # ---- checkpoint (MOLE/utils/Uscheduler.py:66-92) ----------------------------------------------
    @staticmethod
    def save_states(state_file="MOLE_states", grad=False):
        """``[[layer state, ...], [expert optimizer state, gate optimizer state]]`` in
        ``<state_file>.pt``; a layer state is ``{gate, experts, grad}`` with the GPU-resident
        experts first (``MOLEModule.get_layer_state``)."""
        model_state = [inst.get_layer_state(grad) for inst in MOLE.MOLEModule._instance]
        optim_state = UniScheduler._optimizer.get_optim_state()
        torch.save([model_state, optim_state], state_file + ".pt")

    @staticmethod
    def load_states(state_file="MOLE_states", grad=False):
        model_state, optim_state = torch.load(state_file + ".pt", weights_only=False)
        # parameters (and gradients) first, then the optimizer -- whose restore takes one step to
        # build its state tensors -- then the parameters again to undo that step
        for i, inst in enumerate(MOLE.MOLEModule._instance):
            inst.set_layer_state(model_state[i], grad)
        UniScheduler._optimizer.set_optim_state(optim_state)
        for i, inst in enumerate(MOLE.MOLEModule._instance):
            inst.set_layer_state(model_state[i], grad)

    # ---- optimizer (MOLE/utils/Uscheduler.py:94-153) ----------------------------------------------
    @staticmethod
    def build_optimizer(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, gate_only=False,
                        adamW=False):
        sched = UniScheduler._instance
        sched.adamW = adamW
        cpu_params, gpu_params, gate_params = [], [], []
        for inst in MOLE.MOLEModule._instance:
            if not gate_only:
                if sched.device_s_experts == -1:
                    cpu_params += inst.d_experts_param()
                gpu_params += inst.s_experts_param()
            if gate_only or sched.gate_control_by_MOLE:
                gate_params += inst.gate_param()
        if not gate_only and sched.device_s_experts != -1:
            cpu_params += UnifiedCPUTensor.get_cpu_experts()
        if cpu_params or gpu_params or gate_params:
            UniScheduler._optimizer = mixed_optim.MOLEMixedAdam(
                cpu_params, gpu_params, gate_params, lr, betas, eps, weight_decay, adamW)
        else:
            UniScheduler._optimizer = None
            return None
        if UniScheduler._optimizer.hasCPU:
            MOLE.MOLEModule._cpu_optimizer = UniScheduler._optimizer.cpu_optimizer
        UniScheduler.adam_set()
        return UniScheduler._optimizer

    @staticmethod
    def clear():
        MOLE_util.clear_virtual_mem()

    @staticmethod
    def set_hybrid(hybrid_adam_count):
        if UniScheduler._instance.hybrid_adam:
            UniScheduler._instance.hybrid_adam_count = hybrid_adam_count

    @staticmethod
    def adam_set():
        """Hyper-parameters and step count to the layers' cores for the GPU Adam step; call it
        once per optimizer step when ``adv_adam`` is on (the step count enters the bias
        correction)."""
        sched, opt = UniScheduler._instance, UniScheduler._optimizer
        if opt is not None and opt.hasCPU and sched.adv_adam:
            MOLE.MOLEModule._cpu_optimizer.adam_setting(
                MOLE.MOLEModule._instance, sched.adamW, sched.hybrid_adam_count, sched.hybrid_adam)

    @staticmethod
    def zero_grad():
        opt = UniScheduler._optimizer
        if opt is not None and opt.hasCPU:
            for inst in MOLE.MOLEModule._instance:
                inst.MOLECore.set_lazy_zero()

    # ---- step bookkeeping and profiling ----------------------------------------------------------
    @staticmethod
    def clear_timer():
        Utimer.UATimer.clear()

    @staticmethod
    def track_fwd_start():
        Utimer.UATimer.track_fwd_start()

    @staticmethod
    def set_step(cur_step):
        """At the beginning of every step."""
        UniScheduler._instance.cur_step = cur_step
        if UniScheduler.time_it():
            UniScheduler.clear_timer()
            UniScheduler.track_fwd_start()
        UniScheduler.clear()

    @staticmethod
    def time_it():
        return UniScheduler._instance.cur_step < UniScheduler._instance.profile_step

    @staticmethod
    def prefetch_it():
        inst = UniScheduler._instance
        return inst.cur_step > inst.profile_step and inst.prefetch_on

    @staticmethod
    def dummy_fetch():
        return [m.dummy_fetch(1) for m in MOLE.MOLEModule._instance]

    @staticmethod
    def attach_step_time(step_time, cur_step):
        inst = UniScheduler._instance
        if inst.schedule_hybrid and 0 <= cur_step - 10 <= MOLE.MOLEModule._instance[0].d_experts:
            inst.hybrid_adam_extra.append(step_time)

    @staticmethod
    def schedule_hybrid_adam(cur_step):
        """Search for the split between GPU-stepped and host-stepped experts: steps 10 .. 10 + d
        try every count in turn, the fastest one is kept (MOLE/utils/Uscheduler.py:199-225)."""
        inst = UniScheduler._instance
        if not inst.schedule_hybrid:
            return
        d = MOLE.MOLEModule._instance[0].d_experts
        if 0 <= cur_step - 10 <= d:
            UniScheduler.set_hybrid(cur_step - 10)
        if cur_step == d + 11:
            times = []
            for entry in inst.hybrid_adam_extra:
                t = entry[0] if isinstance(entry, (list, tuple)) else entry
                if Udist.MOLEDist.get_MOLE_world_size() > 1:
                    tt = torch.tensor(float(t), device=inst.device)
                    torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.AVG)
                    t = tt.item()
                times.append(t)
            best = min(range(len(times)), key=times.__getitem__) if times else 0
            UniScheduler.set_hybrid(best)

    @staticmethod
    def profile_prefetch(force_prefetch_scheme=""):
        """During the profiling steps: running averages of the gaps in front of every MoE layer
        (forward and backward) and of one expert's fetch time, then the prefetch counts."""
        inst = UniScheduler._instance
        if not UniScheduler.time_it() or inst.cur_step < 2:
            return

        def running(old, new):
            if old is None:
                return new
            return [(a + b) / 2 for a, b in zip(old, new)]

        fetch_time = UniScheduler.dummy_fetch()
        ftime = sum(fetch_time) / max(len(fetch_time), 1)
        inst.ftime = ftime if inst.ftime is None else (inst.ftime + ftime) / 2
        fwd_stat, bwd_stat = Utimer.UATimer.stats()
        if len(fwd_stat) > 0:
            inst.fwd_stat = running(inst.fwd_stat, list(fwd_stat))
        if len(bwd_stat) > 0:
            inst.bwd_stat = running(inst.bwd_stat, list(bwd_stat))
        if inst.prefetch_on and inst.fwd_stat is not None and inst.bwd_stat is not None:
            UniScheduler.set_prefetch_scheme(force_prefetch_scheme)

    @staticmethod
    def set_prefetch_scheme(force_prefetch_scheme=""):
        """Experts each layer can fetch while the model runs up to it = gap / fetch time of one
        expert (ceil, or floor with ``prefetch_floor``); ranks agree on the minimum.  Local
        scheme: every layer prefetches for itself.  Global scheme: ``fast_assign_prefetch`` lets
        layers with spare time fetch for later layers into spare pool slots."""
        inst = UniScheduler._instance
        layers = MOLE.MOLEModule._instance
        n = len(layers)
        rnd = math.floor if inst.prefetch_floor else math.ceil
        ftime = max(inst.ftime or 0.0, 1e-9)
        inst.fwd_pf = [int(rnd(f / ftime)) for f in inst.fwd_stat]
        inst.bwd_pf = [int(rnd(b / ftime)) for b in inst.bwd_stat]
        if force_prefetch_scheme != "":      # e.g. "[[1,1,1,1],[1,1,1,1]]": forward counts, backward counts
            scheme = (ast.literal_eval(force_prefetch_scheme)
                      if isinstance(force_prefetch_scheme, str) else force_prefetch_scheme)
            inst.global_prefetch = False
            inst.fwd_pf, inst.bwd_pf = list(scheme[0]), list(scheme[1])
        inst.fwd_pf = (inst.fwd_pf + [0] * n)[:n]
        inst.bwd_pf = (inst.bwd_pf + [0] * n)[:n]
        if inst.deactivate_first_prefetch and n > 0:
            inst.fwd_pf[0] = 0
        inst.E = [m.d_experts for m in layers]
        inst.revE = inst.E[::-1]
        if Udist.MOLEDist.get_MOLE_world_size() > 1:
            for name in ("fwd_pf", "bwd_pf"):
                t = torch.tensor(getattr(inst, name), device=inst.device)
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
                setattr(inst, name, [int(v) for v in t.tolist()])
        pool_size = max(0, layers[0].pool_size) if n else 0
        if not inst.global_prefetch:
            for i, m in enumerate(layers):
                m.global_prefetch = False
                m.local_prefetch_fwd_count = min(inst.fwd_pf[i], m.d_experts, pool_size)
                m.local_prefetch_bwd_count = min(inst.bwd_pf[n - 1 - i], m.d_experts, pool_size)
        else:
            gp_fwd, lp_fwd = MOLE_util.fast_assign_prefetch(pool_size, inst.fwd_pf, inst.E)
            gp_bwd, lp_bwd = MOLE_util.fast_assign_prefetch(pool_size, inst.bwd_pf, inst.revE)
            for i, m in enumerate(layers):
                m.global_prefetch = True
                m.local_prefetch_fwd_count = lp_fwd[i]
                m.local_prefetch_bwd_count = lp_bwd[n - 1 - i]
                m.global_prefetch_fwd_count = sorted(gp_fwd[i], reverse=True)
                # backward runs the layers in reverse: positions of the backward sequence -> layer ids
                m.global_prefetch_bwd_count = sorted([[n - 1 - x[0], x[1]] for x in gp_bwd[n - 1 - i]])

    @staticmethod
    def prefetch_fwd():
        """Before the forward pass: the first MoE layer's prefetch (every other layer's is
        triggered by the layer in front of it, MOLE/moe/layer.py:464-472)."""
        if UniScheduler.prefetch_it():
            first = MOLE.MOLEModule._instance[0]
            if UniScheduler._instance.global_prefetch:
                first.global_prefetch_fwd()
            first.local_prefetch_fwd()

    @staticmethod
    def sync_tran():
        torch.cuda.synchronize()
        for ins in MOLE.MOLEModule._instance:
            ins.MOLECore.clear_tran_tmp()
