"""``MOLEMixedAdam``: one Adam over three parameter populations (interface of
MOLE/optim/mixed_optim.py:155-343).

  GPU-resident experts and the gate   ``torch.optim.Adam`` / ``AdamW`` on the device
  offloaded experts                   ``CPUAdam`` on the pinned host arrays, or -- with
                                      ``adv_adam`` -- the fused GPU step that ``MOLECore``
                                      runs right behind each expert batch's backward; then
                                      ``CPUAdam.step`` only advances the step counters

The reference's ``CPUAdam`` calls DeepSpeed's AVX kernel (MOLE/optim/mixed_optim.py:18-27, a
dependency that is not part of its tree); this one is the same update written with PyTorch's CPU
tensor ops, in place, with the arithmetic of ``_MOLECore::adam`` (MOLE/cpp/define.hpp:543-579) so
that a hybrid run (some experts stepped on the GPU, the rest here) applies one formula.
"""
from __future__ import annotations

from copy import deepcopy

import torch


class CPUAdam(torch.optim.Optimizer):
    """Adam over offloaded expert tensors.  Each parameter is a pinned host tensor
    ``[count, ...]`` carrying ``grad_``, ``momentum`` and ``variance`` twins
    (``CPUHostBatchedParameter``, MOLE/utils/Uparam.py:145-193)."""
    optimizer_id = 0

    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0, adamw_mode=True):
        default = {"lr": lr, "bias_correction": bias_correction, "betas": betas, "eps": eps,
                   "weight_decay": weight_decay, "adamw_mode": adamw_mode}
        super().__init__(params, default)
        self.opt_id = CPUAdam.optimizer_id
        CPUAdam.optimizer_id += 1
        self.adv_adam = False
        self.hybrid_adam = False
        self.hybrid_adam_count = 0

    def _state_of(self, p):
        state = self.state[p]
        if len(state) == 0:
            state["step"] = 0
            state["exp_avg"] = p.momentum
            state["exp_avg_sq"] = p.variance
        return state

    @torch.no_grad()
    def zero_grad(self):
        # gradients are overwritten by the next backward's device-to-host store: mark, don't fill
        for group in self.param_groups:
            for p in group["params"]:
                if getattr(p, "grad_", None) is not None:
                    p.grad_.lazy_zero = True

    @torch.no_grad()
    def adam_setting(self, moes, adamW, hybrid_adam_count, hybrid_adam):
        """Hands the hyper-parameters to every layer's core for the GPU step
        (MOLE/optim/mixed_optim.py:76-101)."""
        self.hybrid_adam_count = hybrid_adam_count
        self.hybrid_adam = hybrid_adam
        self.adv_adam = True
        beta1 = beta2 = lr = eps = wd = None
        step = 0
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                if getattr(p, "grad_", None) is None:
                    continue
                step = self._state_of(p)["step"]
        for moe in moes:
            moe.MOLECore.set_adam(beta1, beta2, step, lr, wd, eps, adamW, hybrid_adam_count)

    @torch.no_grad()
    def step(self, closure=None, groups=None, scale=1.0):
        all_on_gpu = self.adv_adam and (not self.hybrid_adam or self.hybrid_adam_count == -1)
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                if getattr(p, "grad_", None) is None:
                    continue
                state = self._state_of(p)
                state["step"] += 1
                if all_on_gpu:
                    continue            # the GPU step has already updated p, momentum, variance
                first = self.hybrid_adam_count if self.adv_adam else 0
                if first >= p.shape[0]:
                    continue
                t = state["step"]
                pv, g = p.data[first:], p.grad_[first:]
                m, v = state["exp_avg"][first:], state["exp_avg_sq"][first:]
                # fp32 arithmetic whatever the storage type
                pf, gf, mf, vf = pv.float(), g.float(), m.float(), v.float()
                if group["adamw_mode"]:
                    pf.mul_(1 - wd * lr)
                else:
                    gf = gf + wd * pf
                mf.mul_(beta1).add_(gf, alpha=1 - beta1)
                vf.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
                c1 = 1 - beta1 ** t if group["bias_correction"] else 1.0
                c2 = 1 - beta2 ** t if group["bias_correction"] else 1.0
                pf.addcdiv_(mf / c1, (vf / c2).sqrt_().add_(eps), value=-lr)
                pv.copy_(pf)
                m.copy_(mf)
                v.copy_(vf)


class MOLEMixedAdam:
    def __init__(self, CPUParams, GPUParams, GateParams, lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0, adamW=False):
        self.GateParams = GateParams
        self.CPUParams = CPUParams
        self.GPUParams = GPUParams
        self.hasCPU = len(CPUParams) > 0 and CPUParams[0] is not None
        self.hasGPU = len(GPUParams) > 0
        self.hasGate = len(GateParams) > 0
        dev_cls = torch.optim.AdamW if adamW else torch.optim.Adam
        kw = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        if self.hasCPU:
            self.cpu_optimizer = CPUAdam(CPUParams, bias_correction=True, adamw_mode=adamW, **kw)
        if self.hasGPU:
            self.gpu_optimizer = dev_cls(params=GPUParams, **kw)
        if self.hasGate:
            self.gate_optimizer = dev_cls(params=GateParams, **kw)

    # ---- checkpoint state (MOLE/optim/mixed_optim.py:205-277) -----------------------------------
    @torch.no_grad()
    def get_optim_state(self):
        """``[expert_state, gate_state]``: per parameter kind the moments of the GPU-resident
        experts followed by those of the offloaded ones (dimension 0), all on the host."""
        def host(opt):
            st = deepcopy(opt.state_dict()["state"])
            for k in st:
                st[k]["exp_avg"] = st[k]["exp_avg"].cpu()
                st[k]["exp_avg_sq"] = st[k]["exp_avg_sq"].cpu()
            return st
        gate_state = host(self.gate_optimizer) if self.hasGate else None
        gpu_state = host(self.gpu_optimizer) if self.hasGPU else None
        cpu_state = host(self.cpu_optimizer) if self.hasCPU else None
        if self.hasGPU and self.hasCPU:
            assert sorted(cpu_state.keys()) == sorted(gpu_state.keys()), "four parameter kinds each"
            expert_state = gpu_state
            for k in expert_state:
                for name in ("exp_avg", "exp_avg_sq"):
                    expert_state[k][name] = torch.cat([gpu_state[k][name], cpu_state[k][name]], dim=0)
        else:
            expert_state = gpu_state if self.hasGPU else cpu_state
        return [expert_state, gate_state]

    @torch.no_grad()
    def set_optim_state(self, states):
        """Inverse of ``get_optim_state``.  The device optimizers' state is loaded through
        ``load_state_dict`` (which creates the moment tensors on the parameters' device), so no
        step has to be taken to "build" it as the reference does (mixed_optim.py:207-208) -- a
        step without gradients would not build anything."""
        expert_state, gate_state = states

        def load(opt, saved, take):
            sd = opt.state_dict()
            sd["state"] = {k: {"step": torch.as_tensor(saved[k]["step"], dtype=torch.float32).clone(),
                               "exp_avg": take(k, saved[k]["exp_avg"]).clone(),
                               "exp_avg_sq": take(k, saved[k]["exp_avg_sq"]).clone()}
                           for k in range(sum(len(g["params"]) for g in sd["param_groups"]))}
            opt.load_state_dict(sd)

        if self.hasGate:
            load(self.gate_optimizer, gate_state, lambda k, t: t)
        if self.hasGPU:
            counts = [p.shape[0] for p in self.GPUParams]
            load(self.gpu_optimizer, expert_state, lambda k, t: t[:counts[k]])
        if self.hasCPU:
            for k, p in enumerate(self.cpu_optimizer.param_groups[0]["params"]):
                st = self.cpu_optimizer._state_of(p)
                n = st["exp_avg"].shape[0]
                st["exp_avg"].copy_(expert_state[k]["exp_avg"][-n:])
                st["exp_avg_sq"].copy_(expert_state[k]["exp_avg_sq"][-n:])
                s = expert_state[k]["step"]
                st["step"] = int(s.item()) if torch.is_tensor(s) else int(s)

    # ---- the usual optimizer surface --------------------------------------------------------------
    @torch.no_grad()
    def zero_grad(self):
        # set_to_none=False: the GPU-resident experts' gradient tensors are the buffers the expert
        # pipeline writes (and, with acc_step > 1, adds) into; they must stay where they are
        if self.hasGate:
            self.gate_optimizer.zero_grad()
        if self.hasGPU:
            self.gpu_optimizer.zero_grad(set_to_none=False)
        if self.hasCPU:
            self.cpu_optimizer.zero_grad()

    def _optimizers(self):
        return [o for has, o in ((self.hasGPU, getattr(self, "gpu_optimizer", None)),
                                 (self.hasCPU, getattr(self, "cpu_optimizer", None)),
                                 (self.hasGate, getattr(self, "gate_optimizer", None))) if has]

    def get_lr(self):
        return [group["lr"] for o in self._optimizers() for group in o.param_groups]

    def set_lr(self, lr):
        value = lr[0] if isinstance(lr, list) else lr
        for o in self._optimizers():
            for group in o.param_groups:
                group["lr"] = value

    @torch.no_grad()
    def step(self, CPU_step=True, GPU_step=True, Gate_step=True, AllreduceGate=True):
        if self.hasGate and Gate_step:
            self.gate_optimizer.step()
            # data-parallel ranks route with the same gate: average it after the step
            # (MOLE/optim/mixed_optim.py:326-329)
            if AllreduceGate and torch.distributed.is_available() and torch.distributed.is_initialized() \
                    and torch.distributed.get_world_size() > 1:
                for p in self.GateParams:
                    torch.distributed.all_reduce(p, op=torch.distributed.ReduceOp.AVG)
        if self.hasGPU and GPU_step:
            self.gpu_optimizer.step()
        if self.hasCPU and CPU_step:
            self.cpu_optimizer.step()
