"""``MOLEModule``: the MoE FFN layer with GPU-resident ("static") and host-offloaded ("dynamic")
experts, with the constructor, ``forward`` signature, attributes and helper methods of
MOLE/moe/layer.py:18-500 so that it drops into code written against the reference.

What runs underneath is this package's CUDA library: fused gate + routing-index build,
vectorised dispatch / combine, the grouped tcgen05 expert GEMMs (CUDA-core fp32 GEMMs for
fp32), the NCCL expert-parallel exchange and the stream-ordered host-to-device expert fetch.

Keyword-only additions (defaults reproduce the reference): ``dtype`` (the reference hard-wires
float32, MOLE/moe/layer.py:43,89-96), ``normalize_gate``, ``gelu_bwd`` ("exact" or the
reference kernel's "tanh" derivative, MOLE/cpp/gelu.cu:3-14) and ``ffn_backend`` (1 runs the
bf16 FFN on the CUDA-core kernels, for bisecting numerics).
"""
from __future__ import annotations

import time

import torch

from .. import core, ops
from ..core import MOLECore
from ..utils import Ugate
from ..utils.Uact import build_activation_fwd
from ..utils.Udist import MOLEDist
from ..utils.Uparam import CPUHostBatchedParameter, GPUHostBatchedParameter, UnifiedCPUTensor
from ..utils.Utimer import UATimer
from .functions import BatchFusedFWD, Combine, Dispatch, GateRoute, pfetchbwd


class MOLEModule(torch.nn.Module):
    _instance = []
    _fwdgaps = []
    _bwdgaps = []
    _forwarding_count = None
    _backwarding_count = None
    _cpu_optimizer = None
    use_prefetch = True
    _moe_scale = 1.0
    step = 0

    def __init__(self, total_d_experts, total_s_experts, embed_dim, ffn_dim, pool_size, topk,
                 ebatch_size, dist, act, acc_step, adv_adam, use_pool,
                 pool_for_extra=[False, False, False], overlap=True, gate_control_by_umoe=True,
                 hybrid_adam=False, device_s_experts=-1, *, dtype=torch.float32,
                 normalize_gate=False, gelu_bwd="exact", ffn_backend=0, fuse_combine=None):
        super().__init__()
        self.acc_step = acc_step
        self.topk = topk
        self.dtype = dtype
        self.normalize_gate = normalize_gate
        # True: the gate-weighted combine runs inside the second GEMM's epilogue (one rank, bf16,
        # top-1 / top-2; an error where that is not possible).  None / False: the separate combine
        # kernel -- measured equally fast on the benchmark shape, and it sums a token's rows in
        # fp32 before the one rounding, as the reference's decode does.
        self.fuse_combine = fuse_combine

        self.local_rank = dist["local_rank"]
        self.world_size = dist["world_size"]
        self.rank = dist["rank"]
        self.device = torch.device(f"cuda:{self.local_rank}")
        MOLEDist(local_rank=self.local_rank)      # the expert-parallel communicator (singleton)

        assert total_d_experts % self.world_size == 0
        assert total_s_experts % self.world_size == 0
        assert isinstance(act, str)
        use_pool = use_pool if pool_size != -1 else False
        # expert parallelism equals data parallelism: every rank owns E / W experts
        self.d_experts = total_d_experts // self.world_size
        self.s_experts = total_s_experts // self.world_size
        self.total_experts = total_d_experts + total_s_experts
        if self.d_experts > 0 and not use_pool:
            raise ValueError("offloaded experts need the slot pool (pool_size >= 1, use_pool=True)")

        if self.d_experts > 0:
            core.create_UniMem(self.local_rank, pool_size, dtype,
                               [[ffn_dim, embed_dim], [ffn_dim], [ffn_dim, embed_dim], [embed_dim]])
        self.MOLECore = MOLECore(use_pool, pool_for_extra[0], pool_for_extra[1], pool_for_extra[2],
                                 self.s_experts, self.d_experts, ebatch_size, self.world_size, act,
                                 adv_adam, acc_step, 0, self.local_rank, len(MOLEModule._instance),
                                 self.total_experts, dtype=dtype, gelu_bwd=gelu_bwd,
                                 ffn_backend=ffn_backend)
        self.pool_size = pool_size
        self.use_pool = use_pool
        self.ebatch_size = ebatch_size
        self.embed_dim = embed_dim
        self.ffn_dim = ffn_dim

        # the gate is a plain list entry unless the caller wants torch to own it
        self.gate = [Ugate.MOLETopk(embed_dim, self.total_experts)]
        if not gate_control_by_umoe:
            self.gate = torch.nn.ModuleList(self.gate)
        self.gate[0].linear = self.gate[0].linear.to(device=self.device, dtype=dtype)

        # zero-size parameter that keeps the expert pipeline's backward reachable when the
        # layer input does not require grad
        self.dummy_param = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=dtype))
        self.capacity_on = True
        self.act_str = act
        self.act = build_activation_fwd(act)

        gpu = dict(count=self.s_experts, dtype=dtype, device=self.device, moe=self.MOLECore)
        self.FC1_W_GPU = GPUHostBatchedParameter(size=[ffn_dim, embed_dim], p_id=0, **gpu)
        self.FC1_B_GPU = GPUHostBatchedParameter(size=[ffn_dim], bias=True, p_id=1, fan_in=embed_dim, **gpu)
        self.FC2_W_GPU = GPUHostBatchedParameter(size=[ffn_dim, embed_dim], p_id=2, transposed=True, **gpu)
        self.FC2_B_GPU = GPUHostBatchedParameter(size=[embed_dim], bias=True, p_id=3, fan_in=ffn_dim, **gpu)

        UnifiedCPUTensor()
        UnifiedCPUTensor.init([[ffn_dim, embed_dim], [ffn_dim], [ffn_dim, embed_dim], [embed_dim]],
                              device_s_experts, dtype)
        cpu = dict(count=self.d_experts, dtype=dtype, moe=self.MOLECore,
                   device_s_experts=device_s_experts)
        self.FC1_W_CPU = CPUHostBatchedParameter(size=[ffn_dim, embed_dim], p_id=0, **cpu)
        self.FC1_B_CPU = CPUHostBatchedParameter(size=[ffn_dim], p_id=1, bias=True, fan_in=embed_dim, **cpu)
        self.FC2_W_CPU = CPUHostBatchedParameter(size=[ffn_dim, embed_dim], p_id=2, transposed=True, **cpu)
        self.FC2_B_CPU = CPUHostBatchedParameter(size=[embed_dim], p_id=3, bias=True, fan_in=ffn_dim, **cpu)

        self.overlap = overlap
        self.adv_adam = adv_adam
        self.hybrid_adam = hybrid_adam
        self.hybrid_adam_count = 0
        self.use_prefetch = False
        self.local_prefetch_fwd_count = 0
        self.local_prefetch_bwd_count = 0
        self.global_prefetch_fwd_count = 0
        self.global_prefetch_bwd_count = 0
        self.global_prefetch = False
        self.grad_use_pool, self.mome_use_pool, self.vari_use_pool = pool_for_extra
        self.timer = UATimer()
        self.l_aux = None
        self._route_counts = None
        self.last_plan = None
        # A dict here makes every step leave references to the expert pipeline's output rows
        # ("rows", [E, Cs, M], what combine reads) and to the gradient rows that come back from it
        # ("dx_rows"), so that a checker can compare them with a reference after the step.
        self.parity_tap = None

        self.moe_id = len(MOLEModule._instance)
        MOLEModule._instance.append(self)
        if hybrid_adam:
            for ins in MOLEModule._instance:
                assert self.d_experts == ins.d_experts, "Mixed Adam only support all moes have same experts"

    # ---- prefetch hooks (MOLE/moe/layer.py:138-180) -------------------------------------------
    def set_hybrid_adam_count(self, hybrid_adam_count):
        self.hybrid_adam_count = hybrid_adam_count

    def dummy_fetch(self, batch_size):
        torch.cuda.synchronize()
        t0 = time.time()
        if self.pool_size >= 1 and self.d_experts > 0:
            self.MOLECore.dummy_fetch(min(self.d_experts, batch_size))
        torch.cuda.synchronize()
        return time.time() - t0

    def global_prefetch_fwd(self):
        for moe_id, n in self.global_prefetch_fwd_count:
            MOLEModule._instance[moe_id].MOLECore.prefetch_fwd(n)

    def global_prefetch_bwd(self):
        for moe_id, n in self.global_prefetch_bwd_count:
            MOLEModule._instance[moe_id].MOLECore.prefetch_bwd(n)

    def local_prefetch_fwd(self):
        self.MOLECore.prefetch_fwd(self.local_prefetch_fwd_count)

    def local_prefetch_bwd(self):
        self.MOLECore.prefetch_bwd(self.local_prefetch_bwd_count)

    def prefetch_fwd(self, batch_size):
        self.MOLECore.prefetch_fwd(batch_size)

    def prefetch_bwd(self, batch_size):
        self.MOLECore.prefetch_bwd(batch_size)

    def set_prefetch(self, fwd_prefetch_num, bwd_prefetch_num):
        self.fwd_prefetch_num = fwd_prefetch_num
        self.bwd_prefetch_num = bwd_prefetch_num
        self.actual_prefetch_num = max(fwd_prefetch_num, bwd_prefetch_num)
        self.use_prefetch = True
        self.prefetched_fwd = 0
        self.prefetched_bwd = 0

    def unset_lazy_zero(self):
        for p in (self.FC1_W_CPU, self.FC1_B_CPU, self.FC2_W_CPU, self.FC2_B_CPU):
            p.unset_lazy_zero()

    # ---- state (MOLE/moe/layer.py:349-427) ------------------------------------------------------
    def _expert_containers(self):
        gpu = (self.FC1_W_GPU, self.FC1_B_GPU, self.FC2_W_GPU, self.FC2_B_GPU)
        cpu = (self.FC1_W_CPU, self.FC1_B_CPU, self.FC2_W_CPU, self.FC2_B_CPU)
        return [(gpu, i) for i in range(self.s_experts)] + [(cpu, i) for i in range(self.d_experts)]

    @torch.no_grad()
    def set_layer_state(self, states, grad):
        gate_state = states["gate"]
        self.gate[0].linear.weight.copy_(gate_state[0])
        if self.gate[0].linear.bias is not None:
            self.gate[0].linear.bias.copy_(gate_state[1])
        for j, (kinds, i) in enumerate(self._expert_containers()):
            for p, src in zip(kinds, states["experts"][j]):
                p.fetch_single(i).copy_(src)
        if grad:
            grad_state = states["grad"]
            j = 0
            for j, (kinds, i) in enumerate(self._expert_containers()):
                for p, src in zip(kinds, grad_state[j]):
                    p.fetch_single_grad(i).copy_(src)
            j = self.s_experts + self.d_experts
            self.gate[0].linear.weight.grad = grad_state[j].to(self.gate[0].linear.weight.device)
            if self.gate[0].linear.bias is not None:
                self.gate[0].linear.bias.grad = grad_state[j + 1].to(self.gate[0].linear.bias.device)

    @torch.no_grad()
    def get_layer_state(self, grad):
        lin = self.gate[0].linear
        state = {"gate": [lin.weight.cpu(), lin.bias.cpu() if lin.bias is not None else None]}
        state["experts"] = [[p.fetch_single(i).cpu() for p in kinds]
                            for kinds, i in self._expert_containers()]
        grads = []
        if grad:
            grads = [[p.fetch_single_grad(i).cpu() for p in kinds]
                     for kinds, i in self._expert_containers()]
            grads.append(lin.weight.grad.cpu())
            grads.append(lin.bias.grad.cpu() if lin.bias is not None else None)
        state["grad"] = grads
        return state

    # ---- forward (MOLE/moe/layer.py:429-476) ----------------------------------------------------
    def forward(self, input_, adam_param={"beta1": 0.9, "beta2": 0.999, "lr": 0.001, "t": 100,
                                          "lam": 1, "eps": 1e-8},
                capacity_factor=1.0, time_it=False, prefetch=False):
        original_shape = input_.shape
        original_dtype = input_.dtype
        if prefetch:
            input_ = pfetchbwd.apply(input_, self)

        resized_input = input_.reshape(-1, self.embed_dim)
        if resized_input.dtype != self.dtype:
            resized_input = resized_input.to(self.dtype)
        resized_input = resized_input.contiguous()

        gate = self.gate[0]
        T = resized_input.shape[0]
        cap = ops.capacity(T, self.total_experts, self.topk, capacity_factor)
        holder = {}
        gates, l_aux = GateRoute.apply(resized_input, gate.linear.weight,
                                       getattr(gate, "logit_bias", None), self.topk, cap,
                                       self.normalize_gate, holder)
        plan = holder["plan"]
        self.l_aux = l_aux
        self.last_plan = plan
        # when x needs a gradient the gate's backward will run after the dispatch's and can fuse
        # the two contributions to dx
        holder["gate_needs_x_grad"] = bool(resized_input.requires_grad and torch.is_grad_enabled())
        # several ranks of one node: rows are stored straight into the consuming rank's memory
        # (dispatch -> owners, FC2 -> sources, and the mirror in backward) instead of all-to-alls
        peer = self.MOLECore.peer_for(plan.Cs, self.embed_dim, self.dtype, resized_input.device)
        holder["peer"] = peer
        holder["tap"] = self.parity_tap
        dispatched_input = Dispatch.apply(resized_input, plan, holder)

        self._route_counts = plan.counts
        self._peer_exchange = peer
        # the combine as part of the second GEMM's epilogue where that is possible
        can_fuse = peer is None and self.MOLECore.can_fuse_combine(plan, self.embed_dim)
        if self.fuse_combine and not can_fuse:
            raise RuntimeError("fuse_combine=True needs one rank, bf16, top-1/top-2 and the default FFN backend")
        fuse = {"plan": plan, "gates": gates} if (can_fuse and self.fuse_combine) else None
        self._fuse = fuse
        experts_output = BatchFusedFWD.apply(dispatched_input, self, self.dummy_param, time_it, prefetch)
        self._route_counts = None
        self._peer_exchange = None
        self._fuse = None
        if self.parity_tap is not None:
            self.parity_tap["rows"] = experts_output

        expert_output = Combine.apply(experts_output, gates, plan, peer,
                                      fuse["y"] if fuse is not None else None)
        out = expert_output.reshape(original_shape).to(original_dtype)

        if prefetch:
            last = len(MOLEModule._instance) - 1
            if self.moe_id < last:
                nxt = MOLEModule._instance[self.moe_id + 1]
                if self.global_prefetch:
                    nxt.global_prefetch_fwd()
                nxt.local_prefetch_fwd()
            elif self.moe_id == last:
                if self.global_prefetch:
                    MOLEModule._instance[-1].global_prefetch_bwd()
                MOLEModule._instance[-1].local_prefetch_bwd()
        return out

    # ---- parameter accessors (MOLE/moe/layer.py:478-500) -----------------------------------------
    def d_experts_param(self):
        if self.d_experts == 0:
            return []
        return [p.all_tensors for p in (self.FC1_W_CPU, self.FC1_B_CPU, self.FC2_W_CPU, self.FC2_B_CPU)]

    def s_experts_param(self):
        if self.s_experts == 0:
            return []
        return [p.fetch_all_with_grad()
                for p in (self.FC1_W_GPU, self.FC1_B_GPU, self.FC2_W_GPU, self.FC2_B_GPU)]

    def gate_param(self):
        lin = self.gate[0].linear
        return [lin.weight] if lin.bias is None else [lin.weight, lin.bias]
