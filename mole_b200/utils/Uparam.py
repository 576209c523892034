"""Batched expert parameter containers (interface of MOLE/utils/Uparam.py).

``GPUHostBatchedParameter``  ``[count, *size]`` on the device with a dense gradient twin
                             (MOLE/utils/Uparam.py:337-405).
``CPUHostBatchedParameter``  ``[count, *size]`` in pinned host memory with ``grad_``,
                             ``momentum`` and ``variance`` twins (Uparam.py:145-305); these are
                             the offloaded experts the pool streams in.
``UnifiedCPUTensor``         one contiguous pinned block per kind carved into views
                             (Uparam.py:8-142), used when ``device_s_experts > 0``.

Initialisation follows the reference: weights ``kaiming_uniform_(a=sqrt(5))`` with
``fan_in`` mode, ``fan_out`` for the transposed FC2; biases ``U(+-1/sqrt(fan_in))``.
"""
from __future__ import annotations

import math

import torch


def _pinned_zeros(shape, dtype):
    return torch.zeros(shape, dtype=dtype, device="cpu", pin_memory=torch.cuda.is_available())


def _init_batched(t: torch.Tensor, count: int, bias: bool, fan_in: int, transposed: bool) -> None:
    # initialise in fp32 and cast, so bf16 storage does not change the distribution's support
    for i in range(count):
        tmp = torch.empty(t[i].shape, dtype=torch.float32, device=t.device)
        if bias:
            bound = 1 / math.sqrt(fan_in)
            torch.nn.init.uniform_(tmp, -bound, bound)
        else:
            torch.nn.init.kaiming_uniform_(tmp, a=math.sqrt(5),
                                           mode="fan_out" if transposed else "fan_in")
        t[i].copy_(tmp)


class UnifiedCPUTensor(object):
    """Singleton owning one pinned block each for parameters, grads, momentum and variance."""
    _instance = None

    def __new__(cls, *args, **kw):
        if cls._instance is None:
            inst = object.__new__(cls)
            inst.inited = False
            inst.blocks = {}
            inst.offset = {}
            cls._instance = inst
        return cls._instance

    def __init__(self, *args, **kw):
        pass

    @staticmethod
    def init(sizes, device_s_experts, dtype):
        inst = UnifiedCPUTensor._instance
        if inst.inited or device_s_experts <= 0:
            return
        per_expert = sum(math.prod(s) for s in sizes)
        inst.numel = per_expert * device_s_experts
        for kind in ("param", "grad", "momentum", "variance"):
            inst.blocks[kind] = _pinned_zeros(inst.numel, dtype)
            inst.offset[kind] = 0
        # the whole block is one optimizer parameter (Uparam.py:136-138)
        inst.blocks["param"].grad_ = inst.blocks["grad"]
        inst.blocks["param"].momentum = inst.blocks["momentum"]
        inst.blocks["param"].variance = inst.blocks["variance"]
        inst.blocks["grad"].lazy_zero = True
        inst.inited = True

    @staticmethod
    def get_cpu_experts():
        inst = UnifiedCPUTensor._instance
        return [inst.blocks["param"]] if inst is not None and inst.inited and inst.numel > 0 else []

    @staticmethod
    def _carve(kind, size, count):
        inst = UnifiedCPUTensor._instance
        n = count * math.prod(size)
        o = inst.offset[kind]
        if o + n > inst.numel:
            raise RuntimeError("UnifiedCPUTensor block exhausted")
        inst.offset[kind] = o + n
        return inst.blocks[kind][o:o + n].view(count, *size)

    @staticmethod
    def get_tensor(size, device_s_experts, count, dtype, p_id):
        return UnifiedCPUTensor._carve("param", size, count)

    @staticmethod
    def get_grad(size, device_s_experts, count, dtype, p_id):
        return UnifiedCPUTensor._carve("grad", size, count)

    @staticmethod
    def get_momentum(size, device_s_experts, count, dtype, p_id):
        return UnifiedCPUTensor._carve("momentum", size, count)

    @staticmethod
    def get_variance(size, device_s_experts, count, dtype, p_id):
        return UnifiedCPUTensor._carve("variance", size, count)


class CPUHostBatchedParameter(object):
    def __init__(self, size, count, dtype, moe, p_id, bias=False, fan_in=0, transposed=False,
                 device_s_experts=-1):
        self.count = count
        self.size = size
        self.dtype = dtype
        self.device = "cpu"
        self.p_id = p_id
        self.adam_state = True
        self.bias = bias
        self.moe = moe
        if count > 0:
            if device_s_experts == -1:
                self.all_tensors = _pinned_zeros((count, *size), dtype)
                grad = _pinned_zeros((count, *size), dtype)
                mome = _pinned_zeros((count, *size), dtype)
                vari = _pinned_zeros((count, *size), dtype)
            else:
                self.all_tensors = UnifiedCPUTensor.get_tensor(size, device_s_experts, count, dtype, p_id)
                grad = UnifiedCPUTensor.get_grad(size, device_s_experts, count, dtype, p_id)
                mome = UnifiedCPUTensor.get_momentum(size, device_s_experts, count, dtype, p_id)
                vari = UnifiedCPUTensor.get_variance(size, device_s_experts, count, dtype, p_id)
            _init_batched(self.all_tensors, count, bias, fan_in, transposed)
            self.all_tensors.adam_state = self.adam_state
            self.all_tensors.grad_ = grad
            self.all_tensors.momentum = mome
            self.all_tensors.variance = vari
            self.all_tensors.grad_.lazy_zero = True
            moe.set_CPUParamCore(p_id, self.all_tensors, grad, mome, vari, self.bias, self.p_id)
        else:
            self.all_tensors = None

    def fetch_single(self, id):
        return self.all_tensors[id]

    def fetch_single_grad(self, id):
        return self.all_tensors.grad_[id]

    def fetch_batch(self, view_base, start, end):
        return self.all_tensors[start:end]

    def set_lazy_zero(self):
        if self.all_tensors is not None:
            self.all_tensors.grad_.lazy_zero = True

    def unset_lazy_zero(self):
        if self.all_tensors is not None:
            self.all_tensors.grad_.lazy_zero = False


class GPUHostBatchedParameter(object):
    def __init__(self, size, count, dtype, device, moe, p_id, bias=False, fan_in=0,
                 transposed=False):
        self.count = count
        self.size = size
        self.dtype = dtype
        self.device = device
        self.bias = bias
        self.moe = moe
        self.p_id = p_id
        if count > 0:
            self.all_tensors = torch.empty((count, *size), device=device, dtype=dtype)
            self.grad_tensors = torch.zeros((count, *size), device=device, dtype=dtype)
            _init_batched(self.all_tensors, count, bias, fan_in, transposed)
            self.all_tensors.grad = self.grad_tensors
            moe.set_GPUParamCore(p_id, self.all_tensors, self.grad_tensors, self.bias)
        else:
            self.all_tensors = 0
        self.lazy_zero_grad = True

    def fetch_single(self, id):
        return self.all_tensors[id]

    def fetch_single_grad(self, id):
        return self.grad_tensors[id]

    def fetch_batch(self, start, end):
        return self.all_tensors[start:end]

    def fetch_all_with_grad(self):
        ret = self.all_tensors
        ret.grad = self.grad_tensors
        return ret
