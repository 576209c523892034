"""Stream roles of the expert pipeline (interface of MOLE/utils/Ustream.py:6-73).

The streams are created by the C library (``mole_ctx_create``, which replaces the 16-stream
manager of MOLE/cpp/stream.cpp:38-144) and wrapped as ``torch.cuda.ExternalStream`` so that
PyTorch allocations and kernels can be ordered against them.  Roles: 1 = host-to-device
transfer, 2 = compute, 3 = communication, 4 = device-to-host transfer.  As in the reference the
compute stream becomes PyTorch's current stream when the context is built.
"""
from __future__ import annotations

import ctypes as C

import torch

from .._lib import check, lib


class ExpertStreamCtx(object):
    _instance = None

    def __new__(cls, *args, **kw):
        if cls._instance is None:
            inst = object.__new__(cls)
            inst.disable = bool(kw.get("disable", False))
            inst.device = torch.device(kw.get("device", "cuda:0"))
            idx = int(inst.device.index or 0)
            inst.default = torch.cuda.current_stream(device=inst.device)
            handle = C.c_void_p()
            check(lib.mole_ctx_create(idx, int(inst.disable), C.byref(handle)))
            inst.handle = handle
            inst.stream_pool = []
            for i in range(16):
                s = C.c_void_p()
                check(lib.mole_ctx_stream(handle, i, C.byref(s)))
                inst.stream_pool.append(
                    inst.default if inst.disable or not s.value
                    else torch.cuda.ExternalStream(s.value, device=inst.device))
            inst.max_stream_count = len(inst.stream_pool)
            cls._instance = inst
            if not inst.disable and kw.get("set_current", True):
                torch.cuda.set_stream(inst.stream_pool[2])
        return cls._instance

    def __init__(self, *args, **kw):
        pass

    @classmethod
    def get(cls, device=None, disable=False) -> "ExpertStreamCtx":
        if cls._instance is None:
            # built on demand by the layer: PyTorch's current stream stays what it is and plays
            # the compute role
            cls(device=device if device is not None else torch.device("cuda", torch.cuda.current_device()),
                disable=disable, set_current=False)
        return cls._instance

    @staticmethod
    def max_stream_count():
        return ExpertStreamCtx._instance.max_stream_count

    @staticmethod
    def stream(idx):
        return ExpertStreamCtx._instance.stream_pool[idx]

    @staticmethod
    def tran_stream():
        return ExpertStreamCtx._instance.stream_pool[1]

    @staticmethod
    def comp_stream():
        return ExpertStreamCtx._instance.stream_pool[2]

    @staticmethod
    def comm_stream():
        return ExpertStreamCtx._instance.stream_pool[3]

    @staticmethod
    def tran_back_stream():
        return ExpertStreamCtx._instance.stream_pool[4]

    @staticmethod
    def default_stream():
        return ExpertStreamCtx._instance.default

    @staticmethod
    def all_streams_cdata():
        return [s.cuda_stream for s in ExpertStreamCtx._instance.stream_pool]

    @staticmethod
    def wait(waiter: torch.cuda.Stream, waited: torch.cuda.Stream) -> None:
        """``waiter`` waits for everything enqueued so far on ``waited``."""
        inst = ExpertStreamCtx._instance
        check(lib.mole_ctx_wait(inst.handle, C.c_void_p(waiter.cuda_stream),
                                C.c_void_p(waited.cuda_stream)))

    @staticmethod
    def record(stream: torch.cuda.Stream) -> int:
        """Ticket for the work enqueued on ``stream`` so far (a per-record event)."""
        inst = ExpertStreamCtx._instance
        t = C.c_int64()
        check(lib.mole_ctx_event_record(inst.handle, C.c_void_p(stream.cuda_stream), C.byref(t)))
        return t.value

    @staticmethod
    def wait_ticket(waiter: torch.cuda.Stream, ticket: int) -> None:
        """``waiter`` waits for the work named by ``ticket`` only."""
        inst = ExpertStreamCtx._instance
        check(lib.mole_ctx_event_wait(inst.handle, ticket, C.c_void_p(waiter.cuda_stream)))
