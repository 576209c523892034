"""ctypes binding of ``libmole_b200.so`` (declared in ``include/mole_b200.h``).

There is no fallback: if the shared library is missing the import fails with a message
saying how to build it, and every call that returns a non-zero status raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
# MOLE_B200_LIB points at another build of the same library (kernel A/B comparisons)
LIB_PATH = Path(os.environ.get("MOLE_B200_LIB") or _HERE / "lib" / "libmole_b200.so")

MOLE_F32, MOLE_BF16 = 0, 1
ACT_GELU, ACT_RELU = 0, 1
GELU_BWD_EXACT, GELU_BWD_TANH = 0, 1

STATUS_NAMES = {0: "MOLE_OK", -1: "MOLE_ERR_INVALID", -2: "MOLE_ERR_CUDA", -3: "MOLE_ERR_NCCL",
                -4: "MOLE_ERR_UNSUPPORTED", -5: "MOLE_ERR_STATE", -6: "MOLE_ERR_DEVICE"}


class MoleError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class FfnDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "dtype", "act", "gelu_bwd", "M", "F", "L", "n_src", "Cs", "e_begin", "e_end",
        "n_slots", "n_grad_slots", "accumulate", "compact", "backend")]


_p, _i32, _i64 = C.c_void_p, C.c_int32, C.c_int64
_pi32, _pi64 = C.POINTER(C.c_int32), C.POINTER(C.c_int64)

# name -> (restype, argtypes); every symbol declared in include/mole_b200.h
SIGNATURES = {
    "mole_version": (C.c_int, []),
    "mole_last_error_string": (C.c_char_p, []),
    "mole_capacity_stride": (_i64, [_i64]),
    "mole_device_fault": (C.c_int, [_p, _pi32]),
    "mole_device_fault_poll": (C.c_int, [_p]),
    "mole_device_fault_peek": (C.c_int, [_pi32]),
    "mole_launch_count": (C.c_int, [_pi64]),
    "mole_profile_gemm": (C.c_int, [_i32]),
    "mole_profile_read": (C.c_int, [C.POINTER(C.c_float), _pi32, _i32, _pi32]),
    "mole_route_workspace_bytes": (C.c_int, [_i64, _i32, _i32, _pi64]),
    "mole_gate_route_fwd": (C.c_int, [_p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                      _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _p]),
    "mole_gate_route_fwd_static": (C.c_int, [_p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                             _p, _p, _p, _p, _p, _p, _p, _p, _p, _p]),
    "mole_route_from_scores": (C.c_int, [_p, _i64, _i32, _i32, _i32, _i32,
                                         _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _p]),
    "mole_gate_bwd": (C.c_int, [_p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _p, _p]),
    "mole_gate_wgrad_workspace_bytes": (C.c_int, [_i64, _i32, _i32, _i32, _pi64]),
    "mole_gate_wgrad": (C.c_int, [_p, _p, _i64, _i32, _i32, _i32, _p, _p, _i64, _p]),
    "mole_dispatch_fwd": (C.c_int, [_p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _p, _p]),
    "mole_combine_fwd": (C.c_int, [_p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _p, _p]),
    "mole_combine_bwd": (C.c_int, [_p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32,
                                   _p, _p, _p]),
    "mole_dispatch_bwd": (C.c_int, [_p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                    _p, _p]),
    "mole_ffn_workspace_bytes": (C.c_int, [C.POINTER(FfnDesc), _pi64]),
    "mole_ffn_fwd": (C.c_int, [C.POINTER(FfnDesc), _p, _pi32, _p, _p, _p, _p, _p, _p, _p, _p,
                               _p, _i64, _p]),
    "mole_ffn_fwd_combine": (C.c_int, [C.POINTER(FfnDesc), _p, _pi32, _p, _p, _p, _p, _p, _p, _p, _p,
                                       _p, _p, _p, _i32, _p, _p, _i64, _p]),
    "mole_ffn_bwd": (C.c_int, [C.POINTER(FfnDesc), _p, _pi32, _pi32, _p, _p, _p, _p, _p, _p,
                               _p, _p, _p, _p, _p, _p, _p, _i64, _p]),
    "mole_ctx_create": (C.c_int, [_i32, _i32, C.POINTER(_p)]),
    "mole_ctx_destroy": (C.c_int, [_p]),
    "mole_ctx_stream": (C.c_int, [_p, _i32, C.POINTER(_p)]),
    "mole_ctx_wait": (C.c_int, [_p, _p, _p]),
    "mole_ctx_event_record": (C.c_int, [_p, _p, _pi64]),
    "mole_ctx_event_wait": (C.c_int, [_p, _i64, _p]),
    "mole_ctx_synchronize": (C.c_int, [_p, _i32]),
    "mole_comm_unique_id": (C.c_int, [C.POINTER(C.c_uint8)]),
    "mole_comm_create": (C.c_int, [C.POINTER(C.c_uint8), _i32, _i32, _i32, C.POINTER(_p)]),
    "mole_comm_destroy": (C.c_int, [_p]),
    "mole_all2all": (C.c_int, [_p, _p, _p, _i64, _i64, _p]),
    "mole_ffn_fwd_peer": (C.c_int, [C.POINTER(FfnDesc), _p, _pi32, _p, _p, _p, _p, _p, _p, _p,
                                    C.POINTER(_p), _i32, _p, _i64, _p]),
    "mole_ffn_bwd_peer": (C.c_int, [C.POINTER(FfnDesc), _p, _pi32, _pi32, _p, _p, _p, _p, _p, _p, _p,
                                    C.POINTER(_p), _i32, _p, _p, _p, _p, _p, _i64, _p]),
    "mole_dispatch_fwd_peer": (C.c_int, [_p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32,
                                         C.POINTER(_p), C.POINTER(_p), _p, _i32, _i32, _p]),
    "mole_combine_bwd_peer": (C.c_int, [_p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _i32, _i32,
                                        C.POINTER(_p), _p, _i32, _i32, _p, _p]),
    "mole_peer_put_i32": (C.c_int, [_p, _i32, C.POINTER(_p), _i32, _i32, _p]),
    "mole_peer_alloc": (C.c_int, [_i64, C.POINTER(_p)]),
    "mole_peer_free": (C.c_int, [_p]),
    "mole_peer_export": (C.c_int, [_p, C.POINTER(C.c_uint8)]),
    "mole_peer_open": (C.c_int, [C.POINTER(C.c_uint8), C.POINTER(_p)]),
    "mole_peer_close": (C.c_int, [_p]),
    "mole_barrier": (C.c_int, [_p, _p, _p]),
    "mole_peer_barrier": (C.c_int, [C.POINTER(_p), _i32, _i32, _i32, _i64, _p]),
    "mole_pool_create": (C.c_int, [_p, _i32, _i32, _i32, _i32, C.POINTER(_p)]),
    "mole_pool_destroy": (C.c_int, [_p]),
    "mole_pool_base": (C.c_int, [_p, _i32, C.POINTER(_p)]),
    "mole_pool_view_size": (C.c_int, [_p, _pi32]),
    "mole_pool_clear_virtual": (C.c_int, [_p]),
    "mole_pool_prefetch": (C.c_int, [_p, _i32, _i32, _pi32]),
    "mole_pool_pop_prefetched": (C.c_int, [_p, _i32, _pi32]),
    "mole_pool_fetch": (C.c_int, [_p, C.POINTER(_p), _i64, _i32, _i32, _i32, _i32, _pi32]),
    "mole_pool_wait_fetch": (C.c_int, [_p, _i32, _p]),
    "mole_pool_mark_used": (C.c_int, [_p, _i32, _i32, _p]),
    "mole_pool_log": (C.c_int, [_p, _pi32, _i32, _pi32]),
    "mole_pool_abs_slot": (C.c_int, [_p, _i32, _pi32]),
    "mole_store_to_host": (C.c_int, [_p, _p, _p, _i64, _p]),
    "mole_adam_update": (C.c_int, [_p, _p, _p, _p, _p, _i64, _i32, C.c_float, C.c_float, _i32,
                                   C.c_float, C.c_float, C.c_float, _i32, _p]),
    "mole_fast_assign_prefetch": (C.c_int, [_i32, _pi32, _pi32, _i32, _pi32, _pi32, _i32, _pi32]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library is the only implementation of this "
            "package (there is no CPU or PyTorch fallback).  Build it with "
            "`python mole_b200/build.py` (needs nvcc).")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int) -> None:
    if status != 0:
        raise MoleError(status, lib.mole_last_error_string().decode(errors="replace"))


def capacity_stride(capacity: int) -> int:
    return int(lib.mole_capacity_stride(capacity))
