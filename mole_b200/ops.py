"""Tensor-level wrappers over the C ABI.

PyTorch owns device memory and streams; every function here checks shapes, allocates outputs
with ``torch.empty`` and hands raw pointers to ``libmole_b200.so`` on the current stream.
None of them has a PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import FfnDesc, check, lib

_DTYPES = {torch.float32: _lib.MOLE_F32, torch.bfloat16: _lib.MOLE_BF16}
_ACTS = {"gelu": _lib.ACT_GELU, "relu": _lib.ACT_RELU}
_GELU_BWD = {"exact": _lib.GELU_BWD_EXACT, "tanh": _lib.GELU_BWD_TANH}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; the kernels cover float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None or isinstance(t, int):
        return t          # a raw device address (slot-pool base) passes through
    if not t.is_cuda:
        raise RuntimeError("mole_b200 kernels take CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError("mole_b200 kernels take contiguous tensors")
    return t.data_ptr()


def _stream() -> int:
    # the raw handle of the current stream of the current device; torch.cuda.current_stream()
    # builds a Stream object through several Python layers (17 us a call, a dozen calls a step)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def capacity(T: int, E: int, k: int, capacity_factor: float) -> int:
    """``C = max(1, ceil(k * capacity_factor * T / E))`` with T the tokens on this rank."""
    return max(1, int(math.ceil(k * capacity_factor * T / E)))


@dataclass
class RoutePlan:
    """Routing-index build of one batch (all device tensors)."""
    T: int
    E: int
    k: int
    C: int            # capacity
    Cs: int           # capacity stride of the row buffers (C rounded up to 128)
    normalize: bool
    scores: torch.Tensor      # [T, E] f32
    idx: torch.Tensor         # [T, k] i32
    slot: torch.Tensor        # [T, k] i32, kept iff slot < C
    gates: torch.Tensor       # [T, k] f32, 0 where dropped
    counts: torch.Tensor      # [E] i32
    offsets: torch.Tensor     # [E + 1] i32
    perm: torch.Tensor        # [T * k] i32
    first_hist: torch.Tensor  # [E] i32
    l_aux: torch.Tensor       # [1] f32


def _alloc_plan(T, E, k, C, normalize, device, scores=None) -> RoutePlan:
    i32 = dict(dtype=torch.int32, device=device)
    f32 = dict(dtype=torch.float32, device=device)
    return RoutePlan(
        T, E, k, C, _lib.capacity_stride(C), bool(normalize),
        scores if scores is not None else torch.empty(T, E, **f32),
        torch.empty(T, k, **i32), torch.empty(T, k, **i32), torch.empty(T, k, **f32),
        torch.empty(E, **i32), torch.empty(E + 1, **i32), torch.empty(T * k, **i32),
        torch.empty(E, **i32), torch.empty(1, **f32))


def _route_workspace(T, E, k, device) -> torch.Tensor:
    n = C.c_int64()
    check(lib.mole_route_workspace_bytes(T, E, k, C.byref(n)))
    return torch.empty(n.value, dtype=torch.uint8, device=device)


def gate_route(x: torch.Tensor, wg: torch.Tensor, k: int, cap: int,
               logit_bias: Optional[torch.Tensor] = None, normalize: bool = False) -> RoutePlan:
    """Fused gate + routing-index build: ``softmax(x @ wg^T + bias)``, top-k, slots, permutation."""
    T, M = x.shape
    E = wg.shape[0]
    if wg.shape[1] != M or wg.dtype != x.dtype:
        raise ValueError("gate weight must be [E, M] in the dtype of x")
    if logit_bias is not None and (logit_bias.dtype != torch.float32 or logit_bias.numel() != E):
        raise ValueError("logit_bias must be float32 [E]")
    plan = _alloc_plan(T, E, k, cap, normalize, x.device)
    ws = _route_workspace(T, E, k, x.device)
    check(lib.mole_gate_route_fwd(
        _ptr(x), _ptr(wg), _ptr(logit_bias), T, M, E, k, cap, int(normalize), _dt(x),
        _ptr(plan.scores), _ptr(plan.idx), _ptr(plan.slot), _ptr(plan.gates), _ptr(plan.counts),
        _ptr(plan.offsets), _ptr(plan.perm), _ptr(plan.first_hist), _ptr(plan.l_aux),
        _ptr(ws), ws.numel(), _stream()))
    return plan


def gate_route_static(x: torch.Tensor, wg: torch.Tensor, k: int, cap: int,
                      logit_bias: Optional[torch.Tensor] = None, normalize: bool = False,
                      plan: Optional[RoutePlan] = None) -> RoutePlan:
    """``gate_route`` through the entry point that allocates nothing: the routing scratch is the
    library's built-in 4 MiB array.  For hosts that have given all device memory to their own
    pool or must not trigger a driver allocation; pass a pre-allocated ``plan`` to keep this
    wrapper allocation-free too.  Calls that overlap on the GPU race on the shared scratch."""
    T, M = x.shape
    E = wg.shape[0]
    if wg.shape[1] != M or wg.dtype != x.dtype:
        raise ValueError("gate weight must be [E, M] in the dtype of x")
    if plan is None:
        plan = _alloc_plan(T, E, k, cap, normalize, x.device)
    check(lib.mole_gate_route_fwd_static(
        _ptr(x), _ptr(wg), _ptr(logit_bias), T, M, E, k, cap, int(normalize), _dt(x),
        _ptr(plan.scores), _ptr(plan.idx), _ptr(plan.slot), _ptr(plan.gates), _ptr(plan.counts),
        _ptr(plan.offsets), _ptr(plan.perm), _ptr(plan.first_hist), _ptr(plan.l_aux), _stream()))
    return plan


def route_from_scores(scores: torch.Tensor, k: int, cap: int, normalize: bool = False) -> RoutePlan:
    """Routing-index build from given fp32 scores (identical scores in, identical integers out)."""
    if scores.dtype != torch.float32:
        raise TypeError("scores must be float32")
    T, E = scores.shape
    plan = _alloc_plan(T, E, k, cap, normalize, scores.device, scores=scores)
    ws = _route_workspace(T, E, k, scores.device)
    check(lib.mole_route_from_scores(
        _ptr(scores), T, E, k, cap, int(normalize), _ptr(plan.idx), _ptr(plan.slot),
        _ptr(plan.gates), _ptr(plan.counts), _ptr(plan.offsets), _ptr(plan.perm),
        _ptr(plan.first_hist), _ptr(plan.l_aux), _ptr(ws), ws.numel(), _stream()))
    return plan


def gate_bwd(plan: RoutePlan, dgates: torch.Tensor,
             d_l_aux: Optional[torch.Tensor]) -> torch.Tensor:
    dlogits = torch.empty(plan.T, plan.E, dtype=torch.float32, device=dgates.device)
    check(lib.mole_gate_bwd(
        _ptr(plan.scores), _ptr(plan.idx), _ptr(plan.slot), _ptr(dgates), _ptr(d_l_aux),
        _ptr(plan.first_hist), plan.T, plan.E, plan.k, plan.C, int(plan.normalize),
        _ptr(dlogits), _stream()))
    return dlogits


def gate_wgrad(dlogits: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``dlogits^T @ x`` as fp32 ``[E, M]``."""
    T, M = x.shape
    E = dlogits.shape[1]
    dwg = torch.zeros(E, M, dtype=torch.float32, device=x.device)
    n = C.c_int64()
    check(lib.mole_gate_wgrad_workspace_bytes(T, M, E, _dt(x), C.byref(n)))
    ws = torch.empty(n.value, dtype=torch.uint8, device=x.device)
    check(lib.mole_gate_wgrad(_ptr(dlogits), _ptr(x), T, M, E, _dt(x), _ptr(dwg), _ptr(ws),
                              ws.numel(), _stream()))
    return dwg


def dispatch(x: torch.Tensor, plan: RoutePlan, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[T, M] -> [E, Cs, M]`` capacity-strided rows."""
    T, M = x.shape
    if out is None:
        out = torch.empty(plan.E, plan.Cs, M, dtype=x.dtype, device=x.device)
    check(lib.mole_dispatch_fwd(_ptr(x), _ptr(plan.counts), _ptr(plan.offsets), _ptr(plan.perm),
                                T, M, plan.E, plan.k, plan.Cs, _dt(x), _ptr(out), _stream()))
    return out


def combine(rows: torch.Tensor, plan: RoutePlan, gates: torch.Tensor) -> torch.Tensor:
    """``[E, Cs, M] -> [T, M]``: gate-weighted sum of each token's kept rows."""
    M = rows.shape[-1]
    y = torch.empty(plan.T, M, dtype=rows.dtype, device=rows.device)
    check(lib.mole_combine_fwd(_ptr(rows), _ptr(plan.idx), _ptr(plan.slot), _ptr(gates), plan.T, M,
                               plan.E, plan.k, plan.C, plan.Cs, _dt(rows), _ptr(y), _stream()))
    return y


def combine_bwd(dy: torch.Tensor, rows: torch.Tensor, plan: RoutePlan, gates: torch.Tensor):
    M = rows.shape[-1]
    drows = torch.empty_like(rows)
    dgates = torch.empty(plan.T, plan.k, dtype=torch.float32, device=rows.device)
    check(lib.mole_combine_bwd(_ptr(dy), _ptr(rows), _ptr(gates), _ptr(plan.counts),
                               _ptr(plan.offsets), _ptr(plan.perm), plan.T, M, plan.E, plan.k,
                               plan.Cs, _dt(rows), _ptr(drows), _ptr(dgates), _stream()))
    return drows, dgates


def dispatch_bwd(ddisp: Optional[torch.Tensor], plan: RoutePlan, M: int, dtype, device,
                 dlogits: Optional[torch.Tensor] = None,
                 wg: Optional[torch.Tensor] = None) -> torch.Tensor:
    dx = torch.empty(plan.T, M, dtype=dtype, device=device)
    check(lib.mole_dispatch_bwd(_ptr(ddisp), _ptr(plan.idx), _ptr(plan.slot), _ptr(dlogits),
                                _ptr(wg), plan.T, M, plan.E, plan.k, plan.C, plan.Cs,
                                _DTYPES[dtype], _ptr(dx), _stream()))
    return dx


# ---- grouped FFN -----------------------------------------------------------------------
def make_ffn_desc(dtype, act: str, gelu_bwd: str, M: int, F: int, L: int, n_src: int, Cs: int,
                  e_begin: int, e_end: int, n_slots: int, accumulate: bool = False,
                  backend: int = 0, n_grad_slots: int = 0, compact: int = 0) -> FfnDesc:
    return FfnDesc(_DTYPES[dtype], _ACTS[act], _GELU_BWD[gelu_bwd], M, F, L, n_src, Cs,
                   e_begin, e_end, n_slots, n_grad_slots, int(accumulate), compact, backend)


def ffn_workspace(desc: FfnDesc, device) -> torch.Tensor:
    n = C.c_int64()
    check(lib.mole_ffn_workspace_bytes(C.byref(desc), C.byref(n)))
    return torch.empty(n.value, dtype=torch.uint8, device=device)


def _slot_array(slots: Optional[Sequence[int]], L: int):
    if slots is None:
        return None
    if len(slots) != L:
        raise ValueError("slot map must have one entry per local expert")
    return (C.c_int32 * L)(*slots)


def ffn_fwd(desc: FfnDesc, counts, x, w1, b1, w2, b2, x1, h, out, ws,
            slot_of_expert: Optional[Sequence[int]] = None) -> None:
    check(lib.mole_ffn_fwd(C.byref(desc), _ptr(counts), _slot_array(slot_of_expert, desc.L),
                           _ptr(x), _ptr(w1), _ptr(b1), _ptr(w2), _ptr(b2), _ptr(x1), _ptr(h),
                           _ptr(out), _ptr(ws), ws.numel(), _stream()))


def ffn_fwd_combine(desc: FfnDesc, counts, x, w1, b1, w2, b2, x1, h, out, plan: RoutePlan, gates, y,
                    ws, slot_of_expert: Optional[Sequence[int]] = None) -> None:
    """``ffn_fwd`` whose second GEMM also adds ``gates * out_row`` into ``y[token]`` (``y`` zeroed
    by the caller): the combine fused into the W2 epilogue."""
    check(lib.mole_ffn_fwd_combine(C.byref(desc), _ptr(counts), _slot_array(slot_of_expert, desc.L),
                                   _ptr(x), _ptr(w1), _ptr(b1), _ptr(w2), _ptr(b2), _ptr(x1), _ptr(h),
                                   _ptr(out), _ptr(plan.offsets), _ptr(plan.perm), _ptr(gates), plan.k,
                                   _ptr(y), _ptr(ws), ws.numel(), _stream()))


def ffn_bwd(desc: FfnDesc, counts, dout, x, x1, h, w1, w2, dx1, dx, gw1, gb1, gw2, gb2, ws,
            slot_of_expert: Optional[Sequence[int]] = None,
            grad_slot_of_expert: Optional[Sequence[int]] = None) -> None:
    check(lib.mole_ffn_bwd(C.byref(desc), _ptr(counts), _slot_array(slot_of_expert, desc.L),
                           _slot_array(grad_slot_of_expert, desc.L), _ptr(dout), _ptr(x), _ptr(x1),
                           _ptr(h), _ptr(w1), _ptr(w2), _ptr(dx1), _ptr(dx), _ptr(gw1), _ptr(gb1),
                           _ptr(gw2), _ptr(gb2), _ptr(ws), ws.numel(), _stream()))


# ---- push-style exchange (rows stored straight into the owner's / source's memory) -----------
def dispatch_peer(x: torch.Tensor, plan: RoutePlan, peer) -> None:
    """Dispatch whose rows (and per-expert counts) land in the receive buffers of the experts'
    owners; ``peer`` is a ``core.PeerExchange``."""
    T, M = x.shape
    all_counts = None
    if peer.packed:
        # every rank learns every rank's counts first, so that rows can go straight to their final
        # place in the owner's per-expert run
        check(lib.mole_peer_put_i32(_ptr(plan.counts), plan.E, peer.table["allcounts"], peer.world,
                                    peer.rank, _stream()))
        peer.barrier()
        all_counts = peer.allcounts
    check(lib.mole_dispatch_fwd_peer(_ptr(x), _ptr(plan.counts), _ptr(plan.offsets), _ptr(plan.perm),
                                     T, M, plan.E, plan.k, plan.Cs, _dt(x), peer.table["x0"],
                                     peer.table["counts"], _ptr(all_counts), peer.world, peer.rank,
                                     _stream()))


def combine_bwd_peer(dy: torch.Tensor, rows: torch.Tensor, plan: RoutePlan, gates: torch.Tensor,
                     peer) -> torch.Tensor:
    """Combine backward whose row gradients land in the owners' buffers; returns ``dgates``."""
    M = rows.shape[-1]
    dgates = torch.empty(plan.T, plan.k, dtype=torch.float32, device=rows.device)
    check(lib.mole_combine_bwd_peer(_ptr(dy), _ptr(rows), _ptr(gates), _ptr(plan.counts),
                                    _ptr(plan.offsets), _ptr(plan.perm), plan.T, M, plan.E, plan.k,
                                    plan.Cs, _dt(rows), peer.table["g"],
                                    _ptr(peer.allcounts) if peer.packed else None, peer.world,
                                    peer.rank, _ptr(dgates), _stream()))
    return dgates


def ffn_fwd_peer(desc: FfnDesc, counts, x, w1, b1, w2, b2, x1, h, peer, ws,
                 slot_of_expert: Optional[Sequence[int]] = None) -> None:
    check(lib.mole_ffn_fwd_peer(C.byref(desc), _ptr(counts), _slot_array(slot_of_expert, desc.L),
                                _ptr(x), _ptr(w1), _ptr(b1), _ptr(w2), _ptr(b2), _ptr(x1), _ptr(h),
                                peer.table["ret"], peer.rank, _ptr(ws), ws.numel(), _stream()))


def ffn_bwd_peer(desc: FfnDesc, counts, dout, x, x1, h, w1, w2, dx1, peer, gw1, gb1, gw2, gb2, ws,
                 slot_of_expert: Optional[Sequence[int]] = None,
                 grad_slot_of_expert: Optional[Sequence[int]] = None) -> None:
    check(lib.mole_ffn_bwd_peer(C.byref(desc), _ptr(counts), _slot_array(slot_of_expert, desc.L),
                                _slot_array(grad_slot_of_expert, desc.L), _ptr(dout), _ptr(x),
                                _ptr(x1), _ptr(h), _ptr(w1), _ptr(w2), _ptr(dx1), peer.table["dx"],
                                peer.rank, _ptr(gw1), _ptr(gb1), _ptr(gw2), _ptr(gb2), _ptr(ws),
                                ws.numel(), _stream()))


def device_fault_poll() -> None:
    """Enqueues a copy of the fault word behind the current stream's work (no host wait)."""
    check(lib.mole_device_fault_poll(_stream()))


def device_fault_peek() -> int:
    """Value of the last polled copy that has landed (0 before the first)."""
    f = C.c_int32()
    check(lib.mole_device_fault_peek(C.byref(f)))
    return f.value


def device_fault() -> int:
    """Code left by a kernel whose bounded wait ran out (0 = none); synchronises the stream."""
    f = C.c_int32()
    check(lib.mole_device_fault(_stream(), C.byref(f)))
    return f.value
