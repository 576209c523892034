"""Autograd functions of the MoE layer.  Each stage of the reference ``forward``
(MOLE/moe/layer.py:429-476) is one ``torch.autograd.Function`` over the C ABI:

  GateRoute       gate + extract_critical   (layer.py:442-447)   -> gates, l_aux, routing plan
  Dispatch        fast_encode               (layer.py:448-449)   -> [E, Cs, M] rows
  BatchFusedFWD   the expert pipeline       (layer.py:453)       -> [E, Cs, M] rows
  Combine         fast_decode               (layer.py:456-458)   -> [T, M]
  pfetchbwd       backward-prefetch trigger (layer.py:435-436)

``BatchFusedFWD`` and ``pfetchbwd`` are used by the reference layer but defined nowhere in its
tree; they are written here from their call sites and from ``_MOLECore::forward/backward``
(MOLE/cpp/define.hpp:594-606).
"""
from __future__ import annotations

import torch

from .. import ops
from ..utils.Utimer import UATimer


class GateRoute(torch.autograd.Function):
    """``(x, wg) -> (gates [T, k] f32, l_aux [] f32)``; the integer routing plan is returned
    through ``holder['plan']``.

    ``holder`` is also how ``Dispatch.backward`` hands over its incoming gradient: autograd runs
    it before this node (it was recorded later), and the gradient of ``x`` through the gate
    (``dlogits @ Wg``) and through the dispatch (sum of the token's rows) is then produced by one
    fused kernel here instead of two kernels and an addition."""

    @staticmethod
    def forward(ctx, x, wg, logit_bias, k, cap, normalize, holder):
        plan = ops.gate_route(x, wg, k, cap, logit_bias, normalize)
        holder["plan"] = plan
        ctx.plan = plan
        ctx.holder = holder
        ctx.save_for_backward(x, wg)
        return plan.gates, plan.l_aux.view(())

    @staticmethod
    def backward(ctx, dgates, dl_aux):
        x, wg = ctx.saved_tensors
        plan = ctx.plan
        ctx.holder["gate_backward_done"] = True
        ddisp = ctx.holder.pop("pending_ddisp", None)
        if dgates is None:
            dgates = torch.zeros_like(plan.gates)
        dl = None if dl_aux is None else dl_aux.reshape(1).float().contiguous()
        dlogits = ops.gate_bwd(plan, dgates.contiguous(), dl)
        dwg = dx = None
        if ctx.needs_input_grad[1]:
            dwg = ops.gate_wgrad(dlogits, x).to(wg.dtype)
        if ctx.needs_input_grad[0] or ddisp is not None:
            dx = ops.dispatch_bwd(ddisp, plan, x.shape[1], x.dtype, x.device, dlogits, wg)
        return dx, dwg, None, None, None, None, None


class Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan, holder=None):
        ctx.plan = plan
        ctx.holder = holder
        ctx.meta = (x.shape[1], x.dtype, x.device)
        peer = holder.get("peer") if holder is not None else None
        if peer is not None:
            # rows go straight into the owners' memory; the local [E, Cs, M] tensor is a
            # placeholder that carries the autograd edge only
            ops.dispatch_peer(x, plan, peer)
            return x.new_zeros(1).expand(plan.E, plan.Cs, x.shape[1])
        return ops.dispatch(x, plan)

    @staticmethod
    def backward(ctx, ddisp):
        M, dtype, device = ctx.meta
        h = ctx.holder
        if h is not None and h.get("tap") is not None:
            peer = h.get("peer")
            h["tap"]["dx_rows"] = peer.dx if peer is not None else ddisp
        if h is not None and h.get("gate_needs_x_grad") and not h.get("gate_backward_done"):
            # the gate's backward is still to come and will emit the fused gradient of x
            h["pending_ddisp"] = ddisp.contiguous()
            return None, None, None
        return ops.dispatch_bwd(ddisp.contiguous(), ctx.plan, M, dtype, device), None, None


class Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, gates, plan, peer=None, fused_y=None):
        ctx.plan = plan
        ctx.peer = peer
        ctx.save_for_backward(rows, gates)
        if fused_y is not None:        # already produced by the expert pipeline's last epilogue
            return fused_y
        return ops.combine(rows, plan, gates)

    @staticmethod
    def backward(ctx, dy):
        rows, gates = ctx.saved_tensors
        if ctx.peer is not None:        # row gradients go straight to the experts' owners
            dgates = ops.combine_bwd_peer(dy.contiguous(), rows, ctx.plan, gates, ctx.peer)
            return dy.new_zeros(1).expand_as(rows), dgates, None, None, None
        drows, dgates = ops.combine_bwd(dy.contiguous(), rows, ctx.plan, gates)
        return drows, dgates, None, None, None


class BatchFusedFWD(torch.autograd.Function):
    """``apply(dispatched_input, module, dummy_param, time_it, prefetch)`` as the reference layer
    calls it.  ``module._route_counts`` (set by the layer) holds the valid rows of every
    (expert) chunk; without it every chunk is taken as full, which is the reference's
    capacity-padded computation."""

    @staticmethod
    def forward(ctx, dispatched_input, module, dummy_param, time_it=False, prefetch=False):
        core = module.MOLECore
        counts = getattr(module, "_route_counts", None)
        E, Cs, M = dispatched_input.shape
        if counts is None:
            counts = torch.full((E,), Cs, dtype=torch.int32, device=dispatched_input.device)
        ctx.core = core
        ctx.counts = counts
        ctx.input_requires_grad = ctx.needs_input_grad[0]
        ctx.dummy_shape = dummy_param.shape
        timer = module.timer if time_it and hasattr(module, "timer") else None
        ctx.peer = getattr(module, "_peer_exchange", None)
        ctx.time_it = bool(time_it)
        ctx.moe_id = getattr(module, "moe_id", 0)
        if time_it:
            # the gap since the step began (or since the previous MoE layer finished) is the time
            # this layer's experts could have been travelling: the scheduler sizes prefetches by it
            UATimer.track_fwd_end()
        if timer:
            timer.start_fwd()
        if ctx.peer is not None:
            out = core.forward_peer(ctx.peer, True)
        else:
            # the layer may ask for the combine to be fused into the second GEMM's epilogue
            fuse = getattr(module, "_fuse", None)
            combine = None
            if fuse is not None:
                plan, gates = fuse["plan"], fuse["gates"]
                y = torch.zeros(plan.T, M, dtype=dispatched_input.dtype, device=dispatched_input.device)
                fuse["y"] = y
                combine = (plan, gates.detach(), y)
            out = core.forward(dispatched_input.contiguous(), counts, True, combine=combine)
        if timer:
            timer.stop_fwd()
        if time_it:
            last = len(type(module)._instance) - 1
            if ctx.moe_id >= last:
                UATimer.track_bwd_start()       # next: the gap in front of the last layer's backward
            else:
                UATimer.track_fwd_start()
        return out

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.time_it:
            UATimer.track_bwd_end()
        dx = BatchFusedFWD._backward(ctx, grad_out)
        if ctx.time_it and ctx.moe_id > 0:
            UATimer.track_bwd_start()
        dummy_grad = torch.zeros(ctx.dummy_shape, device=grad_out.device, dtype=grad_out.dtype)
        return dx, None, dummy_grad, None, None

    @staticmethod
    def _backward(ctx, grad_out):
        if ctx.peer is not None:
            dx = ctx.core.backward_peer(ctx.peer, ctx.input_requires_grad)
        else:
            dx = ctx.core.backward(grad_out.contiguous(), ctx.counts, ctx.input_requires_grad)
        return dx


class pfetchbwd(torch.autograd.Function):
    """Identity in forward; in backward (which runs after the layer's own backward) it starts the
    host-to-device prefetch for the previous layer's backward, mirroring how forward prefetches
    the next layer (MOLE/moe/layer.py:464-472)."""

    @staticmethod
    def forward(ctx, input_, module):
        ctx.module = module
        return input_.view_as(input_)

    @staticmethod
    def backward(ctx, grad):
        m = ctx.module
        inst = type(m)._instance
        if m.moe_id > 0:
            prev = inst[m.moe_id - 1]
            if m.global_prefetch:
                prev.global_prefetch_bwd()
            prev.local_prefetch_bwd()
        return grad, None
