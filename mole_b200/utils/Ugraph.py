"""A training step of GPU-resident MoE layers captured in a CUDA graph.

A forward + backward of one layer is two dozen kernel launches of a few microseconds to half a
millisecond each; enqueued one by one they leave ~2 us between kernels and tie the step's time to
how fast the host can enqueue (a busy host makes the GPU wait).  ``GraphedStep`` runs the step a
few times on a side stream, captures one run into a ``torch.cuda.CUDAGraph`` and then replays it:
one launch per step, nothing left for the host to do.

What can be captured: layers whose experts all live on the GPU, on one rank (the offload
pipeline and the expert-parallel exchange take host-side decisions per step -- pool slots, stream
tickets, barrier sequence numbers -- and stay eager).  The step function must be static: same
shapes, same capacity factor, inputs updated in place (``x.copy_(...)``) between replays.  Every
tensor the step produces is allocated once, inside the capture; ``outputs`` keeps what the step
function returned.

One rule comes from autograd: the accumulation of a gradient into a leaf (a parameter, an input
with ``requires_grad``) is tied to the stream that was current when the leaf was created, and a
captured step must not reach out to another stream.  So create the layer and such inputs under
``torch.cuda.stream(s)`` and hand the same ``s`` to ``GraphedStep`` (it warms up and captures
there); a layer that has run eagerly before should drop what keeps the old autograd graph alive
(``layer.l_aux = None``).  The reference has no counterpart (it enqueues every kernel of every step).
"""
from __future__ import annotations

import torch

from .. import ops


class GraphedStep:
    def __init__(self, step_fn, stream: torch.cuda.Stream, warmup: int = 3, poll_every: int = 16):
        self.step_fn = step_fn
        self.poll_every = max(1, int(poll_every))
        self.replays = 0
        side = stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):       # first-use set-up (function attributes, tensor
                step_fn()                          # maps, workspaces) must not happen under capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            self.outputs = step_fn()

    def __call__(self):
        self.graph.replay()
        self.replays += 1
        # a captured stream takes no fault poll (mole_device_fault_poll): ask behind a replay
        if self.replays % self.poll_every == 0:
            ops.device_fault_poll()
            code = ops.device_fault_peek()
            if code:
                raise RuntimeError(f"a kernel of a replayed step gave up on a bounded wait (fault code {code})")
        return self.outputs
