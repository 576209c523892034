"""Top-k softmax gate of the MoE layer (interface of MOLE/utils/Ugate.py:5-14).

``MOLETopk(model_dim, total_experts)`` owns a bias-free ``linear``; calling it returns the
softmax scores ``[T, E]`` in fp32, computed by the same fused CUDA kernel the layer uses.
``logit_bias`` (fp32 ``[E]``, optional, not a parameter) is added to the logits before the
softmax; the skewed-routing benchmark uses it to make expert popularity follow a Zipf law.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class MOLETopk(torch.nn.Module):
    def __init__(self, model_dim: int, total_experts: int) -> None:
        super().__init__()
        self.total_experts = total_experts
        self.linear = torch.nn.Linear(model_dim, total_experts, bias=False)
        self.logit_bias: Optional[torch.Tensor] = None

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x = input.reshape(-1, input.shape[-1]).contiguous()
        plan = ops.gate_route(x, self.linear.weight.detach().contiguous(), 1, 1,
                              self.logit_bias, False)
        return plan.scores
