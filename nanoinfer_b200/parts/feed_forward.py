"""Feed-forward parts.  Built in: the dense SwiGLU."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import Part, WeightSlot


class SwiGLU(Part):
    """y = down(silu(gate(x)) * up(x)); gate and up are one fused projection
    (src/model/llama.cpp:364-379, src/op/kernels/cuda/swiglu_kernel.cu:25-40)."""

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        i = spec.intermediate_size
        return {"gate": WeightSlot((i, hidden_size)), "up": WeightSlot((i, hidden_size)),
                "down": WeightSlot((hidden_size, i))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.inter = spec.intermediate_size
        self.w_gate_up = rt.weight(torch.cat([weights["gate"], weights["up"]], dim=0))
        self.w_down = rt.weight(weights["down"])

    adds_into_residual = True   # forward() accepts residual= and may add its output there

    def forward(self, x: torch.Tensor, ctx, residual=None):
        rt = self.rt
        gate_up = rt.linear(x, self.w_gate_up)
        act = rt.empty(x.shape[0], self.inter)
        ops.swiglu(gate_up, act)
        return rt.linear(act, self.w_down, residual=residual)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
