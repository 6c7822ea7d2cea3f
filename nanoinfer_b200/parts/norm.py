"""RMSNorm, fused with the residual addition that precedes it."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import Part, WeightSlot


class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * gain, statistics in FP32
    (src/op/kernels/cuda/rmsnorm_kernel.cu:49-104; eps inside the root, :79)."""

    # What a kernel that runs this norm inside itself computes (with ``gain`` and ``eps``): the
    # skinny products fuse norms of this kind only.
    fused_kind = "rmsnorm"

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        return {"weight": WeightSlot((hidden_size,), init="ones")}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.eps = float(spec.eps)
        self.gain = rt.gain(weights["weight"])

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.hidden_size)
        ops.add_rmsnorm(h, delta, self.gain, self.eps, out, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm, replace=True)
