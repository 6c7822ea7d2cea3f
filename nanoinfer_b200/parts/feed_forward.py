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
        gate, up = weights["gate"], weights["up"]
        # blocked layout: 8 gate rows, then their 8 up rows - a gate value and its up value land
        # in the same 16-row tile of the projection, and the activation kernel works on 16 bytes
        self.blocked = self.inter % 8 == 0
        if self.blocked:
            i, d = gate.shape
            w13 = torch.stack([gate.view(i // 8, 8, d), up.view(i // 8, 8, d)], dim=1).reshape(2 * i, d)
        else:
            w13 = torch.cat([gate, up], dim=0)
        self.w_gate_up = rt.weight(w13)
        self.w_down = rt.weight(weights["down"])

    adds_into_residual = True   # forward() accepts residual= and may add its output there
    graph_safe = "all"

    def weights_in_order(self) -> tuple:
        return (self.w_gate_up, self.w_down)

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        return self.blocked and self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    hands_off_norm = True       # forward_fused_norm / forward_prenormed accept then_norm= and may return its NormHandoff

    def forward(self, x: torch.Tensor, ctx, residual=None):
        rt = self.rt
        n = x.shape[0]
        act = rt.empty(n, self.inter)
        if self.blocked and rt.skinny(n, self.hidden_size):
            ops.gemv_bf16(x, self.w_gate_up, act, ops.SWIGLU_BF16,     # activation in the epilogue
                          warm=rt.warm(self.w_down, 0, which=2))
        elif self.blocked and rt.tensor_core_gemm(n, self.hidden_size):
            ops.gemm_tc(x, self.w_gate_up, act, ops.SWIGLU_BF16)       # tcgen05 product, activation fused
        elif self.blocked and rt.mid_batch(n, self.hidden_size, rt.MID_GATE_UP):
            ops.gemm_swap_tc(x, self.w_gate_up, act, ops.SWIGLU_BF16)  # weights on the tile's lanes, activation fused
        else:
            gate_up = rt.linear(x, self.w_gate_up)
            ops.swiglu(gate_up, act, blocked=self.blocked)
        if residual is not None and rt.mid_batch(n, self.inter, rt.MID_DOWN):
            ops.gemm_swap_tc(act, self.w_down, residual, ops.ADD_F32)
            return None
        return rt.linear(act, self.w_down, residual=residual, warm=rt.warm_after(ctx, which=4))

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, residual=None, then_norm=None):
        """As forward, with x = norm(h): norm, projection and activation in one launch.  ``then_norm``:
        the norm that reads the stream next; where the down projection can prepare it, its
        NormHandoff is returned instead of None."""
        rt = self.rt
        act = rt.empty(h.shape[0], self.inter)
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_gate_up, act, ops.SWIGLU_BF16,
                           warm=rt.warm(self.w_down, 0, which=2))
        return self._down(act, ctx, residual, then_norm)

    def forward_prenormed(self, pre, ctx, residual=None, then_norm=None):
        """As forward_fused_norm, with the norm prepared by the kernel that last added into the stream."""
        rt = self.rt
        act = rt.empty(pre.x.shape[0], self.inter)
        ops.gemv_bf16(pre.x, self.w_gate_up, act, ops.SWIGLU_BF16, warm=rt.warm(self.w_down, 0, which=2), pre=pre)
        return self._down(act, ctx, residual, then_norm)

    def _down(self, act, ctx, residual, then_norm):
        rt = self.rt
        handoff = rt.handoff(then_norm, act.shape[0], self.hidden_size, self.inter) if residual is not None else None
        out = rt.linear(act, self.w_down, residual=residual, warm=rt.warm_after(ctx, which=4), handoff=handoff)
        return handoff if handoff is not None else out


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
