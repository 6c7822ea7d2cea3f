"""Heads: how the wanted rows of the residual stream become FP32 logits."""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import Part, WeightSlot


class LinearHead(Part):
    """Final norm of the wanted rows, then the product with a [vocab, hidden] matrix
    (src/model/llama.cpp:381-389).  A tied head stores no matrix: it is handed the embedding's
    table as its "weight" (one device copy; the reference uploads the shared matrix twice,
    src/model/llama.cpp:576-578,652-657)."""

    graph_safe = "all"

    @staticmethod
    def weight_slots(spec, hidden_size):
        return {} if spec.tied else {"weight": WeightSlot((spec.vocab_size, hidden_size))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.vocab_size = spec.vocab_size
        self.weight = rt.weight(weights["weight"])     # already on the device when it is the embedding's table

    def weights_in_order(self) -> tuple:
        return (self.weight,)

    def forward(self, h, delta, norm, ctx) -> torch.Tensor:
        """h FP32 [T, hidden] with ``delta`` still to be added (or None); returns FP32 logits
        [ctx.n_logit_rows, vocab] for rows ctx.logit_rows."""
        rt = self.rt
        if ctx.n_logit_rows == 0:
            return rt.empty(0, self.vocab_size, dtype=torch.float32)
        if delta is None and rt.skinny(ctx.n_logit_rows, self.hidden_size) and rt.fuses_norm(norm):
            # few rows: final norm, row selection and output projection in one launch
            logits = rt.empty(ctx.n_logit_rows, self.vocab_size, dtype=torch.float32)
            ops.gemv_norm_bf16(h, norm.gain, norm.eps, ctx.logit_rows, self.weight, logits, ops.STORE_F32)
            return logits
        x = norm.forward(h, delta, rows=ctx.logit_rows)
        return rt.linear(x, self.weight, out_dtype=torch.float32)


register_part("head", "linear", LinearHead, replace=True)
