"""Embeddings: how a step's token ids become rows of the FP32 residual stream."""
from __future__ import annotations

from ..config.registry import register_part
from ..kernels import ops
from .base import Part, WeightSlot


class TableEmbedding(Part):
    """Row ``id`` of a [vocab, hidden] table, widened to FP32
    (src/op/kernels/cuda/embedding_kernel.cu:7-31; the reference keeps the stream in the weights'
    precision, here it is FP32 from the first row on).

    ``table`` is the matrix on the device in the compute dtype; a tied head reads it too."""

    graph_safe = "all"

    @staticmethod
    def weight_slots(spec, hidden_size):
        return {"weight": WeightSlot((spec.vocab_size, hidden_size))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.table = rt.weight(weights["weight"])

    def forward(self, tokens, h) -> None:
        """tokens int32 [T] on the device; fills h [T, hidden] FP32."""
        ops.embedding(tokens, self.table, h)


register_part("embedding", "table", TableEmbedding, replace=True)
