"""The decoder assembled from a configuration: embedding, scheduled blocks, final norm,
output projection.  Which parts a layer has, and in which order layers run, is data.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import registry
from ..config.model_config import ModelConfig
from ..weights.plan import tensor_plan


class DecoderModel:
    def __init__(self, config: ModelConfig, weights: Dict[str, torch.Tensor], rt) -> None:
        self.config, self.rt = config, rt
        arch = registry.architecture(config.architecture)
        d = config.hidden_size
        by_scope: Dict[tuple, Dict[str, torch.Tensor]] = {}
        for p in tensor_plan(config):
            if p.name not in weights:
                raise KeyError(f"weight '{p.name}' is missing")
            by_scope.setdefault(p.scope, {})[p.slot] = weights[p.name]
        emb = config.embedding_spec()
        self.embedding = registry.part("embedding", emb.kind)(emb, d, by_scope.get(("embedding",), {}), rt)
        self.blocks = []
        for i, layer in enumerate(config.layers):
            cls = registry.part("arrangement", layer.arrangement)
            self.blocks.append(cls(layer, d, lambda what, i=i: by_scope.get(("layer", i, what), {}), rt))
        self.final_norm = registry.part("norm", config.final_norm.kind)(
            config.final_norm, d, by_scope.get(("final_norm",), {}), rt)
        head = config.head_spec()
        head_weights = dict(by_scope.get(("lm_head",), {}))
        if head.tied:
            table = getattr(self.embedding, "table", None)
            if table is None:
                raise ValueError(f"a tied head needs an embedding with a table; '{emb.kind}' has none")
            head_weights["weight"] = table      # the embedding's own device copy
        self.head = registry.part("head", head.kind)(head, d, head_weights, rt)
        # per scheduled run: the matrices read after it (the next run's, then the head's)
        order = [tuple(getattr(self.blocks[run.layer], "weights_in_order", tuple)()) for run in config.schedule]
        order.append(tuple(self.head.weights_in_order()))
        self._read_after = [order[r + 1] for r in range(len(config.schedule))]
        # per scheduled run: the norm that reads the stream after it, if it can come prepared (see
        # NormHandoff); the head keeps its own fused norm, so the last run hands nothing over
        firsts = [getattr(self.blocks[run.layer], "first_norm", lambda: None)() for run in config.schedule]
        self._norm_after = firsts[1:] + [None]
        self._fused = False      # the fused decode step: not looked at yet / None (does not apply) / the object

    def cache_needs(self) -> List[Optional[object]]:
        """Per schedule entry: what its mixer keeps between steps (None if it reads
        another run's cache or keeps nothing)."""
        needs = []
        for run in self.config.schedule:
            if run.cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.blocks[run.layer].mixer.cache_need())
        return needs

    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step's tokens through every scheduled layer; return FP32 logits
        [len(ctx.logit_rows), vocab] for the wanted rows only."""
        rt, cfg = self.rt, self.config
        if ctx.decode_only and self._fused is not None:
            if self._fused is False:
                from .fused_decode import FusedDecode
                self._fused = FusedDecode.build(self, caches)
            if self._fused is not None and self._fused.takes(ctx):
                return self._fused.run(ctx)      # a step of a few single tokens: one persistent kernel
        h = rt.empty(ctx.n_tokens, cfg.hidden_size, dtype=torch.float32)
        self.embedding.forward(ctx.tokens, h)
        delta = None
        for r, run in enumerate(cfg.schedule):
            ctx.read_after, ctx.norm_after = self._read_after[r], self._norm_after[r]
            delta = self.blocks[run.layer].forward(h, delta, ctx, caches[r])
        ctx.read_after, ctx.norm_after = (), None
        return self.head.forward(h, delta, self.final_norm, ctx)
