"""The decoder assembled from a configuration: embedding, scheduled blocks, final norm,
output projection.  Which parts a layer has, and in which order layers run, is data.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import registry
from ..config.model_config import ModelConfig
from ..kernels import ops
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
        self.embedding = rt.weight(by_scope[("embedding",)]["weight"])
        self.blocks = []
        for i, layer in enumerate(config.layers):
            cls = registry.part("arrangement", layer.arrangement)
            self.blocks.append(cls(layer, d, lambda what, i=i: by_scope.get(("layer", i, what), {}), rt))
        self.final_norm = registry.part("norm", config.final_norm.kind)(
            config.final_norm, d, by_scope.get(("final_norm",), {}), rt)
        # a tied output projection is the embedding table itself: one device copy
        # (the reference uploads the shared matrix twice, src/model/llama.cpp:576-578,652-657)
        self.lm_head = (self.embedding if config.tie_word_embeddings
                        else rt.weight(by_scope[("lm_head",)]["weight"]))
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
        ops.embedding(ctx.tokens, self.embedding, h)
        delta = None
        for r, run in enumerate(cfg.schedule):
            delta = self.blocks[run.layer].forward(h, delta, ctx, caches[r])
        if ctx.n_logit_rows == 0:
            return rt.empty(0, cfg.vocab_size, dtype=torch.float32)
        norm = self.final_norm
        if (delta is None and rt.skinny(ctx.n_logit_rows, cfg.hidden_size) and hasattr(norm, "gain")
                and hasattr(norm, "eps")):
            # few rows: final norm, row selection and output projection in one launch
            logits = rt.empty(ctx.n_logit_rows, cfg.vocab_size, dtype=torch.float32)
            ops.gemv_norm_bf16(h, norm.gain, norm.eps, ctx.logit_rows, self.lm_head, logits, ops.STORE_F32)
            return logits
        x = norm.forward(h, delta, rows=ctx.logit_rows)
        return rt.linear(x, self.lm_head, out_dtype=torch.float32)
