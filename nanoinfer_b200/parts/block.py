"""Arrangements: how a layer's norms, mixer and feed-forward are put together."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.registry import part, register_part


class PreNormBlock:
    """h += mixer(norm1(h)); h += ffn(norm2(h))  (src/model/llama.cpp:324-379).

    The residual stream h is FP32 and updated in place.  Each addition is fused into the
    norm that follows it, so a block takes the addition still pending from the block before
    and returns its own.
    """

    def __init__(self, layer_spec, hidden_size: int, weights_of, rt) -> None:
        """``weights_of(what)`` returns {slot: tensor} for what in
        "mixer_norm" | "mixer" | "ffn_norm" | "feed_forward"."""
        self.mixer_norm = part("norm", layer_spec.mixer_norm.kind)(
            layer_spec.mixer_norm, hidden_size, weights_of("mixer_norm"), rt)
        self.mixer = part("mixer", layer_spec.mixer.kind)(
            layer_spec.mixer, hidden_size, weights_of("mixer"), rt)
        self.ffn_norm = part("norm", layer_spec.ffn_norm.kind)(
            layer_spec.ffn_norm, hidden_size, weights_of("ffn_norm"), rt)
        self.feed_forward = part("feed_forward", layer_spec.feed_forward.kind)(
            layer_spec.feed_forward, hidden_size, weights_of("feed_forward"), rt)

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        x = self.mixer_norm.forward(h, delta)
        if getattr(self.mixer, "adds_into_residual", False):
            a = self.mixer.forward(x, ctx, cache, residual=h)     # may add in place and return None
        else:
            a = self.mixer.forward(x, ctx, cache)
        x = self.ffn_norm.forward(h, a)
        if getattr(self.feed_forward, "adds_into_residual", False):
            return self.feed_forward.forward(x, ctx, residual=h)
        return self.feed_forward.forward(x, ctx)


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)
