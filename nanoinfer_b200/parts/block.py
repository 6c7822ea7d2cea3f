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

    def weights_in_order(self) -> tuple:
        return tuple(getattr(self.mixer, "weights_in_order", tuple)()) + tuple(getattr(self.feed_forward, "weights_in_order", tuple)())

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        n = h.shape[0]
        mixer, ffn = self.mixer, self.feed_forward
        after = ctx.read_after                       # what runs after this block
        ctx.read_after = tuple(getattr(ffn, "weights_in_order", tuple)()) + tuple(after)   # ... after the mixer
        try:
            a = self._mix(h, delta, ctx, cache, n)
        finally:
            ctx.read_after = after
        if a is None and _fuses(ffn, self.ffn_norm, n):
            return ffn.forward_fused_norm(h, self.ffn_norm, ctx, residual=h)
        x = self.ffn_norm.forward(h, a)
        if getattr(ffn, "adds_into_residual", False):
            return ffn.forward(x, ctx, residual=h)
        return ffn.forward(x, ctx)

    def _mix(self, h, delta, ctx, cache, n):
        mixer = self.mixer
        if delta is None and _fuses(mixer, self.mixer_norm, n):
            a = mixer.forward_fused_norm(h, self.mixer_norm, ctx, cache, residual=h)
        else:
            x = self.mixer_norm.forward(h, delta)
            if getattr(mixer, "adds_into_residual", False):
                a = mixer.forward(x, ctx, cache, residual=h)     # may add in place and return None
            else:
                a = mixer.forward(x, ctx, cache)
        return a


def _fuses(part_obj, norm, n_rows: int) -> bool:
    """A mixer or feed-forward may offer forward_fused_norm(h, norm, ...): it then reads the
    residual stream itself and runs the norm inside its first kernel."""
    return hasattr(part_obj, "forward_fused_norm") and part_obj.can_fuse_norm(norm, n_rows)


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)
