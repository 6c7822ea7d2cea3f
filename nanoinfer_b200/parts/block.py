"""Arrangements: how a layer's norms, mixer and feed-forward are put together."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.registry import part, register_part
from ..kernels.ops import NormHandoff


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

    def first_norm(self):
        """The norm that reads the residual stream first, if its reader (the mixer) can take it
        prepared by the kernel that last added into the stream (a NormHandoff); else None."""
        return self.mixer_norm if hasattr(self.mixer, "forward_prenormed") else None

    def forward(self, h: torch.Tensor, delta, ctx, cache):
        """``delta``: what the block before left - None, an addition still pending on the stream, or a
        NormHandoff (the stream is up to date and this block's first norm comes prepared).  Returns
        the same for the block after."""
        n = h.shape[0]
        mixer, ffn = self.mixer, self.feed_forward
        pre = None
        if isinstance(delta, NormHandoff):
            pre, delta = delta, None
            if pre.norm is not self.mixer_norm or not hasattr(mixer, "forward_prenormed"):
                pre = None                              # not for this block's norm: it is computed as usual
        after = ctx.read_after                       # what runs after this block
        ctx.read_after = tuple(getattr(ffn, "weights_in_order", tuple)()) + tuple(after)   # ... after the mixer
        # the norms that may be handed from kernel to kernel: this block's second one, the next block's first
        to_ffn = self.ffn_norm if hasattr(ffn, "forward_prenormed") and _fuses(ffn, self.ffn_norm, n) else None
        try:
            a = self._mix(h, delta, pre, ctx, cache, n, to_ffn)
        finally:
            ctx.read_after = after
        then = ctx.norm_after if getattr(ffn, "hands_off_norm", False) else None
        if isinstance(a, NormHandoff):
            return ffn.forward_prenormed(a, ctx, residual=h, then_norm=then)
        if a is None and _fuses(ffn, self.ffn_norm, n):
            if then is not None:
                return ffn.forward_fused_norm(h, self.ffn_norm, ctx, residual=h, then_norm=then)
            return ffn.forward_fused_norm(h, self.ffn_norm, ctx, residual=h)
        x = self.ffn_norm.forward(h, a)
        if getattr(ffn, "adds_into_residual", False):
            return ffn.forward(x, ctx, residual=h)
        return ffn.forward(x, ctx)

    def _mix(self, h, delta, pre, ctx, cache, n, to_ffn):
        mixer = self.mixer
        then = {"then_norm": to_ffn} if to_ffn is not None and getattr(mixer, "hands_off_norm", False) else {}
        if pre is not None:
            return mixer.forward_prenormed(pre, ctx, cache, residual=h, **then)
        if delta is None and _fuses(mixer, self.mixer_norm, n):
            a = mixer.forward_fused_norm(h, self.mixer_norm, ctx, cache, residual=h, **then)
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
