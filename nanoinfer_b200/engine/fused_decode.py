"""The fused decode step: when a model is a plain stack of pre-norm blocks with paged attention
and a SwiGLU feed-forward of uniform sizes, a step of up to 8 single tokens runs as ONE persistent
kernel (csrc/decode_fused.cu) instead of five launches per layer.

This is an optimisation over the assembled parts, not a part: it looks at the blocks that the
registry built, takes their weights and constants as they are, and declines (returns None) for
anything else - another mixer or feed-forward, layers of different sizes, float32, more rows.
The per-part path stays the reference for it (tests/test_gpu_fused_decode.py compares the two).
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional

import torch

from ..kernels import ops
from ..parts.block import PreNormBlock
from ..parts.embedding import TableEmbedding
from ..parts.head import LinearHead
from ..parts.feed_forward import SwiGLU
from ..parts.mixer import PagedAttention
from ..parts.norm import RMSNorm


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class FusedDecode:
    """Built once per model and cache; ``run(ctx)`` launches the kernel for a step of single tokens."""

    @classmethod
    def build(cls, model, caches) -> Optional["FusedDecode"]:
        rt, cfg = model.rt, model.config
        if rt.dtype != torch.bfloat16 or not getattr(rt, "fused_decode", True):
            return None
        if type(model.final_norm) is not RMSNorm or not cfg.schedule:
            return None
        if type(model.embedding) is not TableEmbedding or type(model.head) is not LinearHead:
            return None
        blocks = [model.blocks[run.layer] for run in cfg.schedule]
        for b in blocks:
            if type(b) is not PreNormBlock or type(b.mixer) is not PagedAttention or type(b.feed_forward) is not SwiGLU:
                return None
            if type(b.mixer_norm) is not RMSNorm or type(b.ffn_norm) is not RMSNorm or not b.feed_forward.blocked:
                return None
        first = blocks[0].mixer
        for b in blocks:
            m = b.mixer
            same = (m.n_heads, m.n_kv, m.head_dim, m.window, m.scale, m.position.rotary_dim) == \
                   (first.n_heads, first.n_kv, first.head_dim, first.window, first.scale, first.position.rotary_dim)
            if not same or b.feed_forward.inter != blocks[0].feed_forward.inter:
                return None
            if m.position.rotary_dim > 0 and not torch.equal(m.position.inv_freq, first.position.inv_freq):
                return None
            if getattr(m.position, "head_slopes", None) is not None:
                return None
        groups = {c.group for c in caches if c is not None}
        if any(c is None or c.k_pages is None for c in caches) or max(groups) >= ops.FUSED_MAX_GROUPS:
            return None
        if not ops.decode_fused_supports(1, cfg.hidden_size, first.n_heads, first.n_kv, first.head_dim,
                                         first.position.rotary_dim, blocks[0].feed_forward.inter, cfg.vocab_size,
                                         rt.page_size):
            return None
        return cls(model, blocks, caches)

    def __init__(self, model, blocks, caches) -> None:
        rt, cfg = model.rt, model.config
        self.model, self.rt = model, rt
        mixer, ffn = blocks[0].mixer, blocks[0].feed_forward
        self.max_rows = ops.decode_fused_lib().ni_decode_fused_max_rows()
        layers = (ops.FusedLayer * len(blocks))()
        for rec, b, cache in zip(layers, blocks, caches):
            rec.w_qkv, rec.w_o = b.mixer.w_qkv.data_ptr(), b.mixer.w_o.data_ptr()
            rec.w_gate_up, rec.w_down = b.feed_forward.w_gate_up.data_ptr(), b.feed_forward.w_down.data_ptr()
            rec.gain_mixer, rec.gain_ffn = b.mixer_norm.gain.data_ptr(), b.ffn_norm.gain.data_ptr()
            rec.k_pages, rec.v_pages = cache.k_pages.data_ptr(), cache.v_pages.data_ptr()
            rec.eps_mixer, rec.eps_ffn = b.mixer_norm.eps, b.ffn_norm.eps
            rec.write_cache, rec.group = int(cache.writable), cache.group
        raw = torch.frombuffer(bytearray(bytes(layers)), dtype=torch.uint8)
        self.layers = raw.to(rt.device)
        dev, m = rt.device, self.max_rows
        q_dim = mixer.n_heads * mixer.head_dim
        self.h = torch.zeros(m, cfg.hidden_size, dtype=torch.float32, device=dev)
        self.q = torch.zeros(m, q_dim, dtype=torch.bfloat16, device=dev)
        self.att = torch.zeros(m, q_dim, dtype=torch.bfloat16, device=dev)
        self.act = torch.zeros(m, ffn.inter, dtype=torch.bfloat16, device=dev)
        self.logits = torch.zeros(m, cfg.vocab_size, dtype=torch.float32, device=dev)
        self.partials = torch.zeros(ops.decode_fused_partials(m, mixer.n_kv, mixer.head_dim), dtype=torch.float32, device=dev)
        self.tickets = torch.zeros(m * mixer.n_kv, dtype=torch.int32, device=dev)
        self.barrier = torch.zeros(1, dtype=torch.int32, device=dev)
        self.error = ops.error_word(dev)
        p = self.params = ops.FusedParams()
        p.layers, p.inv_freq = self.layers.data_ptr(), mixer.position.inv_freq.data_ptr()
        p.embedding, p.lm_head = model.embedding.table.data_ptr(), model.head.weight.data_ptr()
        p.gain_final, p.eps_final = model.final_norm.gain.data_ptr(), model.final_norm.eps
        p.h, p.q, p.att, p.act, p.logits = (t.data_ptr() for t in (self.h, self.q, self.att, self.act, self.logits))
        p.partials, p.tickets, p.barrier, p.error = (t.data_ptr() for t in (self.partials, self.tickets, self.barrier, self.error))
        p.wait_limit = 0
        p.n_layers, p.d = len(blocks), cfg.hidden_size
        p.n_q_heads, p.n_kv_heads, p.head_dim = mixer.n_heads, mixer.n_kv, mixer.head_dim
        p.rotary_dim, p.inter, p.vocab, p.page_size = mixer.position.rotary_dim, ffn.inter, cfg.vocab_size, rt.page_size
        p.window = int(mixer.window) if mixer.window else 0
        p.scale_log2e = mixer.scale * math.log2(math.e)
        p.skip_arrive_at = -1
        self.n_groups = max(c.group for c in caches) + 1

    def takes(self, ctx) -> bool:
        return ctx.decode_only and 0 < ctx.n_tokens <= self.max_rows and ctx.n_logit_rows <= self.max_rows

    def run(self, ctx) -> torch.Tensor:
        """Launch the step; returns FP32 logits [wanted rows, vocab] (a view of a buffer of this
        object, valid until the next step)."""
        p = self.params
        p.M, p.R = ctx.n_tokens, ctx.n_logit_rows
        p.tokens, p.positions, p.seq_of_token = ctx.tokens.data_ptr(), ctx.positions.data_ptr(), ctx.seq_of_token.data_ptr()
        p.logit_rows = ctx.logit_rows.data_ptr()
        for g in range(self.n_groups):
            p.tables[g] = ctx.block_tables[g].data_ptr()
            p.bt_stride[g] = ctx.block_tables[g].shape[1]
        ops.decode_fused(p)
        return self.logits[:ctx.n_logit_rows]
