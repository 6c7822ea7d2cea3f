"""Token mixers.  The one built in is grouped-query attention over the paged cache."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.model_config import ConfigError
from ..config.registry import part, register_part
from ..kernels import ops
from .base import PagedKVNeed, Part, WeightSlot


class PagedAttention(Part):
    """Grouped-query attention: fused QKV projection, position encoding + cache write,
    attention over this request's pages, output projection.

    The reference runs three projections, RoPE, a cache write and one of two attention
    paths chosen by a whole-batch prefill flag (src/op/attention.cpp:101-198,
    src/model/llama.cpp:327-356).  Here a step may mix portions of prompts and single
    decoded tokens; the kernels find each token's request through the step context.
    """

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        q, kv = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return {"q": WeightSlot((q, hidden_size)), "k": WeightSlot((kv, hidden_size)),
                "v": WeightSlot((kv, hidden_size)), "o": WeightSlot((hidden_size, q))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        if spec.num_heads % spec.num_kv_heads:
            raise ConfigError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim % 16 or not 16 <= spec.head_dim <= 256:
            raise ConfigError(f"head_dim {spec.head_dim} is not supported: the attention kernels "
                              f"take multiples of 16 from 16 to 256")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError("an attention window must be positive")
        self.n_heads, self.n_kv, self.head_dim = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.window = spec.window
        self.scale = float(spec.softmax_scale)
        self.w_qkv = rt.weight(torch.cat([weights["q"], weights["k"], weights["v"]], dim=0))
        self.w_o = rt.weight(weights["o"])
        self.position = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
        if self.position.rotary_dim > spec.head_dim:
            raise ConfigError("rotary_dim must not exceed head_dim")

    def cache_need(self):
        return PagedKVNeed(self.n_kv, self.head_dim, self.window)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        rt = self.rt
        n = x.shape[0]
        qkv = rt.linear(x, self.w_qkv)
        q = rt.empty(n, self.n_heads * self.head_dim)
        table = ctx.block_tables[cache.group]
        pos = self.position
        ops.rope_kv_write(qkv, q, cache.k_pages if cache.writable else None,
                          cache.v_pages if cache.writable else None, ctx.positions,
                          ctx.seq_of_token, table, pos.inv_freq, self.n_heads, self.n_kv,
                          self.head_dim, pos.rotary_dim, pos.interleaved, rt.page_size)
        att = rt.empty(n, self.n_heads * self.head_dim)
        ops.attention(q, cache.k_pages, cache.v_pages, att, ctx, table, self.n_heads, self.n_kv,
                      self.head_dim, rt.page_size, self.window, self.scale)
        return rt.linear(att, self.w_o)


register_part("mixer", "attention", PagedAttention, replace=True)
