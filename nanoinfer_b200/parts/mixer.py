"""Token mixers.  The one built in is grouped-query attention over the paged cache."""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..config.model_config import ConfigError
from ..config.registry import part, register_part
from ..kernels import ops
from .base import PagedKVNeed, Part, StepPlan, WeightSlot


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
        self.position = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
        if self.position.rotary_dim > spec.head_dim:
            raise ConfigError("rotary_dim must not exceed head_dim")
        wq, wk = weights["q"], weights["k"]
        if self.position.rotary_dim > 0 and not self.position.interleaved:
            # Weights stored for "half" pairing (i, i + rot/2): reorder the rows of every head so
            # that the two elements of a rotary pair are neighbours.  Scores do not change (q and
            # k are permuted alike), every kernel then rotates adjacent pairs, and a 16-row tile
            # of the fused projection holds whole pairs.  (The reference's exporter does the same
            # to its weight file, tools/export_llama3.py:571-583.)
            wq = _pairs_adjacent(wq, spec.num_heads, spec.head_dim, self.position.rotary_dim)
            wk = _pairs_adjacent(wk, spec.num_kv_heads, spec.head_dim, self.position.rotary_dim)
        self.w_qkv = rt.weight(torch.cat([wq, wk, weights["v"]], dim=0))
        self.w_o = rt.weight(weights["o"])

    def cache_need(self):
        return PagedKVNeed(self.n_kv, self.head_dim, self.window)

    def weights_in_order(self) -> tuple:
        return (self.w_qkv, self.w_o)

    adds_into_residual = True   # forward() accepts residual= and may add its output there
    graph_safe = "all"          # everything that changes between steps is read from device memory

    # How the attention kernels split a step.  Requests that bring at most SHORT_PORTION tokens are
    # handled token by token by the split-K kernel (which fetches a token's last
    # ops.DECODE_FRESH_KEYS keys late, after the kernel that writes them); longer portions go to the
    # flash-style kernels in tiles of TILE_ROWS query rows, the tile with the most keys first.
    SHORT_PORTION = ops.DECODE_FRESH_KEYS
    TILE_ROWS = ops.PREFILL_TILE_ROWS

    @staticmethod
    def plan_step(q_lens: List[int], starts: List[int]) -> StepPlan:
        """dec_tokens: token indices of the short portions; long_tokens: of the long ones;
        tile_seq / tile_row0: request and first query row of each tile.  The arrays' sizes follow
        from q_lens alone; the tiles' order also from the cached lengths."""
        i32 = np.int32
        if max(q_lens) == 1:       # single tokens only: the kernels take tokens 0 .. n-1 as they come
            none = np.zeros(0, dtype=i32)
            return StepPlan({"dec_tokens": none, "long_tokens": none, "tile_seq": none, "tile_row0": none},
                            {"n_dec": len(q_lens), "n_tiles": 0})
        dec, long_tok, tiles = [], [], []
        at = 0
        for i, (ql, start) in enumerate(zip(q_lens, starts)):
            if ql <= PagedAttention.SHORT_PORTION:
                dec.extend(range(at, at + ql))
            else:
                long_tok.extend(range(at, at + ql))
                tiles.extend((start + r0, i, r0) for r0 in range(0, ql, PagedAttention.TILE_ROWS))
            at += ql
        tiles.sort(key=lambda x: -x[0])      # most keys first
        return StepPlan({"dec_tokens": np.asarray(dec, dtype=i32), "long_tokens": np.asarray(long_tok, dtype=i32),
                         "tile_seq": np.asarray([t[1] for t in tiles], dtype=i32),
                         "tile_row0": np.asarray([t[2] for t in tiles], dtype=i32)},
                        {"n_dec": len(dec), "n_tiles": len(tiles)})

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        """True if forward_fused_norm can take the residual stream itself (few rows, bfloat16)."""
        return self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    hands_off_norm = True       # forward_fused_norm / forward_prenormed accept then_norm= and may return its NormHandoff

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self._forward(x, None, 0.0, ctx, cache, residual)

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, cache, residual=None, then_norm=None):
        """As forward, with x = norm(h): the norm runs inside the projection kernel.  ``then_norm``:
        the norm that reads the stream next; where the output projection can prepare it, its
        NormHandoff is returned instead of None."""
        return self._forward(h, norm.gain, norm.eps, ctx, cache, residual, then_norm=then_norm)

    def forward_prenormed(self, pre, ctx, cache, residual=None, then_norm=None):
        """As forward_fused_norm, with the norm prepared by the kernel that last added into the stream."""
        return self._forward(pre.x, None, 0.0, ctx, cache, residual, then_norm=then_norm, pre=pre)

    def _forward(self, x, gain, eps, ctx, cache, residual, then_norm=None, pre=None):
        rt = self.rt
        n = x.shape[0]
        table = ctx.block_tables[cache.group]
        pos = self.position
        q = rt.empty(n, self.n_heads * self.head_dim)
        k_pages = cache.k_pages if cache.writable else None
        v_pages = cache.v_pages if cache.writable else None
        if rt.skinny(n, self.hidden_size):
            # decode: projection, rotation and cache write in one launch
            ops.gemv_qkv_rope(x, gain, eps, self.w_qkv, q, k_pages, v_pages, ctx.positions, ctx.seq_of_token,
                              table, pos.inv_freq, self.n_heads, self.n_kv, self.head_dim, pos.rotary_dim,
                              rt.page_size, pre=pre)
        elif rt.mid_batch(n, self.hidden_size, rt.MID_QKV) and self.head_dim % 2 == 0:
            # a middle batch: projection on the tensor cores with the weights on the tile's lanes,
            # rotation and cache write in its epilogue
            ops.gemm_swap_tc(x, self.w_qkv, q, ops.ROPE_KV,
                             rope=(ctx.positions, ctx.seq_of_token, table, pos.inv_freq, k_pages, v_pages, self.n_heads,
                                   self.n_kv, self.head_dim, pos.rotary_dim, rt.page_size))
        else:
            qkv = rt.linear(x, self.w_qkv)
            ops.rope_kv_write(qkv, q, k_pages, v_pages, ctx.positions, ctx.seq_of_token, table, pos.inv_freq,
                              self.n_heads, self.n_kv, self.head_dim, pos.rotary_dim, True, rt.page_size)
        att = rt.empty(n, self.n_heads * self.head_dim)
        self._attend(q, cache, att, ctx, table)
        if residual is not None and rt.mid_batch(n, self.n_heads * self.head_dim, rt.MID_OUT):
            ops.gemm_swap_tc(att, self.w_o, residual, ops.ADD_F32)       # added into the residual stream in the epilogue
            return None
        # the attention kernel asked for the head of the next matrix; this one goes on from there
        handoff = rt.handoff(then_norm, n, self.hidden_size, self.n_heads * self.head_dim) if residual is not None else None
        out = rt.linear(att, self.w_o, residual=residual, handoff=handoff,
                        warm=rt.warm_after(ctx, skip=rt.attention_share(ctx), which=1) if ctx.decode_only else None)
        return handoff if handoff is not None else out

    def _attend(self, q, cache, att, ctx, table) -> None:
        """Attention of every token of the step over its own request's pages.

        float32: the plain kernel.  bfloat16: single query tokens (and portions of at most
        two tokens) go to the split-K kernel, longer portions to the flash-style kernel;
        head sizes those do not take fall back to the plain kernel, never to a wrong result."""
        rt = self.rt
        common = (self.n_heads, self.n_kv, self.head_dim, rt.page_size, self.window, self.scale)
        n = q.shape[0]
        slopes = getattr(self.position, "head_slopes", None)
        if rt.dtype != torch.bfloat16 or slopes is not None:
            # float32, or a position encoding that acts on the scores (a bias slope[h] * (k_pos - q_pos)):
            # the plain kernel takes both; the tensor-core kernels know rotations only
            ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token,
                                  table, *common, head_slopes=slopes)
            return
        decode_ok = self.head_dim in ops.DECODE_HEAD_DIMS and self.n_heads // self.n_kv <= 16
        prefill_ok = self.head_dim % 16 == 0 and self.head_dim <= ops.PREFILL_MAX_HEAD_DIM
        plan = None if ctx.decode_only else ctx.plan_of(self)    # a step of single tokens needs no lists
        n_dec = n if plan is None else plan.scalars["n_dec"]
        dec_list = None if plan is None else plan.arrays["dec_tokens"]
        if n_dec > 0:
            if decode_ok and rt.balanced_attention(n_dec, self.n_kv, self.head_dim) and n_dec <= ops.DECODE_BALANCED_MAX_ITEMS:
                # many tokens: their keys dealt evenly over a fixed set of blocks, whatever their lengths
                scratch = rt.workspace("attention_decode_balanced_partials",
                                       ops.attention_decode_balanced_scratch(self.n_heads, self.n_kv, self.head_dim), torch.float32)
                tickets = rt.workspace("attention_decode_tickets", n_dec * self.n_kv, torch.int32, zero=True)
                ops.attention_decode_balanced(q, cache.k_pages, cache.v_pages, att, dec_list, n_dec, ctx.positions,
                                              ctx.seq_of_token, table, *common, scratch, tickets,
                                              warm=rt.warm_attention(self.w_o, ctx))
            elif decode_ok:
                splits = ops.decode_splits(n_dec, self.n_kv, self.head_dim, ctx.max_kv_len)
                scratch = rt.workspace("attention_decode_partials",
                                       n_dec * self.n_heads * splits * (self.head_dim + 2), torch.float32)
                tickets = rt.workspace("attention_decode_tickets", n_dec * self.n_kv, torch.int32, zero=True)
                ops.attention_decode(q, cache.k_pages, cache.v_pages, att, dec_list, n_dec, ctx.positions,
                                     ctx.seq_of_token, table, *common, splits, scratch, tickets,
                                     warm=rt.warm_attention(self.w_o, ctx))
            else:
                ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token,
                                      table, *common, token_list=dec_list)
        if plan is not None and plan.scalars["n_tiles"] > 0:
            if prefill_ok:
                ops.attention_prefill(q, cache.k_pages, cache.v_pages, att, plan.arrays["tile_seq"],
                                      plan.arrays["tile_row0"], plan.scalars["n_tiles"], ctx.cu_q, ctx.kv_len, table,
                                      *common)
            else:
                ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token,
                                      table, *common, token_list=plan.arrays["long_tokens"])


def _pairs_adjacent(w: torch.Tensor, n_heads: int, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """Rows i and i + rot/2 of every head become rows 2i and 2i + 1; rows beyond rot stay."""
    out_dim, in_dim = w.shape
    w = w.view(n_heads, head_dim, in_dim)
    rot = w[:, :rotary_dim].reshape(n_heads, 2, rotary_dim // 2, in_dim).transpose(1, 2)
    return torch.cat([rot.reshape(n_heads, rotary_dim, in_dim), w[:, rotary_dim:]], dim=1).reshape(out_dim, in_dim)


register_part("mixer", "attention", PagedAttention, replace=True)
