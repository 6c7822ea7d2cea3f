"""The sampler: one row of FP32 logits per request -> one token id per request.

All rows greedy: one arg-max launch (the reference's fast path,
src/sampler/configurable_sampler.cpp:89-100).  Otherwise: repetition penalty on the rows that
ask for it, then one launch that handles every row by its own parameters (greedy rows
included, so no host round trip patches them afterwards as in
src/sampler/configurable_sampler.cpp:135-173).

The uniform number of a draw depends only on (seed, index of the generated token), so a
request's tokens do not depend on what else is in the batch.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, vocab_size: int, device) -> None:
        self.vocab_size = vocab_size
        self.device = device
        self.h2d_bytes = 0     # bytes of per-row parameters copied to the device so far
        self._dev = None       # the parameters' place on the device, and the pinned buffers they come from
        self._host, self._events, self._used, self._next = [], [], [], 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               token_indices: Sequence[int],
               generated: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """logits float32 [R, V] (modified in place when a penalty applies); ``seeds[r]`` the
        request's resolved seed (>= 0); ``token_indices[r]`` how many tokens the request has
        generated before this one; ``generated[r]`` its generated ids (for the penalty).
        Returns int32 [R] on the device."""
        n = logits.shape[0]
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if n == 0:
            return out
        if all(p.use_greedy() for p in params):
            ops.argmax(logits, out)
            return out
        if generated is not None and any(p.use_repetition_penalty() for p in params):
            uniq: List[List[int]] = [sorted(set(g)) if p.use_repetition_penalty() else []
                                     for p, g in zip(params, generated)]
            width = max(len(u) for u in uniq)
            if width > 0:
                ids = np.full((n, width), -1, dtype=np.int32)
                for r, u in enumerate(uniq):
                    ids[r, :len(u)] = u
                pen = np.asarray([p.repetition_penalty for p in params], dtype=np.float32)
                ops.repetition_penalty(logits, torch.from_numpy(ids).to(logits.device),
                                       torch.from_numpy(pen).to(logits.device))
        seed_t, count_t, temp_t, top_p_t, top_k_t = self._upload(logits.device, params, seeds, token_indices)
        ops.sample(logits, out, temp_t, top_k_t, top_p_t, seed_t, count_t)
        return out

    # Per-row parameters travel in ONE copy from pinned memory (a copy from pageable memory would
    # hold the host until the stream has run everything before it - the whole step).  Words of 4
    # bytes: seeds int64 [n], token counters int64 [n], temperature, top_p float32 [n], top_k int32 [n].
    _RING = 4

    def _upload(self, device, params, seeds, token_indices):
        n = len(params)
        words = 7 * n
        if self._dev is None or self._dev.numel() < words:
            cap = max(7 * 64, 2 * words)
            self._dev = torch.empty(cap, dtype=torch.int32, device=device)
            pin = device.type == "cuda"
            self._host = [torch.empty(cap, dtype=torch.int32, pin_memory=pin) for _ in range(self._RING)]
            self._events = [torch.cuda.Event() if pin else None for _ in range(self._RING)]
            self._used = [False] * self._RING
        i = self._next
        self._next = (i + 1) % self._RING
        if self._used[i] and self._events[i] is not None:
            self._events[i].synchronize()          # the copy that read this buffer last has run
        h = self._host[i][:words].numpy()
        h[0:2 * n].view(np.int64)[:] = np.asarray(seeds, dtype=np.uint64).view(np.int64)
        h[2 * n:4 * n].view(np.int64)[:] = np.asarray(token_indices, dtype=np.int64)
        h[4 * n:5 * n].view(np.float32)[:] = [p.temperature for p in params]
        h[5 * n:6 * n].view(np.float32)[:] = [p.top_p for p in params]
        h[6 * n:7 * n] = [p.top_k for p in params]
        d = self._dev[:words]
        d.copy_(self._host[i][:words], non_blocking=True)
        if self._events[i] is not None:
            self._events[i].record()
            self._used[i] = True
        self.h2d_bytes += 4 * words
        return (d[0:2 * n].view(torch.int64), d[2 * n:4 * n].view(torch.int64), d[4 * n:5 * n].view(torch.float32),
                d[5 * n:6 * n].view(torch.float32), d[6 * n:7 * n])
