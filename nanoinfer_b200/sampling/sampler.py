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
        f = np.asarray([[p.temperature, p.top_p] for p in params], dtype=np.float32)
        k = np.asarray([p.top_k for p in params], dtype=np.int32)
        sc = np.asarray([[s, c] for s, c in zip(seeds, token_indices)], dtype=np.uint64)
        dev = logits.device
        self.h2d_bytes += f.nbytes + k.nbytes + sc.nbytes
        ft = torch.from_numpy(f).to(dev)
        sct = torch.from_numpy(sc.view(np.int64)).to(dev)
        ops.sample(logits, out, ft[:, 0].contiguous(), torch.from_numpy(k).to(dev),
                   ft[:, 1].contiguous(), sct[:, 0].contiguous(), sct[:, 1].contiguous())
        return out
