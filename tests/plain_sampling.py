"""Plain next-token selection for the tests: arg-max, repetition penalty, temperature, top-k,
top-p and the multinomial draw, written from the reference's formulas with float64 sums.

Order of operations as in src/sampler/configurable_sampler.cpp:102-133: penalty, then
temperature, then top-k/top-p filtering, softmax and the draw.
"""
import torch

M32 = 0xFFFFFFFF


def philox_first_word(seed: int, counter: int) -> int:
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw 2011), key = seed, counter = (counter, 0)."""
    c = [counter & M32, (counter >> 32) & M32, 0, 0]
    k = [seed & M32, (seed >> 32) & M32]
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & M32, p1 & M32, ((p0 >> 32) ^ c[3] ^ k[1]) & M32, p0 & M32]
        k = [(k[0] + 0x9E3779B9) & M32, (k[1] + 0xBB67AE85) & M32]
    return c[0]


def uniform(seed: int, counter: int) -> float:
    return ((philox_first_word(seed, counter) >> 8) + 0.5) / 16777216.0


def penalise(logits: torch.Tensor, generated, penalty: float) -> torch.Tensor:
    """l > 0 ? l / p : l * p on every generated id, once per id
    (src/op/kernels/cpu/sampling_kernel.cpp:27-56)."""
    out = logits.clone().float()
    if penalty != 1.0:
        for t in set(generated):
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


# Two selections that differ by less than this share of the total mass cannot be told apart:
# FP32 exp is good to about 1e-7 relative per element, and the kernel sums mass in fixed point
# with 2^-38 per element truncated (at most 5e-7 of the total for 128k elements).
ROUNDING = 1e-6


def sample(logits, temperature, top_k=-1, top_p=1.0, repetition_penalty=1.0, generated=(), seed=0, index=0,
           rounding=ROUNDING):
    """Returns (token, acceptable, cut_margin).  ``acceptable`` is the set of ids the draw
    reaches when its target moves by +-``rounding`` of the total mass (usually just {token});
    ``cut_margin`` is the distance of the top-p cut to the point where one more or one fewer
    token would be kept, as a share of the total mass (1.0 without top-p)."""
    l = penalise(logits, generated, repetition_penalty)
    if temperature <= 0:
        t = int(torch.argmax(l))
        return t, {t}, 1.0
    z = l * torch.tensor(1.0 / temperature, dtype=torch.float32)         # scaling (sampling_kernel.cpp:67-85)
    V = z.numel()
    kept = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.sort(z, descending=True).values[top_k - 1]
        kept = z >= kth                                                  # top-k (:131-140), ties kept
    e = torch.exp(z - z.max()).double()                                  # softmax numerator (:143-153)
    e[~kept] = 0.0
    cut_margin = 1.0
    if 0.0 < top_p < 1.0:
        order = torch.argsort(e, descending=True, stable=True)
        cums = torch.cumsum(e[order], 0)
        total = e.sum()
        idx = int(torch.nonzero(cums > top_p * total)[0])                # first prefix above p (:156-166)
        thr = e[order][idx]
        kept &= e >= thr
        below = cums[idx - 1] if idx > 0 else torch.tensor(0.0, dtype=torch.float64)
        cut_margin = float(min(abs(cums[idx] - top_p * total), abs(below - top_p * total)) / total)
        e[~kept] = 0.0
    total = e.sum()
    target = uniform(seed, index) * total
    cdf = torch.cumsum(e, 0)                                             # vocabulary order
    tok = int(torch.nonzero(cdf > target)[0])
    lo = int(torch.nonzero(cdf > max(target - rounding * total, 0.0))[0])
    hi_hits = torch.nonzero(cdf > target + rounding * total)
    hi = int(hi_hits[0]) if hi_hits.numel() else tok
    acceptable = {i for i in range(lo, hi + 1) if e[i] > 0}
    return tok, acceptable, cut_margin
