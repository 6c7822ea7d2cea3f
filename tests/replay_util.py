"""Trace builders and comparison helpers for the replay tests.

A trace is a list of steps {"step", "entries": [{"id", "tokens", "want"}], "end"}, the
format bin/trace_run reads.  Each builder cuts the same requests differently; the logits of
a (request, position) must not depend on the cut.
"""
import torch

import plain_llama as plain


def whole(requests):
    """Each request alone and whole, logits at every position."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_by_token(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        s += 1
        for j in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def ragged(requests, sizes=(7, 2, 19, 3, 2, 33, 5, 2, 64, 2, 11)):
    """Portions of changing size, down to two tokens, one request at a time."""
    steps, s = [], 0
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
            s += 1
    return steps


def mixed(requests, max_live=4, prefill_sizes=(5, 2, 13, 3, 24, 2), tail=6, seed=0):
    """Up to ``max_live`` live requests; a request is prefilled in portions and its last
    ``tail`` tokens are fed one by one, so portions of some stand beside single tokens of
    others.  Requests are admitted as earlier ones end, so their pages are used again.
    Every few steps one live request sits a step out."""
    g = torch.Generator().manual_seed(seed)
    waiting = list(requests.items())
    live = {}   # rid -> [tokens, fed, portion counter]
    steps, s = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, int(torch.randint(0, 6, (1,), generator=g))]
        entries, end = [], []
        skip = None
        if len(live) > 1 and s % 3 == 2:
            skip = list(live)[int(torch.randint(0, len(live), (1,), generator=g))]
        for rid, st in live.items():
            if rid == skip:
                continue
            toks, fed, k = st
            left = len(toks) - fed
            if left <= tail:
                n = 1
            else:
                n = min(prefill_sizes[k % len(prefill_sizes)], left - tail) if left - tail >= 2 else left - tail
                st[2] += 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            st[1] += n
            if st[1] == len(toks):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append({"step": s, "entries": entries, "end": end})
        s += 1
    return steps


def wide(requests, n_live, tail=8, joiners=2, per_prefill_step=6):
    """Many requests decoding together.  ``requests`` holds 2 * n_live + joiners requests:
    a first group of ``n_live`` is prefilled (several whole prompts per step), then decodes its
    last ``tail`` tokens together, one step of n_live single tokens after the other; beside some of
    those steps the ``joiners`` bring their prompts in portions and then decode along.  When the
    first group has ended, a second group of n_live takes over its pages (its prompts run beside
    the joiners' single tokens) and decodes together with the joiners."""
    items = list(requests.items())
    assert len(items) == 2 * n_live + joiners
    first, late, second = items[:n_live], items[n_live:n_live + joiners], items[n_live + joiners:]
    fed = {rid: 0 for rid, _ in items}
    steps = []

    def portion(rid, toks, n):
        a = fed[rid]
        fed[rid] = a + n
        return {"id": rid, "tokens": toks[a:a + n], "want": list(range(n))}

    def push(entries):
        end = [e["id"] for e in entries if fed[e["id"]] == len(requests[e["id"]])]
        steps.append({"step": len(steps), "entries": entries, "end": end})

    def prefill(group, beside=()):
        for at in range(0, len(group), per_prefill_step):
            entries = [portion(rid, toks, len(toks) - tail) for rid, toks in group[at:at + per_prefill_step]]
            entries += [portion(rid, toks, 1) for rid, toks in beside if fed[rid] < len(toks)]
            push(entries)

    def decode(group, others):
        """All of ``group`` one token per step until it ends; ``others`` bring portions of 2..9
        tokens in every second step until only their tail is left, then single tokens."""
        k = 0
        while any(fed[rid] < len(toks) for rid, toks in group):
            entries = [portion(rid, toks, 1) for rid, toks in group if fed[rid] < len(toks)]
            for j, (rid, toks) in enumerate(others):
                left = len(toks) - fed[rid]
                if left <= 0:
                    continue
                if left > tail:
                    if k % 2 == j % 2:
                        entries.append(portion(rid, toks, min(2 + (3 * k + 5 * j) % 8, left - tail)))
                else:
                    entries.append(portion(rid, toks, 1))
            push(entries)
            k += 1

    prefill(first)
    decode(first, late)
    prefill(second, beside=late)
    decode(second, late)
    decode([x for x in late if fed[x[0]] < len(x[1])], [])
    assert all(fed[rid] == len(toks) for rid, toks in items)
    return steps


def max_live_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def run_trace(runner, steps):
    """Drive a ModelRunner through a trace; returns {(id, position): logits row (CPU)}."""
    from nanoinfer_b200.engine import StepEntry
    fed, out = {}, {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        if entries:
            logits = runner.step(entries).cpu()
            r = 0
            for e in st["entries"]:
                base = fed.get(e["id"], 0)
                for wpos in e["want"]:
                    out[(e["id"], base + wpos)] = logits[r]
                    r += 1
                fed[e["id"]] = base + len(e["tokens"])
            assert r == logits.shape[0]
        for rid in st["end"]:
            runner.end(rid)
            fed.pop(rid, None)
    return out


def plain_logits(raw, weights, requests):
    return {rid: plain.forward(raw, weights, toks) for rid, toks in requests.items()}


# Tolerances, fixed before the first run:
#  float32: what FP32 rounding in a different order gives (the reference's own kernel tests
#  use 1e-4 absolute on O(1) values).
#  bfloat16: operands rounded to 8 bits of mantissa (relative 2^-9 each) through a few dozen
#  operations: bounded relative to the size of the logits.
F32_RTOL, F32_ATOL = 1e-4, 1e-5
BF16_MAX_REL, BF16_RMS_REL = 0.05, 0.015


def compare(got, want_by_req, dtype, label=""):
    """got: {(id, pos): row}; want_by_req: {id: [T, V]}."""
    assert got, "no logits were produced"
    for (rid, pos), row in got.items():
        ref = want_by_req[rid][pos]
        if dtype == "float32":
            # the absolute rounding error of an FP32 dot product grows with the size of its terms:
            # the absolute bound is taken relative to the largest logit of the row (at least 1)
            torch.testing.assert_close(row, ref, rtol=F32_RTOL, atol=F32_ATOL * max(1.0, ref.abs().max().item()),
                                       msg=lambda m: f"{label} request {rid} position {pos}: {m}")
        else:
            err = (row - ref).abs()
            scale = ref.abs().max().item()
            rms = ref.pow(2).mean().sqrt().item()
            assert err.max().item() <= BF16_MAX_REL * scale, \
                f"{label} request {rid} position {pos}: max error {err.max().item():.4g} > {BF16_MAX_REL} * {scale:.4g}"
            assert err.pow(2).mean().sqrt().item() <= BF16_RMS_REL * rms, \
                f"{label} request {rid} position {pos}: rms error {err.pow(2).mean().sqrt().item():.4g} > {BF16_RMS_REL} * {rms:.4g}"
