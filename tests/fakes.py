"""A runner and a sampler without a GPU, for the scheduler and engine tests (the reference
tests its engine the same way with a MockModel, test/test_engine/test_engine.cpp:11-78)."""
import torch

from nanoinfer_b200.cache import CacheManager, GroupSpec
from nanoinfer_b200.engine import reserve_entries


class FakeConfig:
    def __init__(self, vocab_size):
        self.vocab_size = vocab_size


class FakeRunner:
    """Keeps the cache's books exactly as the real runner does; its "logits" put all weight on
    (sum of the request's tokens so far + position) mod vocab, so the next token is a function
    of the whole history, as in a real model."""

    def __init__(self, vocab=50, num_pages=16, page_size=4, max_requests=4, max_tokens=64, window=None):
        groups = [GroupSpec(1, 16, None)] + ([GroupSpec(1, 16, window)] if window else [])
        self.cache = CacheManager(groups, [num_pages] * len(groups), page_size, max_requests, max_tokens)
        self.config = FakeConfig(vocab)
        self.history = {}
        self.steps = []

    def step(self, entries):
        starts = reserve_entries(self.cache, entries, self.cache.admit)
        rows = []
        self.steps.append([(e.request, len(e.tokens), s) for e, s in zip(entries, starts)])
        for e, s in zip(entries, starts):
            hist = self.history.setdefault(e.request, [])
            assert len(hist) == s or s == 0, "tokens must arrive in order"
            if s == 0:
                hist.clear()
            for i, t in enumerate(e.tokens):
                hist.append(int(t))
                if i in e.want:
                    row = torch.zeros(self.config.vocab_size)
                    row[(sum(hist) + len(hist)) % self.config.vocab_size] = 1.0
                    rows.append(row)
            self.cache.release_passed(e.request)
        return torch.stack(rows) if rows else torch.zeros(0, self.config.vocab_size)

    def end(self, request):
        self.cache.free(request)


class FakeFeedingRunner(FakeRunner):
    """A fake runner that, like the real one, can take the tokens of a step of single tokens from
    the previous step's sampled ids, so that the engine overlaps its steps."""

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.fed_steps = 0

    def can_feed_device_tokens(self, n):
        return n > 0

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            from nanoinfer_b200.engine.request import PENDING_TOKEN
            from nanoinfer_b200.engine import StepEntry
            assert all(list(e.tokens) == [PENDING_TOKEN] for e in entries) and len(device_tokens) == len(entries)
            entries = [StepEntry(e.request, [int(t)], e.want) for e, t in zip(entries, device_tokens.tolist())]
            self.fed_steps += 1
        else:
            assert all(t >= 0 for e in entries for t in e.tokens), "a pending token reached the runner unfed"
        return super().step(entries)


class ArgmaxSampler:
    def sample(self, logits, params, seeds, token_indices, generated=None):
        return torch.argmax(logits, dim=-1).int()


def expected_continuation(prompt, n_new, vocab, stop=()):
    hist, out = list(prompt), []
    for _ in range(n_new):
        t = (sum(hist) + len(hist)) % vocab
        out.append(t)
        hist.append(t)
        if t in stop:
            break
    return out
