"""The engine: requests in, tokens out.  Scheduler -> step function -> sampler, every step.

Same public surface as the reference's Engine (include/nanoinfer/engine/engine.h:23-105):
EngineConfig with its field names and defaults, add_request / step / run / stop / has_work /
get_request / get_request_result / get_scheduler_stats.  Requests are given as token ids
(tokenisation is outside this engine).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..sampling import Sampler, SamplingParams
from .request import InferenceRequest, RequestState
from .scheduler import ScheduledBatch, Scheduler, SchedulerStats
from .step import ModelRunner, StepEntry


@dataclass
class EngineConfig:
    max_batch_size: int = 32            # requests in one step
    max_sequences: int = 128            # requests running at once
    prefill_chunk_size: int = 512       # most prompt tokens of one request per step
    block_size: int = 16                # tokens per cache page
    num_cache_blocks: int = 1024        # pages in the pool
    max_num_batched_tokens: int = 2048  # token budget of one step
    max_model_len: Optional[int] = None  # most tokens a request may hold (default: model limit)
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    overlap_steps: bool = True          # launch a decode step before the previous step's tokens are read
    fused_decode: bool = False          # small decode steps as one persistent kernel (see ModelRunner)


@dataclass
class StepOutput:
    request_id: int
    token: int
    finished: bool


@dataclass
class _InFlight:
    """A launched step whose sampled tokens have not been read yet."""
    batch: ScheduledBatch
    emitting: List[InferenceRequest]
    ids: Optional[torch.Tensor]              # the sampled ids where the sampler left them
    host: Optional[torch.Tensor] = None      # their copy on the host (pinned when ids are on a GPU)
    ready: Optional["torch.cuda.Event"] = None
    error: Optional[torch.Tensor] = None     # the device's error word as it stood after this step, on the host
    epoch: int = 0                           # how many device errors the engine had seen when this step was launched


class Engine:
    def __init__(self, runner, sampler=None, config: Optional[EngineConfig] = None,
                 stop_token_ids: Sequence[int] = ()) -> None:
        """``runner`` provides .cache (a CacheManager), .step(entries) -> logits, .end(request)
        and .config.vocab_size; ``sampler`` provides .sample(...).  Use ``from_model_dir`` for
        the usual construction."""
        self.config = config or EngineConfig()
        self.runner = runner
        self.sampler = sampler
        self.stop_token_ids = tuple(stop_token_ids)
        self.scheduler = Scheduler(runner.cache, self.config.max_batch_size, self.config.max_sequences,
                                   self.config.prefill_chunk_size, self.config.max_num_batched_tokens)
        self._next_id = 0
        self._running = False
        self.num_steps = 0
        self._inflight: Optional[_InFlight] = None
        self._pinned: List[torch.Tensor] = []       # two buffers for sampled ids (+ the error word), used in turn
        self._pinned_next = 0
        self._device_error: Optional[Exception] = None
        self._error_epoch = 0

    @classmethod
    def from_model_dir(cls, model_dir: str, config: Optional[EngineConfig] = None, **overrides) -> "Engine":
        from ..config import load_config
        from ..weights import load_weights
        cfg = config or EngineConfig()
        for k, v in overrides.items():
            if not hasattr(cfg, k):
                raise TypeError(f"unknown engine option '{k}'")
            setattr(cfg, k, v)
        model_config = load_config(model_dir)
        weights = load_weights(model_dir, model_config)
        return cls.from_weights(model_config, weights, cfg)

    @classmethod
    def from_weights(cls, model_config, weights, config: Optional[EngineConfig] = None) -> "Engine":
        cfg = config or EngineConfig()
        runner = ModelRunner(model_config, weights, dtype=cfg.dtype, page_size=cfg.block_size,
                             num_pages=cfg.num_cache_blocks, max_requests=cfg.max_sequences,
                             max_tokens_per_request=cfg.max_model_len,
                             max_portion_tokens=min(cfg.prefill_chunk_size, cfg.max_num_batched_tokens), device=cfg.device,
                             fused_decode=cfg.fused_decode)
        sampler = Sampler(model_config.vocab_size, runner.rt.device)
        return cls(runner, sampler, cfg, stop_token_ids=model_config.eos_token_ids)

    # ---- requests -------------------------------------------------------------------------
    def add_request(self, prompt_tokens: Sequence[int], max_new_tokens: int = 128,
                    sampling_params: Optional[SamplingParams] = None) -> int:
        """Queue a request; returns its id.  Raises ValueError for a request that can never
        run (empty, bad token id, longer than the model or the pool allow)."""
        sp = sampling_params or SamplingParams()
        sp.validate()
        prompt = [int(t) for t in prompt_tokens]
        vocab = self.runner.config.vocab_size
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        bad = [t for t in prompt if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside [0, {vocab})")
        cache = self.runner.cache
        limit = cache.max_tokens_per_request
        if len(prompt) + 1 > limit:
            raise ValueError(f"a prompt of {len(prompt)} tokens leaves no room to generate within the "
                             f"limit of {limit} tokens per request")
        pool_tokens = min(p.num_pages for p in cache.pools) * cache.page_size
        if len(prompt) + 1 > pool_tokens:
            raise ValueError(f"a prompt of {len(prompt)} tokens does not fit the cache pool of "
                             f"{pool_tokens} tokens")
        max_new_tokens = min(max_new_tokens, limit - len(prompt))
        seed = sp.seed if sp.seed >= 0 else int.from_bytes(os.urandom(7), "little")
        rid = self._next_id
        self._next_id += 1
        self.scheduler.add_request(InferenceRequest(rid, prompt, max_new_tokens, sp, seed, self.stop_token_ids))
        return rid

    def get_request(self, request_id: int) -> InferenceRequest:
        return self.scheduler.requests[request_id]

    def get_request_result(self, request_id: int) -> List[int]:
        """The tokens generated so far for the request."""
        return list(self.scheduler.requests[request_id].generated_tokens)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def get_scheduler_stats(self) -> SchedulerStats:
        return self.scheduler.stats()

    # ---- stepping -------------------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        """One scheduling decision and one forward pass over its batch; returns one token for
        every request whose last pending token was in a step that has been read.

        With ``overlap_steps`` a step's sampled ids stay on the device: when the next decision
        is already known (the same requests go on decoding), the next step is launched with
        those ids fed on the device, and only then are they read and reported - the host's
        work hides behind the running step, and a request's tokens are reported one call
        later.  A request that turns out to have hit a stop token has then run one token too
        many; that token is dropped.  In every other situation the tokens are read first."""
        outputs: List[StepOutput] = []
        previous = self._inflight
        chain = previous is not None and self._can_chain(previous)
        if previous is not None and not chain:
            outputs += self._collect(previous)
            previous = self._inflight = None
        launched = self._launch(previous)
        if previous is not None:
            outputs += self._collect(previous)
        self._inflight = launched
        if launched is not None and not self._may_stay_in_flight(launched):
            outputs += self._collect(launched)
            self._inflight = None
        if self._device_error is not None:
            err, self._device_error = self._device_error, None
            self.last_outputs = outputs        # what was booked before the error is not lost
            raise err
        return outputs

    def _may_stay_in_flight(self, step: _InFlight) -> bool:
        return (self.config.overlap_steps and bool(step.emitting)
                and getattr(self.runner, "can_feed_device_tokens", lambda n: False)(len(step.emitting)))

    def _can_chain(self, previous: _InFlight) -> bool:
        return (len(previous.emitting) == len(previous.batch.entries)
                and not any(r.sampling_params.use_repetition_penalty() for r in previous.emitting)
                and self.runner.can_feed_device_tokens(len(previous.emitting))
                and self.scheduler.can_continue_decoding(previous.batch))

    def _launch(self, feed: Optional[_InFlight]) -> Optional[_InFlight]:
        """Schedule, run and sample one step without reading its tokens.  ``feed``: the step
        still in flight whose ids are this step's tokens, in the same order."""
        batch = self.scheduler.schedule()
        if not batch.entries:
            return None
        entries, emitting = [], []
        for req, n in batch.entries:
            want = [n - 1] if n == req.num_remaining else []
            entries.append(StepEntry(req.request_id, req.next_tokens(n), want))
            if want:
                emitting.append(req)
        if feed is not None:
            assert [r for r, _ in batch.entries] == feed.emitting, "the chained batch must repeat the one in flight"
            logits = self.runner.step(entries, device_tokens=feed.ids)
        else:
            logits = self.runner.step(entries)
        step = _InFlight(batch, emitting, None, epoch=self._error_epoch)
        if emitting:
            step.ids = self.sampler.sample(
                logits, [r.sampling_params for r in emitting], [r.seed for r in emitting],
                [len(r.generated_tokens) + r.num_pending for r in emitting], [r.generated_tokens for r in emitting])
            # the error word of the device rides with the ids: a kernel that gave up a bounded wait
            # during this step (or an earlier one that emitted nothing) is seen when they are read
            word = getattr(self.runner, "error_word", None)
            n = len(emitting)
            if step.ids.is_cuda:
                if not self._pinned:
                    cap = max(self.config.max_batch_size, n) + 1
                    self._pinned = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]
                if n + 1 > self._pinned[0].numel():
                    self._pinned = [torch.empty(2 * n + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
                buf = self._pinned[self._pinned_next]
                self._pinned_next ^= 1
                step.host = buf[:n]
                step.host.copy_(step.ids, non_blocking=True)
                if word is not None:
                    step.error = buf[n:n + 1]
                    step.error.copy_(word, non_blocking=True)
                step.ready = torch.cuda.Event()
                step.ready.record()
            else:
                step.host = step.ids
                step.error = word
        self.scheduler.advance(batch, emitting)
        self.num_steps += 1
        return step

    def _collect(self, step: _InFlight) -> List[StepOutput]:
        """Read a launched step's tokens and book them."""
        if not step.emitting:
            return []
        if step.ready is not None:
            step.ready.synchronize()
        if step.epoch != self._error_epoch:
            return []          # launched before a device error was seen: its requests have failed already
        code = int(step.error[0]) if step.error is not None else 0
        if code:
            self._fail_running(code)
            return []
        sampled: Dict[int, int] = {}
        for req, tok in zip(step.emitting, step.host.tolist()):
            if not req.is_finished() and req.num_pending > 0:      # else: it ended meanwhile
                sampled[req.request_id] = int(tok)
        done = {r.request_id for r in self.scheduler.commit(sampled)}
        return [StepOutput(rid, tok, rid in done) for rid, tok in sampled.items()]

    def _fail_running(self, code: int) -> None:
        """A kernel gave up a bounded wait: what the steps since the last check computed and wrote
        into the cache is not to be trusted.  Every running request fails with reason
        "device_error" (pages and slots given back); waiting requests are untouched and the engine
        goes on.  step() raises a KernelError once the books are in order."""
        from ..kernels import ops
        word = getattr(self.runner, "error_word", None)
        if word is not None:
            word.zero_()
        for req in self.scheduler.running_requests():
            self.scheduler.abort(req, "device_error")
        self._error_epoch += 1
        if self._device_error is None:
            self._device_error = ops.KernelError(
                f"a kernel gave up waiting ({ops.describe_device_error(code)}); the running requests "
                f"have failed with reason 'device_error', the engine can go on")

    def run(self) -> None:
        """Step until no request is waiting or running (or stop() is called)."""
        self._running = True
        while self._running and self.has_work():
            self.step()
        self._running = False

    def stop(self) -> None:
        self._running = False

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128,
                 sampling_params: Optional[SamplingParams] = None) -> List[List[int]]:
        """Generate for a list of token-id prompts; returns the generated ids per prompt."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        ids = [self.add_request(p, max_new_tokens, sp) for p, sp in zip(prompts, sampling_params)]
        self.run()
        return [self.get_request_result(i) for i in ids]
