"""One generation request and its life cycle
(the reference's InferenceRequest, src/engine/inference_request.cpp:14-169).

The request holds what only the caller's side needs: its tokens, sampling parameters, stop
tokens, the reason it ended and its times.  Once it has been added to a scheduler, the
counts that scheduling runs on (tokens computed, sampled tokens still on the device, waiting or
running, preemptions) are kept by the compiled scheduler and read from there."""
from __future__ import annotations

import enum
import time
from typing import List, Optional, Sequence

from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    FAILED = "failed"


PENDING_TOKEN = -1     # stands for a token that has been sampled on the device but not read yet


class InferenceRequest:
    def __init__(self, request_id: int, prompt_tokens: Sequence[int], max_new_tokens: int,
                 sampling_params: SamplingParams, seed: int, stop_token_ids: Sequence[int] = ()) -> None:
        self.request_id = request_id
        self.prompt_tokens: List[int] = [int(t) for t in prompt_tokens]
        self.max_new_tokens = max_new_tokens
        self.sampling_params = sampling_params
        self.seed = seed
        self.stop_token_ids = frozenset(stop_token_ids)
        self.generated_tokens: List[int] = []
        self._scheduler = None            # set by Scheduler.add_request
        self._ended: Optional[RequestState] = None
        self.finish_reason: Optional[str] = None
        self.arrival_time = time.perf_counter()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None

    # ---- counts kept by the scheduler -----------------------------------------------------
    def _count(self, field: int) -> int:
        return self._scheduler.request_field(self.request_id, field) if self._scheduler is not None else 0

    @property
    def num_computed_tokens(self) -> int:
        """Tokens whose keys/values are in the cache."""
        return self._count(1)

    @property
    def num_pending(self) -> int:
        """Sampled tokens of this request that are still on the device."""
        return self._count(2)

    @property
    def num_preemptions(self) -> int:
        return self._count(4)

    @property
    def state(self) -> RequestState:
        if self._ended is not None:
            return self._ended
        return RequestState.RUNNING if self._count(0) == 1 else RequestState.WAITING

    # tokens that have to be run: the prompt and everything generated so far
    @property
    def num_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.generated_tokens) + self.num_pending

    @property
    def num_remaining(self) -> int:
        if self._scheduler is not None:
            return self._count(5)
        return len(self.prompt_tokens) + len(self.generated_tokens)

    def next_tokens(self, n: int) -> List[int]:
        """The next ``n`` tokens to run; PENDING_TOKEN where the token is not on the host yet."""
        a = self.num_computed_tokens
        p = len(self.prompt_tokens)
        if a + n <= p:
            return self.prompt_tokens[a:a + n]
        known = (self.prompt_tokens[a:] if a < p else []) + self.generated_tokens[max(a - p, 0):a + n - p]
        return known + [PENDING_TOKEN] * (n - len(known))

    def is_prefill(self) -> bool:
        return self.num_remaining > 1

    def is_finished(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.FAILED)

    def add_token(self, token: int) -> bool:
        """Append a sampled token; returns False when the request is finished by it
        (a stop token or max_new_tokens, src/engine/inference_request.cpp:61-73)."""
        if self.first_token_time is None:
            self.first_token_time = time.perf_counter()
        self.generated_tokens.append(int(token))
        if int(token) in self.stop_token_ids:
            self.finish("stop")
            return False
        if len(self.generated_tokens) >= self.max_new_tokens:
            self.finish("length")
            return False
        return True

    def finish(self, reason: str) -> None:
        self._ended = RequestState.FINISHED
        self.finish_reason = reason
        self.finish_time = time.perf_counter()

    def fail(self, reason: str) -> None:
        self._ended = RequestState.FAILED
        self.finish_reason = reason
        self.finish_time = time.perf_counter()

    def latency_seconds(self) -> Optional[float]:
        return None if self.finish_time is None else self.finish_time - self.arrival_time
