"""One generation request and its life cycle
(the reference's InferenceRequest, src/engine/inference_request.cpp:14-169)."""
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
        self.num_computed_tokens = 0      # tokens whose keys/values are in the cache
        self.num_pending = 0              # sampled tokens of this request that are still on the device
        self.state = RequestState.WAITING
        self.finish_reason: Optional[str] = None
        self.num_preemptions = 0
        self.arrival_time = time.perf_counter()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None

    # tokens that have to be run: the prompt and everything generated so far
    @property
    def num_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.generated_tokens) + self.num_pending

    @property
    def num_remaining(self) -> int:
        return len(self.prompt_tokens) + len(self.generated_tokens) + self.num_pending - self.num_computed_tokens

    def next_tokens(self, n: int) -> List[int]:
        """The next ``n`` tokens to run; PENDING_TOKEN where the token is not on the host yet."""
        a = self.num_computed_tokens
        p = len(self.prompt_tokens)
        if a + n <= p:
            return self.prompt_tokens[a:a + n]
        known = (self.prompt_tokens[a:] if a < p else []) + self.generated_tokens[max(a - p, 0):a + n - p]
        return known + [PENDING_TOKEN] * (n - len(known))

    def pending_reaches_limit(self) -> bool:
        """True if the tokens still on the device take the request to max_new_tokens."""
        return len(self.generated_tokens) + self.num_pending >= self.max_new_tokens

    def is_prefill(self) -> bool:
        return self.num_remaining > 1

    def is_finished(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.FAILED)

    def add_token(self, token: int) -> bool:
        """Append a sampled token; returns False when the request is finished by it
        (a stop token or max_new_tokens, src/engine/inference_request.cpp:61-73)."""
        if self.first_token_time is None:
            self.first_token_time = time.perf_counter()
        self.num_pending = max(0, self.num_pending - 1)
        self.generated_tokens.append(int(token))
        if int(token) in self.stop_token_ids:
            self.finish("stop")
            return False
        if len(self.generated_tokens) >= self.max_new_tokens:
            self.finish("length")
            return False
        return True

    def finish(self, reason: str) -> None:
        self.state = RequestState.FINISHED
        self.finish_reason = reason
        self.finish_time = time.perf_counter()

    def fail(self, reason: str) -> None:
        self.state = RequestState.FAILED
        self.finish_reason = reason
        self.finish_time = time.perf_counter()

    def latency_seconds(self) -> Optional[float]:
        return None if self.finish_time is None else self.finish_time - self.arrival_time
