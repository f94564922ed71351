"""A request and its state, as the scheduler sees it.

States and the ``num_computed_tokens`` counter follow include/photon/scheduler/
inference_request.hpp:35-40,172-191.  Two things differ on purpose.  The logits of the
last prompt token give the first generated token; the reference feeds the last prompt
token a second time instead (inference_request.hpp:208-220).  And ``PREEMPTED`` is
used: a preempted request loses its pages and is computed again from its first token,
its generated tokens included.
"""
from __future__ import annotations

import dataclasses
import enum
import time
from typing import List, Optional, Sequence


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    PREEMPTED = "preempted"


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 0.0            # 0: greedy (first maximum)
    seed: int = 0
    max_new_tokens: int = 16
    ignore_eos: bool = False


class InferenceRequest:
    def __init__(self, request_id: int, prompt_tokens: Sequence[int], params: SamplingParams):
        self.request_id = request_id
        self.prompt_tokens: List[int] = list(prompt_tokens)
        self.params = params
        self.generated_tokens: List[int] = []
        self.num_computed_tokens = 0
        self.state = RequestState.WAITING
        self.finish_reason: Optional[str] = None
        self.num_preemptions = 0
        self.arrival_time = time.monotonic()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None

    # -- sizes
    def prompt_len(self) -> int:
        return len(self.prompt_tokens)

    def num_generated(self) -> int:
        return len(self.generated_tokens)

    def total_tokens(self) -> int:
        return len(self.prompt_tokens) + len(self.generated_tokens)

    def remaining(self) -> int:
        """Tokens that exist but are not in the cache yet."""
        return self.total_tokens() - self.num_computed_tokens

    def is_finished(self) -> bool:
        return self.state == RequestState.FINISHED

    def is_decode(self) -> bool:
        """One token left to feed: the one sampled last."""
        return self.remaining() == 1 and self.num_generated() > 0

    def is_prefill(self) -> bool:
        return not self.is_decode() and self.remaining() > 0

    # -- the next tokens to feed
    def next_tokens(self, n: int) -> List[int]:
        s = self.num_computed_tokens
        p = len(self.prompt_tokens)
        if s + n <= p:
            return self.prompt_tokens[s:s + n]
        if s >= p:
            return self.generated_tokens[s - p:s - p + n]
        return self.prompt_tokens[s:] + self.generated_tokens[:s + n - p]

    # -- transitions
    def start_running(self) -> None:
        self.state = RequestState.RUNNING

    def add_computed_tokens(self, n: int) -> None:
        self.num_computed_tokens += n

    def add_token(self, token: int, eos_token_ids: Sequence[int], max_model_len: int) -> bool:
        """Appends a sampled token; returns True when the request is finished by it."""
        if self.first_token_time is None:
            self.first_token_time = time.monotonic()
        self.generated_tokens.append(int(token))
        if not self.params.ignore_eos and int(token) in eos_token_ids:
            self.finish("eos")
        elif self.num_generated() >= self.params.max_new_tokens:
            self.finish("length")
        elif self.total_tokens() >= max_model_len:
            self.finish("model_len")
        return self.is_finished()

    def finish(self, reason: str) -> None:
        self.state = RequestState.FINISHED
        self.finish_reason = reason
        self.finish_time = time.monotonic()

    def preempt(self) -> None:
        self.state = RequestState.PREEMPTED
        self.num_computed_tokens = 0
        self.num_preemptions += 1

    def latency(self) -> Optional[float]:
        return None if self.finish_time is None else self.finish_time - self.arrival_time
