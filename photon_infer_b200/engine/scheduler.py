"""Continuous-batching scheduler: which requests run in the next step, and how many
tokens of each.

Two phases as in the reference (include/photon/scheduler/continuous_batch_scheduler.hpp:
133-158): first every RUNNING request, then WAITING requests first come first served.
Added here: a token budget per step (``max_num_batched_tokens``), prompt portions of at
most ``chunk_size`` tokens cut to the budget that is left, pages taken exactly when a
step needs them, and a decision for the case that pages run out:

* the RUNNING request admitted last is preempted (its pages are freed, it goes to the
  FRONT of the waiting queue and is computed again from its first token later), until
  the request at hand fits;
* a request that is alone and still does not fit is finished with reason
  ``"out_of_memory"``;
* no request is admitted in a step that preempted one.

The scheduler only talks to the host side of the cache manager, so it runs without a GPU.
"""
from __future__ import annotations

import collections
import dataclasses
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..errors import ErrorCode, PhotonError
from .request import InferenceRequest, RequestState, SamplingParams


@dataclasses.dataclass
class ScheduledItem:
    request: InferenceRequest
    num_tokens: int
    samples: bool                       # the portion reaches the request's last token: sample after it


@dataclasses.dataclass
class ScheduledBatch:
    items: List[ScheduledItem] = dataclasses.field(default_factory=list)
    preempted: List[InferenceRequest] = dataclasses.field(default_factory=list)
    failed: List[InferenceRequest] = dataclasses.field(default_factory=list)

    def batch_size(self) -> int:
        return len(self.items)

    def num_tokens(self) -> int:
        return sum(i.num_tokens for i in self.items)

    def empty(self) -> bool:
        return not self.items


@dataclasses.dataclass
class SchedulerStats:
    num_running: int = 0
    num_waiting: int = 0
    num_finished: int = 0
    total_requests: int = 0
    steps: int = 0
    scheduled_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    page_high_water: Tuple[int, ...] = ()


class ContinuousBatchScheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int = 32, max_sequences: int = 32,
                 chunk_size: int = 256, max_num_batched_tokens: int = 2048, max_model_len: int = 4096,
                 eos_token_ids: Sequence[int] = (), commits_lengths: bool = False):
        self.cache = cache
        # True when no step function advances the cached lengths (a scheduler driven alone)
        self.commits_lengths = commits_lengths
        self.max_batch_size = max_batch_size
        self.max_sequences = min(max_sequences, cache.max_sequences)
        self.chunk_size = chunk_size
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos_token_ids = tuple(eos_token_ids)
        self.waiting: Deque[InferenceRequest] = collections.deque()
        self.running: List[InferenceRequest] = []
        self.requests: Dict[int, InferenceRequest] = {}
        self._next_id = 0
        self._finished = 0
        self._steps = 0
        self._tokens = self._prefill = self._decode = self._preemptions = 0

    # ------------------------------------------------------------------ requests in
    def add_request(self, prompt_tokens: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        if len(prompt_tokens) == 0:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "a request needs at least one prompt token")
        if len(prompt_tokens) >= self.max_model_len:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT,
                              f"the prompt has {len(prompt_tokens)} tokens; the longest request is {self.max_model_len}")
        if params.max_new_tokens <= 0:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "max_new_tokens must be positive")
        rid = self._next_id
        self._next_id += 1
        req = InferenceRequest(rid, prompt_tokens, params)
        self.requests[rid] = req
        self.waiting.append(req)
        return rid

    def abort(self, request_id: int) -> None:
        req = self.requests[request_id]
        if req.state == RequestState.RUNNING:
            self.running.remove(req)
            self.cache.free_request(req.request_id)
        elif req.state in (RequestState.WAITING, RequestState.PREEMPTED):
            self.waiting.remove(req)
        if not req.is_finished():
            req.finish("aborted")
            self._finished += 1

    def get_request(self, request_id: int) -> InferenceRequest:
        return self.requests[request_id]

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def num_running(self) -> int:
        return len(self.running)

    def num_waiting(self) -> int:
        return len(self.waiting)

    # ------------------------------------------------------------------ the decision
    def _portion(self, req: InferenceRequest, budget: int) -> int:
        if req.is_decode():
            return 1 if budget >= 1 else 0
        return max(0, min(self.chunk_size, req.remaining(), budget))

    def _preempt(self, victim: InferenceRequest, batch: ScheduledBatch) -> None:
        self.running.remove(victim)
        self.cache.free_request(victim.request_id)
        victim.preempt()
        self.waiting.appendleft(victim)
        batch.preempted.append(victim)
        self._preemptions += 1

    def schedule_next_batch(self) -> ScheduledBatch:
        batch = ScheduledBatch()
        budget = self.max_num_batched_tokens
        # Phase 1: RUNNING requests in the order they were admitted
        i = 0
        while i < len(self.running):
            req = self.running[i]
            if len(batch.items) >= self.max_batch_size:
                break
            n = self._portion(req, budget)
            if n == 0:
                i += 1
                continue
            placed = False
            while True:
                if self.cache.try_extend(req.request_id, n):
                    placed = True
                    break
                if self.running[-1] is not req:
                    self._preempt(self.running[-1], batch)       # admitted last, not yet in this batch
                    continue
                if len(self.running) > 1 or batch.items:
                    self._preempt(req, batch)                     # others keep running; this one waits
                    break
                # alone and still too large for the pool
                self.running.remove(req)
                self.cache.free_request(req.request_id)
                req.finish("out_of_memory")
                self._finished += 1
                batch.failed.append(req)
                break
            if placed:
                batch.items.append(ScheduledItem(req, n, samples=(n == req.remaining())))
                budget -= n
                i += 1
            # a preempted or failed request left the list: the same index now holds the next one
        # Phase 2: admit WAITING requests, first come first served
        if not batch.preempted:
            while (self.waiting and budget > 0 and len(batch.items) < self.max_batch_size
                   and len(self.running) < self.max_sequences):
                req = self.waiting[0]
                n = self._portion(req, budget)
                if n == 0:
                    break
                if any(need > free for need, free in zip(self.cache.pages_needed_new(n), self.cache.free_pages())):
                    if not self.running:
                        # nothing runs, nothing will free pages: the first portion can never fit
                        self.waiting.popleft()
                        req.finish("out_of_memory")
                        self._finished += 1
                        batch.failed.append(req)
                        continue
                    break
                self.waiting.popleft()
                self.cache.add_request(req.request_id)
                self.cache.extend(req.request_id, n)
                req.start_running()
                self.running.append(req)
                batch.items.append(ScheduledItem(req, n, samples=(n == req.remaining())))
                budget -= n
        if batch.items:
            self._steps += 1
            for it in batch.items:
                self._tokens += it.num_tokens
                if it.num_tokens == 1 and it.request.is_decode():
                    self._decode += 1
                else:
                    self._prefill += it.num_tokens
        return batch

    def continue_decode(self, requests: Sequence[InferenceRequest]) -> ScheduledBatch:
        """The batch that feeds each of these RUNNING requests its next token, for a caller that enqueues
        the step before the previous step's tokens have reached the host (pages already taken)."""
        batch = ScheduledBatch([ScheduledItem(r, 1, True) for r in requests])
        self._steps += 1
        self._tokens += len(batch.items)
        self._decode += len(batch.items)
        return batch

    # ------------------------------------------------------------------ after the step
    def update_after_step(self, batch: ScheduledBatch, sampled: Dict[int, int],
                          skip: Sequence[int] = ()) -> List[InferenceRequest]:
        """``sampled`` maps request ids to the token sampled after their portion (present for every
        item whose ``samples`` is true).  ``skip``: requests that finished while this step was in flight;
        their items are ignored.  Returns the requests that finished."""
        finished = []
        for it in batch.items:
            req = it.request
            if req.request_id in skip:
                continue
            if self.commits_lengths:
                self.cache.commit(req.request_id, it.num_tokens)
            req.add_computed_tokens(it.num_tokens)
            if it.samples:
                if req.add_token(sampled[req.request_id], self.eos_token_ids, self.max_model_len):
                    finished.append(req)
        for req in finished:
            self.running.remove(req)
            self.cache.free_request(req.request_id)
            self._finished += 1
        return finished

    def clear_finished_requests(self) -> None:
        for rid in [r for r, q in self.requests.items() if q.is_finished()]:
            del self.requests[rid]

    def get_stats(self) -> SchedulerStats:
        return SchedulerStats(
            num_running=len(self.running), num_waiting=len(self.waiting), num_finished=self._finished,
            total_requests=self._next_id, steps=self._steps, scheduled_tokens=self._tokens,
            prefill_tokens=self._prefill, decode_tokens=self._decode, preemptions=self._preemptions,
            page_high_water=tuple(g.pool.high_water for g in self.cache.groups))
