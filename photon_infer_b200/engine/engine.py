"""The engine a user talks to: requests in (token ids), generated token ids out.

Named after the reference's ``ContinuousBatchEngine`` (include/photon/scheduler/
continuous_batch_engine.hpp:48-315) and with its methods: ``add_request(prompt,
max_new_tokens)``, ``run_until_complete(print_progress)``; its constructor arguments
``max_batch_size`` and ``chunk_size`` are fields of ``EngineOptions``.  The loop of one
step is the same (schedule, flatten, forward, sample, update), with these differences:
only the rows that are sampled get logits, sampling runs for all rows in one kernel,
and one copy brings the sampled ids to the host.  Tokenizing is outside the engine:
prompts are token ids.
"""
from __future__ import annotations

import dataclasses
import sys
from typing import Dict, List, Optional, Sequence

import torch

from ..config.engine_options import EngineOptions
from ..errors import ErrorCode, PhotonError
from ..sampling.sampler import Sampler, uniform
from .loading import build_runner
from .request import InferenceRequest, SamplingParams
from .runner import ModelRunner, StepEntry
from .scheduler import ContinuousBatchScheduler, ScheduledBatch


@dataclasses.dataclass
class _InFlight:
    """A step whose sampled ids have not been read yet."""
    batch: ScheduledBatch
    samplers: List[InferenceRequest]
    tokens: Optional[torch.Tensor]
    host: Optional[torch.Tensor]        # pinned: the sampled ids, then the four words of the error word
    event: Optional["torch.cuda.Event"]
    dropped: set
    report: "StepReport"


@dataclasses.dataclass
class StepReport:
    num_requests: int
    num_tokens: int
    finished: List[int]
    preempted: List[int]
    failed: List[int]


class ContinuousBatchEngine:
    def __init__(self, model: str, options: Optional[EngineOptions] = None, runner: Optional[ModelRunner] = None):
        """``model``: a folder with ``config.json`` and ``model.safetensors``."""
        self.options = options or EngineOptions()
        self.options.validate()
        self.runner = runner or build_runner(model, self.options)
        spec = self.runner.model.spec
        self.max_model_len = self.runner.max_model_len
        self.scheduler = ContinuousBatchScheduler(
            self.runner.cache, self.options.max_batch_size, self.options.max_sequences, self.options.chunk_size,
            self.options.max_num_batched_tokens, self.max_model_len, spec.eos_token_ids)
        self.sampler = Sampler(self.runner.device)
        self._host_slots: List[Optional[torch.Tensor]] = [None, None]
        self._launches = 0
        self._inflight: Optional[_InFlight] = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], max_new_tokens: int = 16, temperature: float = 0.0,
                    seed: Optional[int] = None, ignore_eos: bool = False) -> int:
        vocab = self.runner.model.spec.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise PhotonError(ErrorCode.INVALID_INDEX, f"prompt token {t} is outside the vocabulary of {vocab}")
        params = SamplingParams(temperature=float(temperature), seed=self.options.seed if seed is None else seed,
                                max_new_tokens=max_new_tokens, ignore_eos=ignore_eos)
        return self.scheduler.add_request([int(t) for t in prompt], params)

    def abort(self, request_id: int) -> None:
        self._drain()
        self.scheduler.abort(request_id)

    def result(self, request_id: int) -> InferenceRequest:
        return self.scheduler.get_request(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ------------------------------------------------------------------ one step
    def step(self) -> StepReport:
        """Runs one step.  Decode steps are pipelined by one (``async_decode``): while the requests and
        their order stay the same, the next step is enqueued with the previous step's ids still on the
        device, and the ids are read (and end-of-sequence is seen) one call later.  The report is that of
        the step whose ids were read in this call."""
        p = self._inflight
        if p is not None:
            if self._can_continue(p):
                nxt = self._launch(self.scheduler.continue_decode([it.request for it in p.batch.items]),
                                   device_tokens=p.tokens, lag=1)
                report = self._complete(p, later=nxt)
                self._inflight = nxt
                return report
            self._inflight = None
            return self._complete(p, later=None)
        batch = self.scheduler.schedule_next_batch()
        if batch.empty():
            return StepReport(0, 0, [], [r.request_id for r in batch.preempted], [r.request_id for r in batch.failed])
        launched = self._launch(batch, device_tokens=None, lag=0)
        if self.options.async_decode and self.runner.use_cuda_graphs and launched.samplers \
                and all(it.num_tokens == 1 and it.samples for it in batch.items):
            self._inflight = launched               # its ids are read by the next call
            return launched.report
        return self._complete(launched, later=None)

    def _launch(self, batch: ScheduledBatch, device_tokens, lag: int) -> "_InFlight":
        report = StepReport(batch.batch_size(), batch.num_tokens(), [], [r.request_id for r in batch.preempted],
                            [r.request_id for r in batch.failed])
        entries, samplers = [], []
        for it in batch.items:
            tokens = [0] if device_tokens is not None else it.request.next_tokens(it.num_tokens)
            entries.append(StepEntry(it.request.request_id, tokens, [it.num_tokens - 1] if it.samples else []))
            if it.samples:
                samplers.append(it.request)
        temps = [r.params.temperature for r in samplers]
        us = [uniform(r.params.seed, r.request_id, r.num_generated() + lag) if r.params.temperature > 0 else 0.0
              for r in samplers]
        result = self.runner.step(entries, pages_taken=True, sampling=(temps, us) if samplers else None,
                                  device_tokens=device_tokens)
        host = event = None
        if samplers:
            n = len(samplers)
            slot = self._host_slots[self._launches % 2]
            if slot is None or slot.numel() < n + 4:
                slot = self._host_slots[self._launches % 2] = torch.empty(max(n + 4, 260), dtype=torch.int32,
                                                                         pin_memory=True)
            host = slot[:n + 4]
            host[:n].copy_(result.tokens, non_blocking=True)
            host[n:].copy_(self.runner.error_flag, non_blocking=True)     # read with the ids: no extra wait
            event = torch.cuda.Event()
            event.record()
            self.d2h_bytes += 4 * (n + 4)
        self._launches += 1
        return _InFlight(batch, samplers, result.tokens, host, event, set(), report)

    def _complete(self, p: "_InFlight", later: Optional["_InFlight"]) -> StepReport:
        sampled: Dict[int, int] = {}
        if p.samplers:
            p.event.synchronize()
            values = p.host.tolist()
            # a bad index or a wait that ran out: the ids of this step come from wrong data
            self.runner.raise_device_error(values[-4:])
            for r, t in zip(p.samplers, values[:-4]):
                if r.request_id not in p.dropped:
                    sampled[r.request_id] = t
        finished = self.scheduler.update_after_step(p.batch, sampled, skip=p.dropped)
        if later is not None:
            for r in finished:
                later.dropped.add(r.request_id)      # the step in flight still carries it; its id is ignored
        p.report.finished = [r.request_id for r in finished]
        return p.report

    def _can_continue(self, p: "_InFlight") -> bool:
        """The next step can be enqueued unseen: same running requests in the same order, nothing waiting,
        no request at its last token or at the longest length, pages for one more token each."""
        sch = self.scheduler
        if sch.waiting or len(sch.running) != len(p.batch.items) or p.dropped:
            return False
        for it, req in zip(p.batch.items, sch.running):
            if it.request is not req:
                return False
            if req.num_generated() + 2 > req.params.max_new_tokens or req.total_tokens() + 2 > self.max_model_len:
                return False
        for req in sch.running:
            if not self.runner.cache.try_extend(req.request_id, 1):
                return False
        return True

    def _drain(self) -> None:
        if self._inflight is not None:
            p, self._inflight = self._inflight, None
            self._complete(p, later=None)

    def run_until_complete(self, print_progress: bool = False) -> Dict[int, List[int]]:
        """Runs steps until no request waits or runs; returns the generated ids of every request."""
        step = 0
        while self.has_work():
            rep = self.step()
            if rep.num_requests == 0 and not rep.failed and not rep.preempted and self._inflight is None:
                raise PhotonError(ErrorCode.INVALID_STATE, "the scheduler has work but scheduled nothing")
            if print_progress and step % 10 == 0:
                st = self.scheduler.get_stats()
                print(f"Step {step}: Running={st.num_running} Waiting={st.num_waiting} Finished={st.num_finished}",
                      file=sys.stderr, flush=True)
            step += 1
        self.runner.check_device_errors()
        return {rid: list(r.generated_tokens) for rid, r in self.scheduler.requests.items()}

    def get_stats(self):
        return self.scheduler.get_stats()


def generate(model: str, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
             seed: int = 0, options: Optional[EngineOptions] = None, ignore_eos: bool = False) -> List[List[int]]:
    """One call from prompts (token ids) to generated token ids, in the order of ``prompts``."""
    engine = ContinuousBatchEngine(model, options)
    ids = [engine.add_request(p, max_new_tokens, temperature, seed, ignore_eos) for p in prompts]
    out = engine.run_until_complete()
    return [out[i] for i in ids]
