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
import time
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
        self._host_tokens: Optional[torch.Tensor] = None
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
        self.scheduler.abort(request_id)

    def result(self, request_id: int) -> InferenceRequest:
        return self.scheduler.get_request(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one step
    def step(self) -> StepReport:
        batch = self.scheduler.schedule_next_batch()
        report = StepReport(batch.batch_size(), batch.num_tokens(), [], [r.request_id for r in batch.preempted],
                            [r.request_id for r in batch.failed])
        if batch.empty():
            return report
        entries, samplers = [], []
        for it in batch.items:
            tokens = it.request.next_tokens(it.num_tokens)
            entries.append(StepEntry(it.request.request_id, tokens, [it.num_tokens - 1] if it.samples else []))
            if it.samples:
                samplers.append(it.request)
        temps = [r.params.temperature for r in samplers]
        us = [uniform(r.params.seed, r.request_id, r.num_generated()) if r.params.temperature > 0 else 0.0
              for r in samplers]
        result = self.runner.step(entries, pages_taken=True, sampling=(temps, us) if samplers else None)
        sampled: Dict[int, int] = {}
        if samplers:
            ids = result.tokens
            n = len(samplers)
            if self._host_tokens is None or self._host_tokens.numel() < n:
                self._host_tokens = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
            self._host_tokens[:n].copy_(ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            host = self._host_tokens[:n].tolist()
            self.d2h_bytes += 4 * n
            sampled = {r.request_id: t for r, t in zip(samplers, host)}
        finished = self.scheduler.update_after_step(batch, sampled)
        report.finished = [r.request_id for r in finished]
        return report

    def run_until_complete(self, print_progress: bool = False) -> Dict[int, List[int]]:
        """Runs steps until no request waits or runs; returns the generated ids of every request."""
        step = 0
        while self.scheduler.has_work():
            rep = self.step()
            if rep.num_requests == 0 and not rep.failed and not rep.preempted:
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
