"""The Python entry point: an `Engine` that generates tokens for prompts of token ids.

    engine = Engine(model="path/to/folder", dtype="bfloat16", max_batch_seqs=32, ...)
    results = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(max_tokens=16))

Options carry RustInfer's names and meanings (run file keys,
crates/infer-protocol/src/config.rs:55-262).  The reference has no Python entry point
(its Python is bench tooling only, pyproject.toml:1-17) and takes text over HTTP; this
engine takes and returns token ids.  One loop drives scheduler, step function and sampler:
the counterpart of the reference's serve loop
(crates/infer-worker/src/application/serve_loop.rs:663-880) without the process split.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..config.run_config import DEFAULT_CAPTURE_SIZES, RunConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, fresh_seed
from .runner import ModelRunner, StepEntry
from .scheduler import Request, Scheduler


@dataclass
class GenerationResult:
    request_id: Any
    prompt: List[int]
    tokens: List[int]
    finish_reason: str
    preemptions: int = 0


@dataclass
class StepOutput:
    request_id: Any
    token: int
    finish_reason: Optional[str]        # None while the request goes on


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    seconds: float = 0.0
    step_ms: List[float] = field(default_factory=list)


class Engine:
    def __init__(self, model: str, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_batch_tokens: int = 8192, max_batch_seqs: int = 32, max_model_len: int = 4096,
                 paged_block_size: int = 16, chunked_prefill_size: int = 0,
                 mem_fraction_static: float = 0.9, num_blocks: int = 0, ignore_eos: bool = False,
                 capture_sizes: Optional[Sequence[int]] = None):
        self.ignore_eos = ignore_eos
        self.chunked_prefill_size = chunked_prefill_size
        if num_blocks <= 0:
            num_blocks = None
        self.runner = ModelRunner(model, dtype=dtype, device=device, max_model_len=max_model_len,
                                  page_size=paged_block_size, num_pages=num_blocks,
                                  max_batch_seqs=max_batch_seqs, max_batch_tokens=max_batch_tokens,
                                  mem_fraction_static=mem_fraction_static,
                                  capture_sizes=list(capture_sizes if capture_sizes is not None
                                                     else DEFAULT_CAPTURE_SIZES))
        self.sampler = Sampler(self.runner.device, self.runner.spec.vocab_size, max_batch_seqs)
        r = self.runner
        self.scheduler = Scheduler(r.cache, r.max_batch_tokens, r.max_batch_seqs, r.max_model_len,
                                   chunked_prefill_size, r.spec.eos_token_ids)
        self._requests: Dict[int, Request] = {}
        self.stats = EngineStats()
        self._next_id = 0

    @classmethod
    def from_run_config(cls, cfg: RunConfig) -> "Engine":
        return cls(model=cfg.model, dtype=cfg.dtype, device=cfg.device,
                   max_batch_tokens=cfg.max_batch_tokens, max_batch_seqs=cfg.max_batch_seqs,
                   max_model_len=cfg.max_model_len, paged_block_size=cfg.paged_block_size,
                   chunked_prefill_size=cfg.chunked_prefill_size,
                   mem_fraction_static=cfg.mem_fraction_static, num_blocks=cfg.num_blocks,
                   ignore_eos=cfg.ignore_eos, capture_sizes=cfg.capture_sizes)

    # ------------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], sampling: Optional[SamplingParams] = None) -> int:
        """Queue one prompt (token ids on the host); returns the request's id."""
        p = sampling or SamplingParams()
        if self.ignore_eos and not p.ignore_eos:
            p = SamplingParams(**{**p.__dict__, "ignore_eos": True})
        req = Request(self._next_id, [int(t) for t in prompt], p,
                      seed=p.seed if p.seed is not None else fresh_seed())
        self._next_id += 1
        self.scheduler.add(req)
        self._requests[req.request_id] = req
        return req.request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> List[StepOutput]:
        """One iteration: schedule a batch, run it, sample.  Returns what each request that
        produced a token in this step got (token ids on the host)."""
        sched = self.scheduler
        before = sched.num_preemptions
        plan = sched.schedule()
        self.stats.preemptions += sched.num_preemptions - before
        if not plan.entries:
            return []
        entries = []
        samplers: List[Request] = []
        for e in plan.entries:
            entries.append(StepEntry(e.request.request_id, e.request.tokens(e.start, e.count),
                                     [e.count - 1] if e.samples else []))
            if e.samples:
                samplers.append(e.request)
        t0 = time.perf_counter()
        logits = self.runner.step(entries, borrow_logits=True)
        sampled: List[int] = []
        if samplers:
            sampled = self.sampler.sample(
                logits, [q.params for q in samplers], [q.seed for q in samplers],
                [len(q.prompt) + len(q.output) for q in samplers])
        self.stats.step_ms.append((time.perf_counter() - t0) * 1e3)
        self.stats.steps += 1
        self.stats.prompt_tokens += sum(e.count for e in plan.entries) - sum(
            1 for e in plan.entries if e.count == 1 and e.request.output)
        self.stats.generated_tokens += len(sampled)
        sched.complete_step(plan, sampled)
        return [StepOutput(q.request_id, t, q.finish_reason) for q, t in zip(samplers, sampled)]

    def abort(self, request_id: int) -> None:
        """Stop a request wherever it is; its pages and slot are given back."""
        q = self._requests.pop(request_id)
        self.scheduler.abort(q)

    def take_finished(self, request_id: int) -> "GenerationResult":
        q = self._requests.pop(request_id)
        return GenerationResult(q.request_id, q.prompt, q.output, q.finish_reason or "aborted", q.preemptions)

    # ------------------------------------------------------------------------ generate
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids on the host); results come back in
        the order of the prompts, as lists of token ids on the host."""
        if sampling is None:
            sampling = SamplingParams()
        params = [sampling] * len(prompts) if isinstance(sampling, SamplingParams) else list(sampling)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        t0 = time.perf_counter()
        while self.scheduler.has_work():
            if not self.step() and not self.scheduler.has_work():
                break
        self.stats.seconds += time.perf_counter() - t0
        self.runner.check_kernel_errors()
        return [self.take_finished(i) for i in ids]
