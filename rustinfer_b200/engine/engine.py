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
from ..ops import kernels as K
from .scheduler import FINISHED, Request, Scheduler


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
class _InFlight:
    plan: Any
    samplers: List[Request]
    turn: int                           # which result buffer its tokens land in
    event: Any
    lazy: bool                          # its tokens may be read after the next launch


@dataclass
class EngineStats:
    stop_flag_mismatches: int = 0
    steps: int = 0
    chained_steps: int = 0              # steps launched with the step before still unread by the host
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    seconds: float = 0.0
    step_ms: List[float] = field(default_factory=list)
    # with `Engine.trace_host` set: seconds the host spent in each part of `step`, summed over the
    # steps (plan, entries, launch: the runner's step; choose: sampler and feedback launches;
    # wait: blocked until the tokens of the step before were on the host; deliver)
    host_seconds: Dict[str, float] = field(default_factory=dict)


class Engine:
    def __init__(self, model: str, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_batch_tokens: int = 8192, max_batch_seqs: int = 32, max_model_len: int = 4096,
                 paged_block_size: int = 16, chunked_prefill_size: int = 0,
                 mem_fraction_static: float = 0.9, num_blocks: int = 0, ignore_eos: bool = False,
                 capture_sizes: Optional[Sequence[int]] = None):
        self.ignore_eos = ignore_eos
        self.trace_host = False             # True: `stats.host_seconds` says where the host's time in `step` goes
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
        # the step in flight, the device buffers its tokens and stop flags land in (two, used
        # in turn, with pinned host twins), and the buffer the next step reads its ids from
        self._inflight: Optional[_InFlight] = None
        self._turn = 0
        dev = self.runner.device
        self._result_dev = [torch.zeros(2 * max_batch_seqs, dtype=torch.int32, device=dev) for _ in range(2)]
        self._result_host = [torch.zeros(2 * max_batch_seqs, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._feed = torch.zeros(max_batch_seqs, dtype=torch.int32, device=dev)

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
        return self.scheduler.has_work() or self._inflight is not None

    # ---------------------------------------------------------------------------- step
    def step(self) -> List[StepOutput]:
        """One iteration: schedule a batch, launch it, choose tokens on the device.

        A step leaves its tokens on the device (`_inflight`), greedy or drawn (a row's uniform
        draw is a function of the request's seed and the token's position, both known to the
        host before the token is): the stop check runs there, the tokens are fed to the next
        step there, and the host reads them only after it has launched that next step, so
        planning and launching overlap the GPU's work.  The tokens a call returns are therefore those of the step before
        the one it launched; `has_unfinished()` stays true until the last ones are read.
        This is the engine's counterpart of RustInfer's one-deep device-resident decode
        pipeline (crates/infer-worker/src/application/runtime/abc_decode.rs:77-89,109-)."""
        sched = self.scheduler
        outs: List[StepOutput] = []
        before = sched.num_preemptions
        clock = time.perf_counter
        trace = self.stats.host_seconds if self.trace_host else None
        t_a = clock()
        plan = sched.schedule()
        self.stats.preemptions += sched.num_preemptions - before
        chain = self._inflight is not None and self._chainable(plan)
        if self._inflight is not None and not chain:
            outs += self._resolve()                           # the plan needs these tokens on the host
            plan.entries = [e for e in plan.entries if e.request.state != FINISHED]
        if not plan.entries:
            return outs
        r = self.runner
        entries: List[StepEntry] = []
        samplers: List[Request] = []
        for e in plan.entries:
            req = e.request
            if e.start == 0:                                  # first portion since (re)admission
                made = len(req.output)
                cap = min(req.params.max_tokens, r.max_model_len - len(req.prompt))
                r.set_request_limits(req.request_id, made, cap, req.params.ignore_eos)
            toks = [0] if chain else req.tokens(e.start, e.count)
            entries.append(StepEntry(req.request_id, toks, [e.count - 1] if e.samples else []))
            if e.samples:
                samplers.append(req)
        t0 = clock()
        if trace is not None:
            trace["plan and entries"] = trace.get("plan and entries", 0.0) + (t0 - t_a)
        logits = r.step(entries, device_tokens=self._feed if chain else None, borrow_logits=True)
        t_b = clock()
        launched = None
        if samplers:
            n = len(samplers)
            positions = [len(q.prompt) + len(q.output) + q.undelivered for q in samplers]
            chosen = self.sampler.sample_device(logits, [q.params for q in samplers],
                                                [q.seed for q in samplers], positions)
            k = self._turn = (self._turn + 1) % 2
            K.decode_feedback(chosen, r.last_want_slots, r.slot_state, r.eos_dev, self._result_dev[k], self._feed)
            self._result_host[k][: 2 * n].copy_(self._result_dev[k][: 2 * n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            launched = _InFlight(plan, samplers, k, ev, True)
        sched.advance(plan)
        t_c = clock()
        if trace is not None:
            trace["launch (runner.step)"] = trace.get("launch (runner.step)", 0.0) + (t_b - t0)
            trace["choose and feed back"] = trace.get("choose and feed back", 0.0) + (t_c - t_b)
        self.stats.steps += 1
        self.stats.chained_steps += 1 if chain else 0
        self.stats.prompt_tokens += sum(e.count for e in plan.entries) - sum(
            1 for e in plan.entries if e.count == 1 and (e.request.output or e.request.undelivered > 1))
        if chain:
            outs += self._resolve()                           # last step's tokens, read while this one runs
        self._inflight = launched
        if launched is not None and not launched.lazy:
            outs += self._resolve()
        self.stats.step_ms.append((time.perf_counter() - t0) * 1e3)
        return outs

    def _chainable(self, plan) -> bool:
        """The planned step can take its input tokens from the device: it is made of the
        very rows whose tokens are in flight, one token each, in the same order."""
        prev = self._inflight
        if not prev.lazy or len(plan.entries) != len(prev.samplers) or not plan.entries:
            return False
        return all(e.count == 1 and e.samples and e.request is q
                   for e, q in zip(plan.entries, prev.samplers))

    def _resolve(self) -> List[StepOutput]:
        """Wait for the tokens of the step in flight, hand them to the scheduler."""
        f, self._inflight = self._inflight, None
        t_w = time.perf_counter()
        f.event.synchronize()
        if self.trace_host:
            h = self.stats.host_seconds
            h["wait for the step before"] = h.get("wait for the step before", 0.0) + (time.perf_counter() - t_w)
        n = len(f.samplers)
        res = self._result_host[f.turn][: 2 * n].tolist()
        tokens, stops = res[:n], res[n:]
        live = [q.state != FINISHED for q in f.samplers]
        self.scheduler.deliver(f.plan, tokens)
        outs = []
        for q, t, s, was_live in zip(f.samplers, tokens, stops, live):
            if not was_live:
                continue
            # the device's stop flag and the host's decision are the same rule twice
            if bool(s) != (q.finish_reason in ("stop", "length")):
                self.stats.stop_flag_mismatches += 1
            outs.append(StepOutput(q.request_id, t, q.finish_reason))
        self.stats.generated_tokens += len(outs)
        return outs

    def abort(self, request_id: int) -> None:
        """Stop a request wherever it is; its pages and slot are given back."""
        if self._inflight is not None:
            self._resolve()
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
        idle = 0
        while self.has_unfinished() and idle < 4:
            steps_before = self.stats.steps
            got = self.step()
            idle = 0 if (got or self.stats.steps != steps_before) else idle + 1
        self.stats.seconds += time.perf_counter() - t0
        self.runner.check_kernel_errors()
        return [self.take_finished(i) for i in ids]
