"""Continuous batching: which requests run in the next step, and with how many tokens.

Every iteration builds one batch for the step function:
  1. each request that is decoding gets its one token;
  2. requests whose prompt is partly computed get their next portion;
  3. waiting requests are admitted first come first served, while a request slot, token
     budget and pages are left.  A request that does not fit whole is admitted with the
     portion that does (crates/infer-scheduler/src/domain/policy/continuous_batching.rs:217-246).
A portion is at most `chunked_prefill_size` tokens (0: no cap) and at most what is left
of `max_batch_tokens`; it may be cut anywhere, down to one token.  Decode rows come first
in the batch, then prompt portions
(crates/infer-worker/src/application/worker_scheduler.rs:666-731).

When pages run out.  A decoding request that cannot get the page its next token needs
makes room by *preemption*: the most recently admitted request that holds pages (never
the only one running) gives all its pages back and returns to the front of the waiting
queue with what it generated appended to its prompt, to be recomputed when pages are
free again.  That is RustInfer's second relief round
(crates/infer-scheduler/src/application/control_fns.rs:172-270,
crates/infer-scheduler/src/domain/inference_session/lifecycle.rs:123-131), with the
victim chosen by admission order instead of output length.  Prompt portions never
preempt: they are shortened to the pages that are free, or wait.  A request that cannot
fit the pool even alone fails with `finish_reason = "kv_pool_exhausted"`.

This class is host logic over a `CacheManager`; it never touches the GPU, so its
decisions are tested with a stand-in step function.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, PREFILL, DECODE, FINISHED = "waiting", "prefill", "decode", "finished"
DRAINING = "draining"     # its last token is chosen but not yet delivered to the host: nothing more to run


@dataclass(eq=False)                     # a request is itself: lists of them are searched by identity, not by comparing prompts
class Request:
    request_id: Any
    prompt: List[int]
    params: SamplingParams
    seed: int = 0
    state: str = WAITING
    output: List[int] = field(default_factory=list)
    computed: int = 0                    # tokens of prompt + output whose keys are in the cache
    admitted_at: int = -1                # admission counter, for the choice of a victim
    preemptions: int = 0
    finish_reason: Optional[str] = None
    undelivered: int = 0                 # tokens chosen on the device that the host has not read yet

    @property
    def sequence(self) -> List[int]:
        return self.prompt + self.output

    def tokens(self, start: int, count: int) -> List[int]:
        """Tokens start .. start+count-1 of prompt + output, without joining the two lists."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n: start - n + count]
        if start + count <= n:
            return self.prompt[start: start + count]
        return self.prompt[start:] + self.output[: start + count - n]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed


@dataclass
class PlannedEntry:
    request: Request
    start: int                           # first token of the portion within request.sequence
    count: int
    samples: bool                        # the portion ends the sequence: its last logits pick a token


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[Any] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int, max_batch_seqs: int,
                 max_model_len: int, chunked_prefill_size: int = 0, eos_token_ids: Sequence[int] = ()):
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_batch_seqs = max_batch_seqs
        self.max_model_len = max_model_len
        self.chunk = chunked_prefill_size
        self.eos = set(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # admission order
        self.finished: List[Request] = []
        self._admissions = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------------ requests
    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        if len(request.prompt) >= self.max_model_len:
            raise ValueError(f"request {request.request_id!r}: prompt of {len(request.prompt)} tokens leaves "
                             f"no room under max_model_len {self.max_model_len}")
        self.waiting.append(request)

    def abort(self, request: Request) -> None:
        if request in self.waiting:
            self.waiting.remove(request)
            request.state, request.finish_reason = FINISHED, "aborted"
        elif request in self.running:
            self._fail(request, "aborted")

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------------ planning
    def _free_after(self, taken: Dict[int, int]) -> Dict[int, int]:
        free = self.cache.free_pages()
        return {g: free[g] - taken.get(g, 0) for g in free}

    def _fits(self, need: Dict[int, int], taken: Dict[int, int]) -> bool:
        free = self._free_after(taken)
        return all(need[g] <= free[g] for g in need)

    @staticmethod
    def _take(need: Dict[int, int], taken: Dict[int, int]) -> None:
        for g, k in need.items():
            taken[g] = taken.get(g, 0) + k

    def _largest_portion(self, req: Request, want: int, taken: Dict[int, int], fresh: bool) -> int:
        """Most tokens (<= want) of `req` the free pages can hold; 0 if not even one."""
        page = self.cache.page_size
        n = want
        while n > 0:
            need = self.cache.pages_needed_fresh(n) if fresh else self.cache.pages_needed(req.request_id, n)
            if self._fits(need, taken):
                return n
            held = 0 if fresh else self.cache.length(req.request_id)
            # drop to the end of the previous page
            n = ((held + n - 1) // page) * page - held
        return 0

    def _preempt(self, victim: Request, plan: StepPlan) -> None:
        self.cache.close(victim.request_id)
        self.running.remove(victim)
        victim.state = WAITING
        victim.computed = 0
        victim.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim.request_id)

    def schedule(self, _gave_way: Sequence[Any] = ()) -> StepPlan:
        """The next step's batch.  `_gave_way`: requests a first pass of this very call
        preempted (the call starts over once when nothing could move); they count as
        preempted by the plan that is returned and are not admitted again by it."""
        plan = StepPlan([], list(_gave_way))
        taken: Dict[int, int] = {}
        budget = self.max_batch_tokens

        # 1. decode rows, oldest first; make room by preempting the youngest
        for req in list(self.running):
            if req.state != DECODE or req not in self.running:
                continue
            while True:
                need = self.cache.pages_needed(req.request_id, 1)
                if self._fits(need, taken):
                    self._take(need, taken)
                    plan.entries.append(PlannedEntry(req, req.computed, 1, True))
                    budget -= 1
                    break
                victims = [r for r in self.running if r is not req
                           and not any(e.request is r for e in plan.entries)]
                if victims:
                    self._preempt(max(victims, key=lambda r: r.admitted_at), plan)
                elif len(self.running) > 1:
                    self._preempt(req, plan)        # the youngest left is this one: it gives way
                    break
                else:
                    # alone in the pool and still short: it can never grow here
                    self._fail(req, "kv_pool_exhausted")
                    break

        # 2. next portions of prompts that are under way
        for req in self.running:
            if req.state != PREFILL or budget <= 0:
                continue
            want = min(req.remaining, budget, self.chunk or req.remaining)
            n = self._largest_portion(req, want, taken, fresh=False)
            if n <= 0:
                continue
            self._take(self.cache.pages_needed(req.request_id, n), taken)
            plan.entries.append(PlannedEntry(req, req.computed, n, n == req.remaining))
            budget -= n

        # 3. admissions, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_batch_seqs \
                and self.cache.slots.free_count > 0:
            req = self.waiting[0]
            if req.request_id in plan.preempted:          # it just gave way; not back in the same step
                break
            if req.undelivered:
                # it gave way while a token of its own was still on the way to the host: its
                # sequence is not complete yet, so it cannot be recomputed before that arrives
                break
            total = len(req.prompt) + len(req.output)
            if any(k > self.cache.pools[g].num_pages
                   for g, k in self.cache.pages_needed_fresh(total + 1).items()):
                # would not fit even with the pool to itself
                self.waiting.popleft()
                self._fail(req, "kv_pool_exhausted", opened=False)
                continue
            want = min(req.remaining, budget, self.chunk or req.remaining)
            # keep a page in hand for every decoding request, so that an admission does not
            # at once force a preemption
            reserve = {g: sum(1 for r in self.running if r.state == DECODE) for g in self.cache.pools}
            self._take(reserve, taken)
            n = self._largest_portion(req, want, taken, fresh=True)
            self._take({g: -k for g, k in reserve.items()}, taken)
            if n <= 0:
                break
            self.waiting.popleft()
            self.cache.open(req.request_id)
            req.state = PREFILL
            req.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(req)
            self._take(self.cache.pages_needed(req.request_id, n), taken)
            plan.entries.append(PlannedEntry(req, req.computed, n, n == req.remaining))
            budget -= n

        # 4. nothing can move although requests are under way: the youngest gives way
        if not plan.entries and any(r.state in (PREFILL, DECODE) for r in self.running):
            if len(self.running) == 1:
                self._fail(self.running[0], "kv_pool_exhausted")
            else:
                self._preempt(max(self.running, key=lambda r: r.admitted_at), plan)
            return self.schedule(plan.preempted) if self.has_work() else plan
        return plan

    # ------------------------------------------------------------------ after the step
    def _fail(self, req: Request, reason: str, opened: bool = True) -> None:
        if opened and self.cache.is_open(req.request_id):
            self.cache.close(req.request_id)
        if req in self.running:
            self.running.remove(req)
        req.state = FINISHED
        req.finish_reason = reason
        self.finished.append(req)

    def complete_step(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """`sampled[i]` is the token chosen for the i-th entry of the plan that samples.
        The step function has already committed the tokens to the cache.  Returns the
        requests that finished with this step."""
        self.advance(plan)
        return self.deliver(plan, sampled)

    def advance(self, plan: StepPlan) -> None:
        """The step has been launched: count its tokens as computed.  What it chose is not
        known yet (`deliver` brings it), so the next step can be planned, and launched with
        the chosen tokens fed on the device, before the host has read them.  A request whose
        chosen token is its last by length runs no further (`DRAINING`)."""
        for e in plan.entries:
            req = e.request
            req.computed += e.count
            if not e.samples:
                continue
            req.undelivered += 1
            req.state = DECODE
            made = len(req.output) + req.undelivered
            if made >= req.params.max_tokens or len(req.prompt) + made >= self.max_model_len:
                req.state = DRAINING

    def deliver(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """The tokens of a launched step have reached the host.  A request that already
        finished (a stop token in an earlier delivery, while this step was in flight) ignores
        what this step chose for it."""
        done: List[Request] = []
        it = iter(sampled)
        for e in plan.entries:
            if not e.samples:
                continue
            req = e.request
            tok = int(next(it))
            if req.state == FINISHED:
                continue
            req.undelivered -= 1
            req.output.append(tok)
            # crates/infer-worker/src/application/runtime/mod.rs:1198-1214: eos unless ignored,
            # or the count of generated tokens reaches max_tokens (the first token counts)
            if tok in self.eos and not req.params.ignore_eos:
                req.finish_reason = "stop"
            elif len(req.output) >= req.params.max_tokens:
                req.finish_reason = "length"
            elif len(req.prompt) + len(req.output) >= self.max_model_len:
                req.finish_reason = "length"
            if req.finish_reason:
                if self.cache.is_open(req.request_id):
                    self.cache.close(req.request_id)
                if req in self.running:
                    self.running.remove(req)
                elif req in self.waiting:              # it gave way while its last token was in flight
                    self.waiting.remove(req)
                req.state = FINISHED
                self.finished.append(req)
                done.append(req)
        return done
