"""The scheduler above the step function: it admits requests, cuts prompts into
portions under a token budget, decodes, finishes and frees.

Every step is planned like this:
  1. every generating request contributes its one next token;
  2. the rest of the token budget goes to prompt portions: first the requests
     already admitted (oldest first), then waiting ones in arrival order, each
     `min(rest of its prompt, rest of the budget, max_portion)` tokens, as long
     as a slot is free and the pages for the portion can be supplied;
  3. a request whose prompt ends in this step samples its first token from
     this step's logits.
When pages run out for the decoding requests, the most recently admitted
request is preempted: its pages and slot are freed and it goes back to the head
of the waiting queue with prompt := prompt + tokens generated so far (its
generator state is kept, so it samples what it would have sampled).  A request
that is alone and still cannot get a page ends with reason `cache_full`.  The
rule is deterministic.

Counterpart in giveen/spite: the scheduler skeleton (slot table, `BatchRequest`,
`BatchOutput`, `FinishReason`; `step` unimplemented,
crates/spite-scheduler/src/lib.rs:30-152) and the generate loop's stopping rule
(an end-of-generation token is not emitted; crates/spite-executor/src/lib.rs:667-676).
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field

from ..sampling.sampler import SampleRow, SamplingParams
from .executor import ContextOverflow, StepEntry


class FinishReason(enum.Enum):
    NOT_DONE = "not_done"
    EOS_TOKEN = "eos_token"
    STOP_TOKEN = "stop_token"
    MAX_TOKENS = "max_tokens"
    CONTEXT_FULL = "context_full"
    CACHE_FULL = "cache_full"


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    GENERATING = "generating"
    DONE = "done"


@dataclass
class Request:
    id: object
    prompt: list
    params: SamplingParams = field(default_factory=SamplingParams)
    state: RequestState = RequestState.WAITING
    output: list = field(default_factory=list)
    finish_reason: FinishReason = FinishReason.NOT_DONE
    n_fed: int = 0              # tokens of prompt + output whose keys are cached
    rng_state: int = 0
    preemptions: int = 0

    def all_tokens(self) -> list:
        return self.prompt + self.output


@dataclass
class StepOutput:
    request_id: object
    token: int | None           # None when the request ended without emitting a token
    done: bool
    finish_reason: FinishReason


@dataclass
class StepPlan:
    entries: list               # (Request, tokens, wants the last row's logits)
    preempted: list             # Requests sent back to the waiting queue
    ended: list                 # (Request, FinishReason) ended by the plan itself


class Scheduler:
    def __init__(self, engine, sampler, *, max_batch_tokens: int = 2048, max_portion: int | None = None,
                 ctx: int | None = None, eos_token_ids=()):
        if max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be positive")
        self.engine = engine
        self.sampler = sampler
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_portion = int(max_portion or max_batch_tokens)
        self.ctx = int(ctx or engine.max_positions)
        self.eos = frozenset(int(t) for t in (eos_token_ids or ()))
        self.waiting: deque = deque()
        self.running: list = []          # in order of admission
        self.finished: dict = {}
        self.counters = {"steps": 0, "tokens": 0, "preemptions": 0}

    # ------------------------------------------------------------------ intake
    def submit(self, request: Request):
        request.params.validate()
        if not request.prompt:
            raise ValueError(f"request {request.id!r} has an empty prompt")
        if len(request.prompt) > self.ctx:
            raise ContextOverflow(f"request {request.id!r}: prompt of {len(request.prompt)} tokens exceeds "
                                  f"the context of {self.ctx}")
        cache = self.engine.cache
        need = -(-(len(request.prompt) + 1) // cache.page_size)
        if any(need > pool.n_pages for pool, key in zip(cache.pools, cache.groups) if key.window.kind == "full"):
            raise ContextOverflow(f"request {request.id!r}: its prompt needs {need} pages, the pool has "
                                  f"{min(p.n_pages for p in cache.pools)}")
        request.rng_state = request.params.seed & ((1 << 64) - 1)
        if request.params.max_tokens == 0:
            self._finish(request, FinishReason.MAX_TOKENS)
            return
        request.state = RequestState.WAITING
        self.waiting.append(request)

    def active_count(self) -> int:
        return len(self.waiting) + len(self.running)

    # ------------------------------------------------------------------ planning
    def plan_step(self) -> StepPlan:
        cache = self.engine.cache
        preempted, ended = [], []
        while True:
            decodes = [r for r in self.running if r.state is RequestState.GENERATING]
            wants = {r.id: 1 for r in decodes}
            if not decodes or cache.can_reserve(wants):
                break
            victim = self.running[-1]
            if len(self.running) == 1:
                ended.append((victim, FinishReason.CACHE_FULL))
                self._finish(victim, FinishReason.CACHE_FULL)
                continue
            self._preempt(victim)
            preempted.append(victim)

        entries = [(r, [r.all_tokens()[r.n_fed]], True) for r in decodes]
        budget = self.max_batch_tokens - len(entries)
        wants = {r.id: 1 for r in decodes}

        def try_portion(r) -> bool:
            nonlocal budget
            toks = r.all_tokens()
            n = min(len(toks) - r.n_fed, budget, self.max_portion)
            if n < 1:
                return False
            trial = dict(wants)
            trial[r.id] = n
            if not self.engine.can_run(trial):
                return False
            wants[r.id] = n
            budget -= n
            entries.append((r, toks[r.n_fed:r.n_fed + n], r.n_fed + n == len(toks)))
            return True

        for r in self.running:
            if r.state is RequestState.PREFILLING and budget > 0:
                try_portion(r)
        while self.waiting and budget > 0 and not preempted:
            r = self.waiting[0]
            if not try_portion(r):
                break                       # arrival order is kept: nobody overtakes the head
            self.waiting.popleft()
            r.state = RequestState.PREFILLING
            self.running.append(r)
        return StepPlan(entries, preempted, ended)

    def _preempt(self, r: Request):
        if self.engine.is_live(r.id):
            self.engine.finish(r.id)
        self.running.remove(r)
        r.n_fed = 0
        r.state = RequestState.WAITING
        r.preemptions += 1
        self.counters["preemptions"] += 1
        self.waiting.appendleft(r)

    def _finish(self, r: Request, reason: FinishReason):
        if self.engine.is_live(r.id):
            self.engine.finish(r.id)
        if r in self.running:
            self.running.remove(r)
        r.state = RequestState.DONE
        r.finish_reason = reason
        self.finished[r.id] = r

    # ------------------------------------------------------------------ running
    def step(self) -> list:
        """Plan and run one step; returns what each request produced in it."""
        plan = self.plan_step()
        outputs = [StepOutput(r.id, None, True, why) for r, why in plan.ended]
        if not plan.entries:
            return outputs
        logits = self.engine.step([StepEntry(r.id, toks, [len(toks) - 1] if want else [])
                                   for r, toks, want in plan.entries])
        self.counters["steps"] += 1
        sampled = []
        for r, toks, want in plan.entries:
            r.n_fed += len(toks)
            self.counters["tokens"] += len(toks)
            if want:
                sampled.append(r)
        tokens, states = self.sampler.sample(
            logits, [SampleRow(r.params, r.all_tokens(), r.rng_state) for r in sampled])
        for r, tok, st in zip(sampled, tokens, states):
            r.rng_state = st
            outputs.append(self._accept(r, int(tok)))
        return outputs

    def _accept(self, r: Request, tok: int) -> StepOutput:
        # an end-of-generation token ends the request and is not emitted
        if tok in self.eos:
            self._finish(r, FinishReason.EOS_TOKEN)
            return StepOutput(r.id, None, True, FinishReason.EOS_TOKEN)
        if tok in r.params.stop_token_ids:
            self._finish(r, FinishReason.STOP_TOKEN)
            return StepOutput(r.id, None, True, FinishReason.STOP_TOKEN)
        r.output.append(tok)
        r.state = RequestState.GENERATING
        if len(r.output) >= r.params.max_tokens:
            self._finish(r, FinishReason.MAX_TOKENS)
            return StepOutput(r.id, tok, True, FinishReason.MAX_TOKENS)
        if len(r.prompt) + len(r.output) >= self.ctx:
            self._finish(r, FinishReason.CONTEXT_FULL)
            return StepOutput(r.id, tok, True, FinishReason.CONTEXT_FULL)
        return StepOutput(r.id, tok, False, FinishReason.NOT_DONE)

    def run_until_done(self, max_steps: int | None = None) -> dict:
        steps = 0
        while self.active_count():
            before = (self.counters["steps"], len(self.finished))
            self.step()
            steps += 1
            if (self.counters["steps"], len(self.finished)) == before:
                raise RuntimeError("the scheduler made no progress: no request fits the cache")
            if max_steps is not None and steps >= max_steps:
                break
        return self.finished
