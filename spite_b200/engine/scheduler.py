"""The scheduler above the step function: it admits requests, cuts prompts into
portions under a token budget, decodes, finishes and frees.

Every step is planned like this:
  1. every generating request contributes its one next token;
  2. the rest of the token budget goes to prompt portions: first the requests
     already admitted (oldest first), then waiting ones in arrival order, each
     `min(rest of its prompt, rest of the budget, max_portion)` tokens, or as
     many of them as the free pages hold; a waiting request is admitted while a
     slot is free and the groups that keep every key have room for its whole
     prompt beside what the running requests still need;
  3. a request whose prompt ends in this step samples its first token from
     this step's logits.
When pages run out for the decoding requests, or no admitted request can run
at all (prompts in progress hold the pages each of them needs next), the most
recently admitted request is preempted: its pages and slot are freed and it goes back to the head
of the waiting queue with prompt := prompt + tokens generated so far (its
generator state is kept, so it samples what it would have sampled).  A request
that is alone and still cannot get a page ends with reason `cache_full`.  The
rule is deterministic.

Decoding ahead.  On a GPU, when a step is made of decoded tokens only, the scheduler does not wait
for the sampled ids: it leaves the step in flight (argmax or the sampling kernel on the device, a
copy to pinned memory under way) and launches the next step with the ids taken from the device,
so the GPU never waits for the host between decode steps.  A request's generator state advances on
the host by the same rule as on the device, and a repetition penalty finds the one token the host
has not read yet on the device.  The ids are read one step late.  What
the late reading changes: a request that ends on an end-of-generation or stop token has one more
step run for it, whose row is thrown away (its cache is freed as usual; rows of a batch do not
depend on each other), and a waiting request is admitted one step later than it could have been.
Ends by token count are known ahead and are not run past.  Whenever the next step is not such a
step (a prompt portion to run, a request to admit, pages to find by preemption), the step in
flight is read first and the plain path above takes over.  The tokens produced are the same.

Counterpart in giveen/spite: the scheduler skeleton (slot table, `BatchRequest`,
`BatchOutput`, `FinishReason`; `step` unimplemented,
crates/spite-scheduler/src/lib.rs:30-152) and the generate loop's stopping rule
(an end-of-generation token is not emitted; crates/spite-executor/src/lib.rs:667-676).
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field

from ..kernels.api import KernelTimeout
from ..sampling.sampler import SampleRow, SamplingParams, lcg_advance
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


@dataclass
class _InFlight:
    """A decode step whose sampled ids are still on the device."""
    requests: list              # row i of `device_tokens` belongs to requests[i]
    device_tokens: object       # int32 [R] on the device
    host_tokens: object         # pinned int32 buffer the copy lands in
    copied: object              # event recorded after the copy
    dead: set = field(default_factory=set)   # ids of requests that ended before this step was read


class Scheduler:
    def __init__(self, engine, sampler, *, max_batch_tokens: int = 2048, max_portion: int | None = None,
                 ctx: int | None = None, eos_token_ids=(), decode_ahead: bool | None = None):
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
        self.counters = {"steps": 0, "tokens": 0, "preemptions": 0, "steps_ahead": 0}
        if decode_ahead is None:
            decode_ahead = bool(getattr(engine, "cuda_graphs", False))
        self.decode_ahead = bool(decode_ahead)
        self._in_flight: _InFlight | None = None
        self._pinned: list = []          # two pinned id buffers, used in turn

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

    # ------------------------------------------------------------------ decoding ahead
    def _ends_by_count(self, r: Request) -> bool:
        """Will the token that is in flight for `r` be its last (by max_tokens or the context)?"""
        n = len(r.output) + 1
        return n >= r.params.max_tokens or len(r.prompt) + n >= self.ctx

    def _leave_in_flight(self, requests, logits, pending=None) -> _InFlight:
        """Sample on the device and start the copy of the ids to the host; `pending`: see `Sampler.sample_on_device`."""
        import torch
        ids, states = self.sampler.sample_on_device(
            logits, [SampleRow(r.params, r.all_tokens(), r.rng_state) for r in requests], pending)
        for r, st in zip(requests, states):
            r.rng_state = st
        if not self._pinned:                 # two buffers: one step is read while the next one's copy runs
            n = max(len(requests), self.engine.cache.slots.n_slots)
            self._pinned = [torch.empty(n, dtype=torch.int32) for _ in range(2)]
            if ids.is_cuda:
                self._pinned = [t.pin_memory() for t in self._pinned]
        self._pinned.reverse()
        host = self._pinned[0]
        host[:len(requests)].copy_(ids, non_blocking=True)
        copied = None
        if ids.is_cuda:
            copied = torch.cuda.Event()
            copied.record()
        return _InFlight(list(requests), ids, host, copied)

    def _read(self, step: _InFlight) -> list:
        """Wait for the ids of a step in flight and take them in."""
        if step.copied is not None:
            step.copied.synchronize()
        self._check_kernels()
        tokens = step.host_tokens[:len(step.requests)].tolist()
        return [self._accept(r, int(tok)) for r, tok in zip(step.requests, tokens) if r.id not in step.dead]

    def _launch_ahead(self) -> _InFlight | None:
        """The step after the one in flight, if it is a pure decode step of requests of that one."""
        cur = self._in_flight
        go_on = [r for r in cur.requests if r.id not in cur.dead and not self._ends_by_count(r)]
        if not go_on or len(self.running) != len([r for r in cur.requests if r.id not in cur.dead]):
            return None                      # nothing left to decode, or someone else (a prompt) is running
        cache = self.engine.cache
        wants = {r.id: 1 for r in go_on}
        if not cache.can_reserve(wants):
            return None                      # pages must be found by preemption: the plain path decides
        if self.waiting:
            head = self.waiting[0]
            n = min(len(head.all_tokens()), self.max_batch_tokens - len(go_on), self.max_portion)
            if n >= 1 and self._room_for_whole_prompt(head) and self._fit(head, n, wants):
                return None                  # the head of the queue can be admitted now
        import torch
        ids = cur.device_tokens
        if len(go_on) != len(cur.requests):
            rows = [i for i, r in enumerate(cur.requests) if r in go_on]
            ids = ids[torch.tensor(rows, dtype=torch.long, device=ids.device)]
        logits = self.engine.step([StepEntry(r.id, [0], [0]) for r in go_on], device_tokens=ids)
        self.counters["steps"] += 1
        self.counters["steps_ahead"] += 1
        self.counters["tokens"] += len(go_on)
        for r in go_on:
            r.n_fed += 1
        # the token a request got from the step in flight is still on the device: the repetition penalty reads it there
        return self._leave_in_flight(go_on, logits, (cur.device_tokens, [cur.requests.index(r) for r in go_on]))

    # ------------------------------------------------------------------ planning
    def _fit(self, r: Request, n: int, wants: dict) -> int:
        """Most tokens, up to `n`, of request `r` that the pools can supply beside `wants` (0: none)."""
        if n < 1 or not self.engine.can_run({**wants, r.id: 1}):
            return 0
        if self.engine.can_run({**wants, r.id: n}):
            return n
        lo, hi = 1, n                        # lo fits, hi does not; more tokens never need fewer pages
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self.engine.can_run({**wants, r.id: mid}):
                lo = mid
            else:
                hi = mid
        return lo

    def _room_for_whole_prompt(self, head: Request) -> bool:
        """Admission rule: beside what the running requests still need to finish their prompts and
        take one decoded token, the groups that keep every key have the pages for the whole prompt
        of `head` and its first token.  Two prompts admitted into a pool that holds neither of them
        to the end would only take pages from each other.  With nothing running the head is always
        admitted: it then gets the pool to itself."""
        if not self.running:
            return True
        cache = self.engine.cache
        need = [0] * len(cache.groups)
        for r in self.running + [head]:
            rest = len(r.all_tokens()) - r.n_fed + (0 if r.state is RequestState.GENERATING else 1)
            for g, k in enumerate(cache.pages_needed(r.id, max(rest, 1))):
                need[g] += k
        return all(n <= pool.n_free for n, pool, key in zip(need, cache.pools, cache.groups)
                   if key.window.kind == "full")

    def plan_step(self) -> StepPlan:
        cache = self.engine.cache
        preempted, ended = [], []
        while True:
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

            def try_portion(r) -> bool:
                nonlocal budget
                toks = r.all_tokens()
                n = self._fit(r, min(len(toks) - r.n_fed, budget, self.max_portion), wants)
                if n < 1:
                    return False
                wants[r.id] = n
                budget -= n
                entries.append((r, toks[r.n_fed:r.n_fed + n], r.n_fed + n == len(toks)))
                return True

            for r in self.running:
                if r.state is RequestState.PREFILLING and budget > 0:
                    try_portion(r)
            if entries or not self.running:
                break
            # Nothing can run although requests are admitted: prompts in progress hold the pages that
            # each of them needs next.  The most recently admitted one gives way (it is recomputed
            # later); a request that is alone and still gets no page cannot be served by this pool.
            victim = self.running[-1]
            if len(self.running) == 1:
                ended.append((victim, FinishReason.CACHE_FULL))
                self._finish(victim, FinishReason.CACHE_FULL)
                break
            self._preempt(victim)
            preempted.append(victim)
        while self.waiting and budget > 0 and not preempted:
            r = self.waiting[0]
            if not self._room_for_whole_prompt(r) or not try_portion(r):
                break                       # arrival order is kept: nobody overtakes the head
            self.waiting.popleft()
            r.state = RequestState.PREFILLING
            self.running.append(r)
        return StepPlan(entries, preempted, ended)

    def _check_kernels(self):
        """Called when the host has just waited for a step's ids, before it takes them in."""
        self.engine.check()

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
        """Plan and run one step; returns what each request produced (with decoding ahead: what was
        read in this call, which is the step before the one launched).

        If a kernel gave up a bounded wait (`KernelTimeout`, noticed when the host has a step's ids or
        starts the next step), nothing of the steps in flight is kept: every running request gives its
        pages back and returns to the queue with the tokens it had, to be recomputed when it runs again,
        and the error goes to the caller, who may go on calling `step`."""
        try:
            return self._step()
        except KernelTimeout:
            self._in_flight = None
            for r in list(reversed(self.running)):
                if r.params.temperature > 0:
                    # a token that was in flight is lost with its draw: the generator goes back to one draw
                    # for every token the request has
                    r.rng_state = r.params.seed & ((1 << 64) - 1)
                    for _ in r.output:
                        r.rng_state = lcg_advance(r.rng_state)
                self._preempt(r)
            raise

    def _step(self) -> list:
        outputs = []
        if self._in_flight is not None:
            ahead = self._launch_ahead()
            outputs = self._read(self._in_flight)
            if ahead is not None:
                ahead.dead = {r.id for r in ahead.requests if r.state is RequestState.DONE}
                if len(ahead.dead) == len(ahead.requests):
                    ahead = None                 # every request of the step launched ahead has just ended: nothing to read
            self._in_flight = ahead
            if ahead is not None or not self.active_count():
                return outputs
        plan = self.plan_step()
        outputs += [StepOutput(r.id, None, True, why) for r, why in plan.ended]
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
        if self.decode_ahead and len(sampled) == len(plan.entries) == len(self.running):
            # every running request gets a token from this step, sampled on the device:
            # leave the ids there and let the next call launch the next step before reading them
            self._in_flight = self._leave_in_flight(sampled, logits)
            return outputs
        tokens, states = self.sampler.sample(
            logits, [SampleRow(r.params, r.all_tokens(), r.rng_state) for r in sampled])
        self._check_kernels()                # the ids are on the host: the step has ended
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
