"""The step function.

`Engine.step(entries)` takes a batch of (request, its next tokens, wanted rows):
portions of prompts beside single decoded tokens, cut anywhere.  It runs only the
tokens it is given, as one batch, against the cache that earlier steps left, and
returns the logits at the wanted places.  A step either runs completely or
changes nothing (pages reserved for it are handed back if it cannot run).

Counterpart in giveen/spite: `Executor::prefill` / `decode_step`
(crates/spite-executor/src/lib.rs:230-277), one sequence at a time, every logit
row computed; errors follow `ExecutorError` (lib.rs:88-100).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache import CacheError, CacheStorage, OutOfPages, OutOfSlots
from .batch import Segment, build_step_batch


class StepError(ValueError):
    """The step's entries are malformed (nothing ran)."""


class ContextOverflow(StepError):
    """A request would pass the model's position limit (lib.rs:96-97 `ContextOverflow`)."""


@dataclass
class StepEntry:
    req_id: object
    tokens: list
    want: list          # indices into `tokens` whose logits are asked for


class Engine:
    def __init__(self, model, *, cache_tokens: int, page_size: int = 64, max_requests: int = 64,
                 max_positions: int | None = None):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.model = model
        self.page_size = page_size
        self.n_pages = max(1, -(-int(cache_tokens) // page_size))
        self.max_positions = int(max_positions or model.plan.max_positions)
        self.storage = CacheStorage(model.cache_specs(), page_size, self.n_pages, max_requests,
                                    model.dtype, model.device)
        self.cache = self.storage.manager
        self.steps_run = 0
        self.tokens_run = 0

    # ------------------------------------------------------------------ requests
    def is_live(self, req_id) -> bool:
        return req_id in self.cache.requests

    def cached_tokens(self, req_id) -> int:
        return self.cache.get(req_id).n_tokens

    def finish(self, req_id):
        """The request ends; its pages and slot go back to the pools."""
        self.cache.release(req_id)

    def can_run(self, wants: dict) -> bool:
        """Would the pools supply {request: number of new tokens} together?"""
        new = sum(1 for r in wants if r not in self.cache.requests)
        return new <= self.cache.slots.n_free and self.cache.can_reserve(wants)

    # ------------------------------------------------------------------ the step
    def step(self, entries) -> torch.Tensor:
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        vocab = self.model.plan.vocab_size
        seen = set()
        for e in entries:
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if len(e.tokens) < 1:
                raise StepError(f"request {e.req_id!r} brings no tokens")
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise StepError(f"request {e.req_id!r}: token id {t} outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"request {e.req_id!r}: wanted row {w} outside its {len(e.tokens)} tokens")
            have = self.cache.requests[e.req_id].n_tokens if e.req_id in self.cache.requests else 0
            if have + len(e.tokens) > self.max_positions:
                raise ContextOverflow(
                    f"request {e.req_id!r}: {have} cached + {len(e.tokens)} new tokens exceed the "
                    f"limit of {self.max_positions} positions")
        if not entries:
            return torch.empty((0, vocab), dtype=torch.float32, device=self.model.device)

        admitted, reserved = [], []
        try:
            for e in entries:
                if e.req_id not in self.cache.requests:
                    self.cache.admit(e.req_id)
                    admitted.append(e.req_id)
            for e in entries:
                self.cache.reserve(e.req_id, len(e.tokens))
                reserved.append(e.req_id)
        except (OutOfPages, OutOfSlots):
            for r in reserved:
                self.cache.rollback(r)
            for r in admitted:
                self.cache.release(r)
            raise

        segments, offset = [], 0
        for e in entries:
            rc = self.cache.requests[e.req_id]
            segments.append(Segment(e.req_id, rc.slot, rc.n_tokens, len(e.tokens), offset, rc.fresh))
            offset += len(e.tokens)
            if rc.fresh and self.storage.state:
                self.storage.clear_state(rc.slot)
        tables = [[self.cache.requests[e.req_id].tables[g] for e in entries]
                  for g in range(self.storage.n_groups)]
        batch = build_step_batch(segments, [e.tokens for e in entries], [e.want for e in entries],
                                 tables, self.model.device)
        try:
            logits = self.model.forward(batch, self.storage)
        except Exception:
            for r in reserved:
                self.cache.rollback(r)
            for r in admitted:
                self.cache.release(r)
            raise
        for e in entries:
            self.cache.commit(e.req_id)
        self.steps_run += 1
        self.tokens_run += offset
        return logits
