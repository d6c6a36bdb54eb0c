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

import collections
from dataclasses import dataclass

import torch

from ..cache import CacheError, CacheStorage, OutOfPages, OutOfSlots
from ..kernels.api import KernelTimeout
from .batch import Segment, StaticDecodeBatch, build_step_batch


class StepError(ValueError):
    """The step's entries are malformed (nothing ran)."""


_LIBRARY_CODES = "1: a loader waited for a free stage, 2: the tensor-core issuer or a consumer waited for data, " \
                 "3: an epilogue or softmax warp waited for a result, 4: the issuer waited for a free accumulator"


class ContextOverflow(StepError):
    """A request would pass the model's position limit (lib.rs:96-97 `ContextOverflow`)."""


@dataclass
class StepEntry:
    req_id: object
    tokens: list
    want: list          # indices into `tokens` whose logits are asked for


class Engine:
    def __init__(self, model, *, cache_tokens: int, page_size: int = 64, max_requests: int = 64,
                 max_positions: int | None = None, cuda_graphs: bool | None = None, max_graphs: int = 32):
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
        # Decode steps (one token per request) are launch-bound: their kernels are captured in
        # a CUDA graph per (rows, context bucket) and replayed.  The number of requests is rounded up
        # to one of a few row counts, so that a batch whose requests end one by one walks through few
        # shapes; the least recently used graph goes when there are more than `max_graphs`.
        if cuda_graphs is None:
            cuda_graphs = model.device.type == "cuda" and model.graph_safe()
        self.cuda_graphs = bool(cuda_graphs)
        self.max_graphs = max(1, int(max_graphs))
        self._graphs: collections.OrderedDict = collections.OrderedDict()
        self._graph_pool = None             # one memory pool for all captures: only one graph's results live at a time
        self.graph_replays = 0
        self.graph_captures = 0

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

    def check(self):
        """Raise `KernelTimeout` if a kernel of an earlier step gave up one of its bounded waits and left
        its output incomplete.  It reads a word that the device writes into host memory and does not
        wait for the device, so it reports on the steps the host has already waited for (by reading
        their logits or sampled ids); `step` calls it for the steps before, the scheduler after every
        read of sampled ids, `bin/trace_run` after every read of logits."""
        errors = self.model.kernels.errors()
        if errors:
            what = ", ".join(f"{lib} (code {code})" for lib, code in sorted(errors.items()))
            raise KernelTimeout(f"a kernel gave up waiting and left its results incomplete: {what}; {_LIBRARY_CODES}. "
                                f"The logits and cached keys of the steps since the last check are not valid.")

    # ------------------------------------------------------------------ the step
    def step(self, entries, device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run one step.  `device_tokens` (int32 [len(entries)] on the device), if given, supplies the
        token of every entry from the device (the ids sampled by the step before, which the host has
        not read yet); every entry then brings one placeholder token, and the step must be one that
        is a decode step (one token an entry)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self.check()
        vocab = self.model.plan.vocab_size
        if device_tokens is not None:
            if any(len(e.tokens) != 1 for e in entries):
                raise StepError("tokens from the device need a decode step: one token an entry")
            if device_tokens.dtype != torch.int32 or device_tokens.numel() != len(entries):
                raise StepError("device_tokens must be int32 with one id per entry")
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

        fresh_pages = [[] for _ in range(self.storage.n_groups)]
        for e in entries:
            for g, pages in enumerate(self.cache.pending_pages(e.req_id)):
                fresh_pages[g] += pages
        self.storage.clear_pages(self.model.kernels, fresh_pages)

        segments, offset = [], 0
        for e in entries:
            rc = self.cache.requests[e.req_id]
            segments.append(Segment(e.req_id, rc.slot, rc.n_tokens, len(e.tokens), offset, rc.fresh))
            offset += len(e.tokens)
            if rc.fresh and self.storage.state:
                self.storage.clear_state(rc.slot)
        tables = [[self.cache.requests[e.req_id].tables[g] for e in entries]
                  for g in range(self.storage.n_groups)]
        try:
            if self.cuda_graphs and all(len(e.tokens) == 1 for e in entries):
                logits = self._decode_step_from_graph(segments, [e.tokens[0] for e in entries], tables, device_tokens)
                rows = [i for i, e in enumerate(entries) if e.want]
                if len(rows) < len(entries):
                    logits = logits[torch.tensor(rows, dtype=torch.long, device=logits.device)]
            else:
                batch = build_step_batch(segments, [e.tokens for e in entries], [e.want for e in entries],
                                         tables, self.model.device)
                if device_tokens is not None:
                    batch.token_ids.copy_(device_tokens)
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

    # ------------------------------------------------------------------ decode steps from CUDA graphs
    @staticmethod
    def decode_rows(n_requests: int) -> int:
        """Rows of the captured decode step that serves `n_requests`: every count up to 8, then steps of
        an eighth to a quarter of the count (10, 12, 14, 16, 20, ..., 32, 40, ..., 64, 80, ...)."""
        if n_requests <= 8:
            return n_requests
        step = 1 << ((n_requests - 1).bit_length() - 3)
        return -(-n_requests // step) * step

    def _decode_step_from_graph(self, segments, tokens, tables, device_tokens=None) -> torch.Tensor:
        """A step of single tokens.  The first step of a shape runs eagerly (it loads and warms
        every kernel), the second is captured, later ones replay the capture.  The returned
        logits live in memory that all captured steps share: they are valid until the next step."""
        n = len(segments)
        S = self.decode_rows(n)
        longest = max(s.start_pos for s in segments) + 1
        bucket = max(128, 1 << (longest - 1).bit_length())
        key = (S, bucket)
        st = self._graphs.get(key)
        if st is None:
            while len(self._graphs) >= self.max_graphs:
                # a replay of the graph that goes may still be running, and its buffers are about to be freed
                torch.cuda.current_stream(self.model.device).synchronize()
                self._graphs.popitem(last=False)
            width = -(-self.max_positions // self.page_size)
            st = _GraphState(StaticDecodeBatch(S, [width] * self.storage.n_groups, self.model.device, bucket))
            self._graphs[key] = st
        else:
            self._graphs.move_to_end(key)
        batch = st.static.fill(segments, tokens, tables)
        if device_tokens is not None:                         # stream-ordered after the copy from the host
            batch.token_ids[:n].copy_(device_tokens)
            if S > n:
                batch.token_ids[n:].copy_(device_tokens[:1].expand(S - n))
        if st.graph is None:
            if st.eager_runs == 0:
                st.eager_runs = 1
                return self.model.forward(batch, self.storage)[:n]
            graph = torch.cuda.CUDAGraph()
            counted = getattr(self.model.kernels, "launches", 0)
            with torch.cuda.graph(graph, pool=self._graph_pool):
                st.logits = self.model.forward(batch, self.storage)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            st.graph = graph
            self.graph_captures += 1
            if hasattr(self.model.kernels, "launches"):          # captured, not run: count them per replay
                st.n_kernels = self.model.kernels.launches - counted
                self.model.kernels.launches = counted
        st.graph.replay()
        if st.n_kernels:
            self.model.kernels.launches += st.n_kernels
        self.graph_replays += 1
        return st.logits[:n]


class _GraphState:
    def __init__(self, static):
        self.static = static
        self.graph = None
        self.logits = None
        self.eager_runs = 0
        self.n_kernels = 0
