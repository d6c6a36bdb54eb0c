"""Sampling options and the batched sampler above the device kernels.

Options, their meaning and their defaults follow giveen/spite's `SamplerConfig`
(crates/spite-sampling/src/lib.rs:82-111) and the settings its `run` command
uses (`default_sampler_config`, crates/spite-executor/src/lib.rs:144-151):
temperature <= 0 is greedy decoding with the penalty off; above 0 a repetition
penalty of 1.1 over the last 64 tokens and top-p 0.95 apply.  Every request has
a 64-bit generator state of its own (lib.rs:343-348), advanced once per drawn
token, so what a request samples does not depend on what else is in the batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

DEFAULT_SEED = 0x1234_5678_9ABC_DEF0        # the constant of crates/spite-cli/src/main.rs:606
_MASK64 = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 0                   # 0: off
    top_p: float = 0.95              # 1: off
    min_p: float = 0.0               # 0: off
    repetition_penalty: float = 1.0  # 1: off
    repeat_last_n: int = 64          # 0: the whole context
    seed: int = 0
    max_tokens: int = 512
    stop_token_ids: tuple = ()

    def validate(self):
        if self.top_k < 0 or self.repeat_last_n < 0 or self.max_tokens < 0:
            raise ValueError("top_k, repeat_last_n and max_tokens must not be negative")
        if self.top_p <= 0.0:
            raise ValueError("top_p must be positive (1 or more switches it off)")
        if self.min_p < 0 or self.min_p > 1:
            raise ValueError("min_p must lie in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        return self


def run_sampling_params(temperature: float, *, seed: int = DEFAULT_SEED, max_tokens: int = 512,
                        stop_token_ids=()) -> SamplingParams:
    """What `spite run --temperature T` samples with (executor/src/lib.rs:144-151)."""
    return SamplingParams(temperature=temperature, repetition_penalty=1.1 if temperature > 0 else 1.0,
                          seed=seed, max_tokens=max_tokens, stop_token_ids=tuple(stop_token_ids))


def lcg_advance(state: int) -> int:
    """One step of the generator (crates/spite-sampling/src/lib.rs:343-348)."""
    return (state * 6364136223846793005 + 1442695040888963407) & _MASK64


def _signed(x: int) -> int:
    return x - (1 << 64) if x >= (1 << 63) else x


@dataclass
class SampleRow:
    params: SamplingParams
    context: list            # prompt + generated tokens so far (for the repetition penalty)
    rng_state: int           # unsigned 64-bit


def is_plain_greedy(params: SamplingParams) -> bool:
    """Greedy decoding that is the argmax alone: temperature 0 and no repetition penalty (the
    filters never remove the maximum)."""
    return params.temperature <= 0 and abs(params.repetition_penalty - 1.0) < 1.2e-7


class Sampler:
    def __init__(self, kernels):
        self.k = kernels
        self._buffers = []                    # pinned staging buffers, used in turn: [tensor, event of its last copy]
        self._turn = 0

    def _staging(self, n_words: int, dev) -> torch.Tensor:
        """A host buffer of at least `n_words` int32 whose last copy to the device has ended: pinned on a GPU
        (three in turn, so that filling one does not wait for the step that still reads another)."""
        if dev.type != "cuda":
            return torch.empty(n_words, dtype=torch.int32)
        if not self._buffers:
            self._buffers = [[None, None] for _ in range(3)]
        self._turn = (self._turn + 1) % len(self._buffers)
        slot = self._buffers[self._turn]
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < n_words:
            slot[0] = torch.empty(max(n_words, 4096), dtype=torch.int32).pin_memory()
        return slot[0]

    def _staged(self, dev):
        if dev.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._buffers[self._turn][1] = ev

    def greedy_on_device(self, logits: torch.Tensor) -> torch.Tensor:
        """The argmax of every row as int32 on the device; nothing is read back."""
        return self.k.argmax(logits)

    def sample(self, logits: torch.Tensor, rows: list) -> tuple[list, list]:
        """`logits` [R, vocab] float32 on the device, `rows` R `SampleRow`s.
        Returns (tokens, new generator states)."""
        if not rows:
            return [], []
        ids, states = self.sample_on_device(logits, rows)
        return ids.tolist(), states

    def sample_on_device(self, logits: torch.Tensor, rows: list, pending=None) -> tuple[torch.Tensor, list]:
        """The same, but the tokens stay on the device (int32 [R]) and nothing is read back: for a scheduler
        that launches the next step before it reads this one's ids.  `pending` = (ids, places): the last
        token of row i's context is not on the host yet, it is ids[places[i]] on the device (places[i] < 0:
        the host's list is complete); the repetition penalty then takes it from there."""
        dev = logits.device
        if all(is_plain_greedy(r.params) for r in rows):
            # the filters never remove the maximum, so greedy decoding is the argmax alone
            return self.k.argmax(logits), [r.rng_state for r in rows]
        ctx, offs, holes, sources = [], [0], [], []
        for i, r in enumerate(rows):
            c = r.context
            late = pending is not None and pending[1][i] >= 0
            if late:
                c = c + [0]                                  # the place of the token that is still on the device
            n = r.params.repeat_last_n
            if n and n < len(c):
                c = c[-n:]
            if abs(r.params.repetition_penalty - 1.0) < 1.2e-7:
                c = []
            ctx += c
            offs.append(len(ctx))
            if late and c:
                holes.append(len(ctx) - 1)
                sources.append(pending[1][i])
        R = len(rows)
        if not ctx:
            ctx = [0]
        # every row's settings, the context and the generator states go to the device in one copy from pinned
        # memory that does not wait for the steps in flight (a tensor made from a list on the device would):
        # int32 words [temperature R | top_k R | top_p R | min_p R | penalty R | offsets R + 1 | context | places of
        # the late tokens in the context and in `pending` | states 2 R]
        a_off, a_ctx = 5 * R, 6 * R + 1
        a_late = a_ctx + len(ctx)
        a_state = (a_late + 2 * len(holes) + 1) // 2 * 2          # 64-bit states on an 8-byte boundary
        n_words = a_state + 2 * R
        host = self._staging(n_words, dev)
        fl = host.view(torch.float32)
        fl[0:R] = torch.tensor([r.params.temperature for r in rows], dtype=torch.float32)
        host[R:2 * R] = torch.tensor([r.params.top_k for r in rows], dtype=torch.int32)
        fl[2 * R:3 * R] = torch.tensor([r.params.top_p for r in rows], dtype=torch.float32)
        fl[3 * R:4 * R] = torch.tensor([r.params.min_p for r in rows], dtype=torch.float32)
        fl[4 * R:5 * R] = torch.tensor([r.params.repetition_penalty for r in rows], dtype=torch.float32)
        host[a_off:a_ctx] = torch.tensor(offs, dtype=torch.int32)
        host[a_ctx:a_late] = torch.tensor(ctx, dtype=torch.int32)
        if holes:
            host[a_late:a_late + 2 * len(holes)] = torch.tensor(holes + sources, dtype=torch.int32)
        host[a_state:n_words].view(torch.int64)[:] = torch.tensor([_signed(r.rng_state & _MASK64) for r in rows], dtype=torch.int64)
        words = torch.empty(n_words, dtype=torch.int32, device=dev)
        words.copy_(host[:n_words], non_blocking=True)
        self._staged(dev)
        fd = words.view(torch.float32)
        context = words[a_ctx:a_late]
        if holes:
            late = words[a_late:a_late + 2 * len(holes)].long()
            context.index_copy_(0, late[:len(holes)], pending[0].index_select(0, late[len(holes):]).to(torch.int32))
        tokens = self.k.sample(
            logits, temperature=fd[0:R], top_k=words[R:2 * R], top_p=fd[2 * R:3 * R], min_p=fd[3 * R:4 * R],
            repetition_penalty=fd[4 * R:5 * R], context=context, context_offsets=words[a_off:a_ctx],
            rng_state=words[a_state:n_words].view(torch.int64))
        # the device advanced the states of the rows that drew; the host mirrors it
        states = [lcg_advance(r.rng_state) if r.params.temperature > 0 else r.rng_state for r in rows]
        return tokens, states
