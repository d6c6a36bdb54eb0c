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

    def greedy_on_device(self, logits: torch.Tensor) -> torch.Tensor:
        """The argmax of every row as int32 on the device; nothing is read back."""
        return self.k.argmax(logits)

    def sample(self, logits: torch.Tensor, rows: list) -> tuple[list, list]:
        """`logits` [R, vocab] float32 on the device, `rows` R `SampleRow`s.
        Returns (tokens, new generator states)."""
        R = len(rows)
        if R == 0:
            return [], []
        dev = logits.device
        if all(is_plain_greedy(r.params) for r in rows):
            # the filters never remove the maximum, so greedy decoding is the argmax alone
            return self.k.argmax(logits).tolist(), [r.rng_state for r in rows]
        ctx, offs = [], [0]
        for r in rows:
            c = r.context
            n = r.params.repeat_last_n
            if n and n < len(c):
                c = c[-n:]
            if abs(r.params.repetition_penalty - 1.0) < 1.2e-7:
                c = []
            ctx += c
            offs.append(len(ctx))
        f32 = lambda vals: torch.tensor(vals, dtype=torch.float32, device=dev)
        i32 = lambda vals: torch.tensor(vals, dtype=torch.int32, device=dev)
        state = torch.tensor([_signed(r.rng_state & _MASK64) for r in rows], dtype=torch.int64, device=dev)
        tokens = self.k.sample(
            logits, temperature=f32([r.params.temperature for r in rows]),
            top_k=i32([r.params.top_k for r in rows]), top_p=f32([r.params.top_p for r in rows]),
            min_p=f32([r.params.min_p for r in rows]),
            repetition_penalty=f32([r.params.repetition_penalty for r in rows]),
            context=i32(ctx if ctx else [0]), context_offsets=i32(offs), rng_state=state).tolist()
        # the device advanced the states of the rows that drew; the host mirrors it
        states = [lcg_advance(r.rng_state) if r.params.temperature > 0 else r.rng_state for r in rows]
        return tokens, states
