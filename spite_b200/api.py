"""The Python entry point: `LLM` and `generate`.

    from spite_b200 import generate
    tokens = generate("path/to/model", [[1, 2, 3]], max_tokens=16, temperature=0.0)

Prompts and results are token ids (no tokenizer is part of this engine).  The
options carry giveen/spite's names and meanings: `max_tokens` (512),
`temperature` (1.0; 0 is greedy), `ctx` (context window, default the model's
maximum) as in `spite run` (crates/spite-cli/src/main.rs:282-306), the sampler
settings of `default_sampler_config` (crates/spite-executor/src/lib.rs:144-151)
and the seed constant of crates/spite-cli/src/main.rs:606.
"""
from __future__ import annotations

from pathlib import Path

from .engine.executor import Engine
from .engine.model import Model
from .engine.scheduler import Request, Scheduler
from .sampling.sampler import DEFAULT_SEED, Sampler, SamplingParams, run_sampling_params


class LLM:
    """A loaded model with its cache, step function, scheduler and sampler."""

    def __init__(self, model, *, dtype="bfloat16", device="cuda:0", ctx: int | None = None,
                 cache_tokens: int | None = None, page_size: int = 64, max_requests: int = 64,
                 max_batch_tokens: int = 2048, kernels=None, decode_ahead: bool | None = None):
        if not isinstance(model, Model):
            model = Model.from_folder(Path(model), dtype=dtype, device=device, kernels=kernels)
        self.model = model
        self.ctx = int(ctx or model.plan.max_positions)
        if cache_tokens is None:
            cache_tokens = min(self.ctx, 8192) * min(max_requests, 8)
        self.engine = Engine(model, cache_tokens=cache_tokens, page_size=page_size,
                             max_requests=max_requests, max_positions=self.ctx)
        self.sampler = Sampler(model.kernels)
        self.max_batch_tokens = max_batch_tokens
        self.decode_ahead = decode_ahead     # None: on where decode steps run from CUDA graphs
        eos = getattr(model.config, "eos_token_id", None) or ()
        self.eos_token_ids = tuple(eos)

    def scheduler(self, **kw) -> Scheduler:
        kw.setdefault("max_batch_tokens", self.max_batch_tokens)
        kw.setdefault("ctx", self.ctx)
        kw.setdefault("eos_token_ids", self.eos_token_ids)
        kw.setdefault("decode_ahead", self.decode_ahead)
        return Scheduler(self.engine, self.sampler, **kw)

    def generate(self, prompts, *, max_tokens: int = 512, temperature: float = 1.0, seed: int = DEFAULT_SEED,
                 stop_token_ids=(), sampling: SamplingParams | None = None, return_requests: bool = False):
        """Generate for every prompt (a list of token ids); returns the new tokens of
        each, in the order of `prompts`.  `sampling` overrides the `run` defaults."""
        sched = self.scheduler()
        for i, p in enumerate(prompts):
            params = sampling or run_sampling_params(temperature, seed=seed, max_tokens=max_tokens,
                                                     stop_token_ids=stop_token_ids)
            params = SamplingParams(**{**params.__dict__})
            sched.submit(Request(id=i, prompt=[int(t) for t in p], params=params))
        done = sched.run_until_done()
        self.last_counters = dict(sched.counters)
        if return_requests:
            return [done[i] for i in range(len(prompts))]
        return [list(done[i].output) for i in range(len(prompts))]


def generate(model, prompts, *, max_tokens: int = 512, temperature: float = 1.0, seed: int = DEFAULT_SEED,
             ctx: int | None = None, dtype="bfloat16", device="cuda:0", stop_token_ids=(), **engine_options):
    """Load `model` (a folder with config.json and model.safetensors, or a `Model`) and
    generate `max_tokens` new tokens for every prompt."""
    llm = LLM(model, dtype=dtype, device=device, ctx=ctx, **engine_options)
    return llm.generate(prompts, max_tokens=max_tokens, temperature=temperature, seed=seed,
                        stop_token_ids=stop_token_ids)
