"""A model built from a `ModelPlan`: embedding, the layers in their run order,
final norm and output head.  It knows parts and a plan, not architectures.

Counterpart in giveen/spite: the `ModelArch` trait with `load_weights`,
`reset_cache` and `forward(tokens, logits_out, ctx)` for one sequence
(crates/spite-models/src/lib.rs:301-335); here `forward` takes a batch of
segments of several requests and returns logits only where they are asked for.
"""
from __future__ import annotations

import torch

from ..cache import FixedState, PagedKV
from ..config import ConfigError, ModelPlan, load_config
from ..kernels import build as kernel_build
from ..parts import BuildContext, ParamSpec, build_part
from ..parts.base import _REGISTRIES
from ..weights import bind_tensors, load_bound_tensors
from ..weights.random_init import tensor_seed

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ConfigError(f"dtype {dtype!r} is not supported; use 'bfloat16' or 'float32'") from None


class Model:
    def __init__(self, plan: ModelPlan, *, dtype="bfloat16", device="cuda:0", kernels=None, config=None):
        self.plan = plan.validate()
        self.config = config
        self.dtype = resolve_dtype(dtype)
        self.device = torch.device(device)
        if kernels is None:
            from ..kernels.cuda import CudaKernels
            kernels = CudaKernels(self.dtype, self.device)
        self.kernels = kernels
        self.ctx = BuildContext(kernels=kernels, dtype=self.dtype, device=self.device)
        blocks = _REGISTRIES["block"]
        self.blocks = []
        for spec in plan.blocks:
            if spec.arrangement not in blocks:
                raise ConfigError(f"no block arrangement {spec.arrangement!r}; known: {', '.join(sorted(blocks))}")
            self.blocks.append(blocks[spec.arrangement](self.ctx, spec))
        self.final_norm = build_part("norm", plan.final_norm, self.ctx)
        self.embed_table = None
        self.head_weight = None
        self._check_caches()

    # ------------------------------------------------------------------ structure
    def parts(self):
        """(full name, part) of every part that owns parameters."""
        for i, b in enumerate(self.blocks):
            for cname, child in b.children().items():
                yield f"layers.{i}.{cname}", child
        yield "final_norm", self.final_norm

    def param_specs(self) -> dict[str, ParamSpec]:
        p = self.plan
        out = {"embed.weight": ParamSpec((p.vocab_size, p.hidden_size))}
        for name, part in self.parts():
            for pname, spec in part.param_specs().items():
                out[f"{name}.{pname}"] = spec
        if not p.tie_word_embeddings:
            out["head.weight"] = ParamSpec((p.vocab_size, p.hidden_size))
        return out

    def kernel_libraries(self) -> list[str]:
        libs = {"elementwise", "gemm_simt"}
        if self.dtype == torch.bfloat16:
            libs |= {"gemm_skinny", "gemm_stream", "gemm_tc", "gemm_tc_pair", "gemm_tc_experts"}
        for _, part in self.parts():
            libs.update(part.kernel_libraries)
        return sorted(libs)

    def graph_safe(self) -> bool:
        """True if a step's kernels can be captured in a CUDA graph: the product kernel set
        and parts that launch nothing but its kernels and never read device data on the host."""
        from ..kernels.cuda import CudaKernels
        return isinstance(self.kernels, CudaKernels) and all(part.graph_safe for _, part in self.parts()) \
            and all(getattr(b, "graph_safe", False) for b in self.blocks)

    def _check_caches(self):
        self._cache_specs = {}
        for call in self.plan.order:
            req = self.blocks[call.layer].cache_request()
            have = self._cache_specs.get(call.cache)
            if have is None:
                self._cache_specs[call.cache] = req
            elif have != req:
                raise ConfigError(
                    f"cache {call.cache} is shared by layers whose mixers need different caches: {have} vs {req}")

    def cache_specs(self) -> dict:
        """{cache id: (PagedKV | None, FixedState | None)} for `CacheStorage`."""
        return dict(self._cache_specs)

    # ------------------------------------------------------------------ weights
    def load_params(self, tensors: dict[str, torch.Tensor]):
        specs = self.param_specs()
        missing = [n for n in specs if n not in tensors]
        extra = [n for n in tensors if n not in specs]
        wrong = [(n, tuple(tensors[n].shape), specs[n].shape) for n in specs
                 if n in tensors and tuple(tensors[n].shape) != tuple(specs[n].shape)]
        if missing or extra or wrong:
            raise ConfigError(f"parameters do not fit the plan: missing {missing}, unknown {extra}, "
                              f"wrong shape {wrong}")
        self.embed_table = tensors["embed.weight"].to(self.device, self.dtype).contiguous()
        self.head_weight = self.embed_table if self.plan.tie_word_embeddings else \
            tensors["head.weight"].to(self.device, self.dtype).contiguous()
        for name, part in self.parts():
            own = {p: tensors[f"{name}.{p}"].to(self.device) for p in part.param_specs()}
            part.bind(own)
        return self

    def init_random(self, seed: int = 0, std: float = 0.02):
        """Fill every parameter on the device: N(0, std) from a generator seeded by
        (seed, parameter name); norm gains one.  For models too large to write to disk."""
        def make(name, spec):
            if spec.init == "ones":
                return torch.ones(spec.shape, dtype=self.dtype, device=self.device)
            g = torch.Generator(device=self.device)
            g.manual_seed(tensor_seed(seed, name))
            t = torch.empty(spec.shape, dtype=self.dtype, device=self.device)
            t.normal_(0.0, std, generator=g)
            return t
        p = self.plan
        self.embed_table = make("embed.weight", ParamSpec((p.vocab_size, p.hidden_size)))
        self.head_weight = self.embed_table if p.tie_word_embeddings else \
            make("head.weight", ParamSpec((p.vocab_size, p.hidden_size)))
        for name, part in self.parts():
            part.bind({pn: make(f"{name}.{pn}", ps) for pn, ps in part.param_specs().items()})
        return self

    def weight_bytes(self) -> int:
        n = self.embed_table.numel() * self.embed_table.element_size()
        if self.head_weight is not self.embed_table:
            n += self.head_weight.numel() * self.head_weight.element_size()
        return n + sum(part.weight_bytes() for _, part in self.parts())

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_config(cls, config, **kw) -> "Model":
        return cls(config.plan(), config=config, **kw)

    @classmethod
    def from_folder(cls, folder, *, dtype="bfloat16", device="cuda:0", kernels=None, build=True) -> "Model":
        """Read config.json, choose the model by its `architectures` entry, compile what
        the model's parts need, and bind model.safetensors by tensor name."""
        config = load_config(folder)
        model = cls.from_config(config, dtype=dtype, device=device, kernels=kernels)
        if build and kernels is None:
            kernel_build.ensure_built(model.kernel_libraries())
        tensors = load_bound_tensors(folder, config, device=model.device)
        return model.load_params(tensors)

    @classmethod
    def from_tensors(cls, config, checkpoint_tensors: dict, *, dtype="bfloat16", device="cuda:0", kernels=None,
                     build=True) -> "Model":
        """The same from checkpoint tensors in memory ({checkpoint tensor name: tensor}, the names and
        layouts a model.safetensors of this architecture would have)."""
        model = cls.from_config(config, dtype=dtype, device=device, kernels=kernels)
        if build and kernels is None:
            kernel_build.ensure_built(model.kernel_libraries())
        return model.load_params(bind_tensors(config, checkpoint_tensors, device=model.device))

    # ------------------------------------------------------------------ running
    def forward(self, batch, storage) -> torch.Tensor:
        """Run the step's tokens through every layer of the run order; returns the
        float32 logits [wanted rows, vocab]."""
        k = self.kernels
        p = self.plan
        h = torch.empty((batch.n_tokens, p.hidden_size), dtype=torch.float32, device=self.device)
        k.embed(self.embed_table, batch.token_ids, h, scale=p.embedding_scale)
        for call in p.order:
            self.blocks[call.layer].forward(h, batch, storage.layer_cache(call.cache, call.write_cache))
        R = batch.logit_rows.numel()
        logits = torch.empty((R, p.vocab_size), dtype=torch.float32, device=self.device)
        if R:
            x = torch.empty((R, p.hidden_size), dtype=self.dtype, device=self.device)
            self.final_norm.forward(h, x, rows=batch.logit_rows)
            k.linear(x, self.head_weight, logits)
            if p.logit_scale != 1.0 or p.logit_softcap is not None:
                k.transform_logits(logits, scale=p.logit_scale, softcap=p.logit_softcap)
        return logits
