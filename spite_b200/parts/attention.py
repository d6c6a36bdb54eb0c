"""Grouped-query attention over the paged cache.

One part serves every attention layer: the window rule (all keys, the keys of
the query's chunk, the last W keys), the position encoding, the per-head norm of
q and k (after or before the rotation, with gains or without) and the
temperature factor are constructor parameters.

Formulas: crates/spite-models/src/llama/llama4.rs:126-207 (projections, rotation
then norm, temperature factor on layers without rotation, append to the cache,
attention, output projection added to the residual stream) and
crates/spite-compute/src/flash_attn.rs:111-156 (scores, mask, softmax, values).
"""
from __future__ import annotations

import math

import torch

from ..cache import PagedKV, Window
from ..config.specs import ConfigError, PartSpec
from .base import Mixer, ParamSpec, QkNorm, build_part, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    graph_safe = True
    kernel_libraries = ("gemm_simt", "attention", "attention_mma", "attention_rows", "attention_tc", "attention_decode")

    def __init__(self, ctx, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window=("full", 0), qk_norm_eps=None, qk_norm_gain=False,
                 qk_norm_before_rotation=False, temperature_tuning=None, softmax_scale=None):
        super().__init__(ctx)
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads evenly")
        if head_dim % 2 or head_dim > 256:
            raise ConfigError(f"head_dim {head_dim} must be even and at most 256")
        self.d, self.nq, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        # only the attention kernels that these sizes can reach are compiled for the model
        libs = ["gemm_simt", "attention"]
        if ctx.dtype == torch.bfloat16 and self.hd % 16 == 0 and self.hd <= 128 and self.nq // self.nkv <= 16:
            libs += ["attention_mma", "attention_rows"]
            if self.hd in (64, 128):
                libs += ["attention_tc", "attention_decode"]
        self.kernel_libraries = tuple(libs)
        self.window = window if isinstance(window, Window) else Window(window[0], int(window[1]))
        self.position = build_part("position", position, ctx)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.qk_norm_gain = bool(qk_norm_gain) and self.qk_norm_eps is not None
        self.qk_norm_before_rotation = bool(qk_norm_before_rotation)
        self.qk_norm = None if self.qk_norm_eps is None else QkNorm(self.qk_norm_eps, self.qk_norm_before_rotation)
        if temperature_tuning is not None:
            floor, scale = temperature_tuning
            if float(floor) != int(floor) or int(floor) < 1:
                raise ConfigError(f"temperature floor_scale {floor} must be a positive integer")
            temperature_tuning = (int(floor), float(scale))
        self.temperature = temperature_tuning
        self.softmax_scale = float(softmax_scale) if softmax_scale else 1.0 / math.sqrt(self.hd)
        self.wqkv = self.wo = None

    def param_specs(self):
        d, nq, nkv, hd = self.d, self.nq, self.nkv, self.hd
        specs = {"q_proj": ParamSpec((nq * hd, d)), "k_proj": ParamSpec((nkv * hd, d)),
                 "v_proj": ParamSpec((nkv * hd, d)), "o_proj": ParamSpec((d, nq * hd))}
        if self.qk_norm_gain:
            specs.update({"q_norm": ParamSpec((hd,), "ones"), "k_norm": ParamSpec((hd,), "ones")})
        return specs

    def bind(self, params):
        dt = self.ctx.dtype
        # q, k and v rows in one matrix: one product per layer instead of three
        self.wqkv = torch.cat([params["q_proj"].to(dt), params["k_proj"].to(dt), params["v_proj"].to(dt)], 0).contiguous()
        self.wo = params["o_proj"].to(dt).contiguous()
        if self.qk_norm_gain:
            self.qk_norm = QkNorm(self.qk_norm_eps, self.qk_norm_before_rotation,
                                  params["q_norm"].to(torch.float32).contiguous(),
                                  params["k_norm"].to(torch.float32).contiguous())

    def weight_bytes(self):
        return (self.wqkv.numel() + self.wo.numel()) * self.wqkv.element_size()

    def cache_request(self):
        return PagedKV(self.window, self.nkv, self.hd), None

    def forward(self, x, h, batch, cache):
        M = x.shape[0]
        k = self.k
        qkv = torch.empty((M, (self.nq + 2 * self.nkv) * self.hd), dtype=x.dtype, device=x.device)
        k.linear(x, self.wqkv, qkv)
        q = torch.empty((M, self.nq * self.hd), dtype=x.dtype, device=x.device)
        k.qk_prepare(qkv, q, batch, cache, num_heads=self.nq, rotation=self.position.rotation(),
                     qk_norm=self.qk_norm, temperature=self.temperature)
        o = torch.empty_like(q)
        # keys and values of earlier positions were cached by earlier steps; this step's own were written by
        # the prepare kernel just before, which is what the attention kernel waits for
        k.paged_attention(q, o, batch, cache, num_heads=self.nq, window=self.window,
                          softmax_scale=self.softmax_scale, cache_settled=True)
        k.linear(o, self.wo, h, accumulate=True)
