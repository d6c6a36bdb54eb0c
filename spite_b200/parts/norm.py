"""RMS norm with a gain vector (crates/spite-models/src/dense.rs:175-181)."""
from __future__ import annotations

import torch

from .base import Norm, ParamSpec, register_norm


@register_norm("rms_norm")
class RmsNorm(Norm):
    graph_safe = True
    kernel_libraries = ("elementwise",)

    def __init__(self, ctx, size: int, eps: float):
        super().__init__(ctx)
        self.size, self.eps = int(size), float(eps)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), "ones")}

    def bind(self, params):
        # the gain is applied in float32; a bfloat16 gain converts exactly
        self.weight = params["weight"].to(torch.float32).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def forward(self, h, out, rows=None):
        self.k.rms_norm(h, self.weight, self.eps, out, rows)
        return out
