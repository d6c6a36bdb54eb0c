"""How the parts of one layer are arranged.

`prenorm_residual` (crates/spite-models/src/llama/llama4.rs:126-127,202-211,272-274):
    h += mixer(norm_a(h));  h += feed_forward(norm_b(h))
The residual stream h stays float32; the sums are done by the epilogues of the
mixer's and the feed-forward's last products.
"""
from __future__ import annotations

import torch

from .base import Block, build_part, register_block


@register_block("prenorm_residual")
class PreNormResidual(Block):
    graph_safe = True
    def __init__(self, ctx, spec):
        super().__init__(ctx)
        self.mixer_norm = build_part("norm", spec.mixer_norm, ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ffn_norm = build_part("norm", spec.ffn_norm, ctx)
        self.ffn = build_part("feed_forward", spec.ffn, ctx)

    def children(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def forward(self, h, batch, cache):
        x = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        self.mixer_norm.forward(h, x)
        self.mixer.forward(x, h, batch, cache)
        self.ffn_norm.forward(h, x)
        self.ffn.forward(x, h, batch)
