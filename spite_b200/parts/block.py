"""How the parts of one layer are arranged.

`prenorm_residual` (crates/spite-models/src/llama/llama4.rs:126-127,202-211,272-274):
    h += mixer(norm_a(h));  h += feed_forward(norm_b(h))
The residual stream h stays float32; the sums are done by the epilogues of the
mixer's and the feed-forward's last products.
"""
from __future__ import annotations

import torch

from .base import Block, register_block


@register_block("prenorm_residual")
class PreNormResidual(Block):
    graph_safe = True
    places = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def forward(self, h, batch, cache):
        x = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        self.mixer_norm.forward(h, x)
        self.mixer.forward(x, h, batch, cache)
        self.ffn_norm.forward(h, x)
        self.ffn.forward(x, h, batch)
