"""The contract between the layer parts and the kernels.

A `KernelSet` is bound to one activation type (bfloat16 or float32).  The
residual stream, norm gains, router weights, softmax statistics and logits are
float32 in both sets.  Parts call these methods and nothing else to touch the
device; a kernel set never learns which model or layer it serves.

Shapes use M for the tokens of the step, d for the model width, T for the
activation type.  All tensors are contiguous and live on the set's device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class KernelError(RuntimeError):
    """A kernel refused its arguments or could not be launched."""


class KernelTimeout(KernelError):
    """A kernel gave up a bounded wait and left its output incomplete: the results of the steps
    since the last check cannot be trusted (ExecutorError in crates/spite-executor/src/lib.rs:88-100
    is the counterpart: a typed error instead of wrong logits)."""


@dataclass
class Routing:
    """Result of `moe_route` for M tokens, E experts and k choices per token."""
    expert_ids: torch.Tensor     # [k, M] int32
    weights: torch.Tensor        # [k, M] float32, sigmoid of the chosen logits
    offsets: torch.Tensor        # [k, E + 1] int32: places of each expert's tokens in sorted_rows
    sorted_rows: torch.Tensor    # [k, M] int32: token indices ordered by expert, ascending within one
    logits: Optional[torch.Tensor] = None   # [M, E] float32 if asked for


class KernelSet:
    """Interface; see `CudaKernels` for the product implementation."""

    dtype: torch.dtype
    device: torch.device

    def errors(self) -> dict:
        """{kernel library: code} for every library one of whose kernels gave up a bounded wait since
        the last call; reading clears.  Does not wait for the device: call it after a point at
        which the host has waited for the step's results."""
        return {}

    # ---- elementwise
    def embed(self, table, token_ids, out_h, *, scale=1.0):
        """out_h[m, :] (float32) = table[token_ids[m], :] (T) * scale."""
        raise NotImplementedError

    def transform_logits(self, logits, *, scale=1.0, softcap=None):
        """In place: logits *= scale; then, with a cap, logits = cap * tanh(logits / cap)."""
        raise NotImplementedError

    def rms_norm(self, h, gain, eps, out, rows=None):
        """out[i, :] (T or float32) = h[r] * rsqrt(mean(h[r]^2) + eps) * gain, r = rows[i] if rows else i.
        h float32 [*, d], gain float32 [d]."""
        raise NotImplementedError

    # ---- matrix products: y = x W^T with W [out, in]
    def linear(self, x, w, out, *, accumulate=False, row_scale=None):
        """out[M, N] = x[M, K] @ w[N, K]^T.  `out` is T, or float32 (logits); with
        `accumulate` it is float32 and the product is added to it (residual stream).
        `row_scale` [M] float32 multiplies the product's rows."""
        raise NotImplementedError

    def linear_swiglu(self, x, w_gate_up, out, *, row_scale=None):
        """out[M, F] (T) = silu(s g) * (s u) with g = x @ w[:F]^T, u = x @ w[F:]^T, s = row_scale or 1."""
        raise NotImplementedError

    def grouped_linear_swiglu(self, x, w_gate_up, sorted_rows, offsets, row_scale, out):
        """Row i of `out` [M, F] (sorted order) is the SwiGLU of token sorted_rows[i] through the
        expert whose range of `offsets` holds i; w_gate_up [E, 2F, K]; row_scale [M] by token."""
        raise NotImplementedError

    def grouped_linear_accumulate(self, a, w_down, sorted_rows, offsets, h):
        """h[sorted_rows[i], :] (float32) += a[i, :] @ w_down[expert of i]^T; w_down [E, d, F]."""
        raise NotImplementedError

    # ---- cache
    def clear_pages(self, kv, page_ids):
        """Zero the pages `page_ids` (a list of ints) of every cache of a group; `kv` is the group's tensor
        [caches, 2, pages, kv heads, page_size, head_dim].  The engine does this when it hands a page out,
        so that a request never multiplies a masked key's zero weight with what another request left there."""
        raise NotImplementedError

    # ---- attention
    def qk_prepare(self, qkv, q_out, batch, cache, *, num_heads, rotation, qk_norm, temperature):
        """Encode positions of q and k, normalise, scale q, append k and v to the cache.
        qkv [M, (nq + 2 nkv) hd] T -> q_out [M, nq hd] T; `cache` is a `LayerCache`.
        `rotation`: a `parts.Rotation` or None; `qk_norm`: a `parts.QkNorm` or None (RMS norm of
        every q and k head, after the rotation unless it says before); `temperature`:
        (floor, scale) or None: q *= ln(floor((pos + 1) / floor) + 1) * scale + 1."""
        raise NotImplementedError

    def paged_attention(self, q, out, batch, cache, *, num_heads, window, softmax_scale, cache_settled=False):
        """out[M, nq hd] = softmax(q K^T * scale over the visible cached keys) V.
        `cache_settled`: the caller promises that the cache rows of positions before each request's first
        token of this step were written by earlier steps (not by the one or two kernels launched just
        before this call), so a kernel may fetch them while the kernel before still runs."""
        raise NotImplementedError

    # ---- mixture of experts
    def moe_route(self, x, w_router, top_k, want_logits=False) -> Routing:
        raise NotImplementedError

    # ---- sampling
    def argmax(self, logits):
        """[R] int32: index of the maximum of each row, the highest index among equals."""
        raise NotImplementedError

    def sample(self, logits, *, temperature, top_k, top_p, min_p, repetition_penalty,
               context, context_offsets, rng_state):
        """[R] int32 tokens; `rng_state` [R] int64 is advanced in place for rows that draw."""
        raise NotImplementedError
