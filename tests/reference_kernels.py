"""Plain torch restatement of every kernel's contract (`spite_b200.kernels.api`).

Two uses, both in tests only:
  * the reference each CUDA kernel is compared with, op by op;
  * a stand-in kernel set with which the engine's host logic (cache, batches,
    scheduler, trace replay) is exercised on a machine without a GPU.
It is slow on purpose: loops over tokens and heads, float32 arithmetic (float64
on request), no fusion.  It is not part of the package and nothing in the
package imports it.
"""
from __future__ import annotations

import math

import torch

from spite_b200.kernels.api import KernelSet, Routing


class TorchReferenceKernels(KernelSet):
    def __init__(self, dtype=torch.float32, device="cpu", acc=torch.float32):
        self.dtype = dtype
        self.device = torch.device(device)
        self.acc = acc

    # ---- elementwise
    def embed(self, table, token_ids, out_h, *, scale=1.0):
        out_h.copy_(table[token_ids.long()].float() * scale)

    def clear_pages(self, kv, page_ids):
        if page_ids:
            kv[:, :, torch.tensor(page_ids, dtype=torch.long)] = 0

    def transform_logits(self, logits, *, scale=1.0, softcap=None):
        logits.mul_(scale)
        if softcap:
            logits.copy_(softcap * torch.tanh(logits / softcap))

    def rms_norm(self, h, gain, eps, out, rows=None):
        x = h if rows is None else h[rows.long()]
        x = x.to(self.acc)
        y = x * (1.0 / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)) * gain.to(self.acc)
        out.copy_(y.to(out.dtype))

    # ---- matrix products
    def _mm(self, x, w):
        return x.to(self.acc) @ w.to(self.acc).T

    def linear(self, x, w, out, *, accumulate=False, row_scale=None):
        y = self._mm(x, w)
        if row_scale is not None:
            y = y * row_scale.to(self.acc)[:, None]
        if accumulate:
            out.add_(y.to(out.dtype))
        else:
            out.copy_(y.to(out.dtype))

    @staticmethod
    def _silu(g):
        return g / (1.0 + torch.exp(-g))

    def linear_swiglu(self, x, w_gate_up, out, *, row_scale=None):
        F = w_gate_up.shape[0] // 2
        y = self._mm(x, w_gate_up)
        if row_scale is not None:
            y = y * row_scale.to(self.acc)[:, None]
        out.copy_((self._silu(y[:, :F]) * y[:, F:]).to(out.dtype))

    def grouped_linear_swiglu(self, x, w_gate_up, sorted_rows, offsets, row_scale, out):
        E, F2, _ = w_gate_up.shape
        F = F2 // 2
        off = offsets.tolist()
        rows = sorted_rows.long()
        for e in range(E):
            lo, hi = off[e], off[e + 1]
            if hi == lo:
                continue
            tok = rows[lo:hi]
            y = self._mm(x[tok], w_gate_up[e])
            if row_scale is not None:
                y = y * row_scale[tok].to(self.acc)[:, None]
            out[lo:hi] = (self._silu(y[:, :F]) * y[:, F:]).to(out.dtype)

    def grouped_linear_accumulate(self, a, w_down, sorted_rows, offsets, h):
        E = w_down.shape[0]
        off = offsets.tolist()
        rows = sorted_rows.long()
        for e in range(E):
            lo, hi = off[e], off[e + 1]
            if hi == lo:
                continue
            h[rows[lo:hi]] += self._mm(a[lo:hi], w_down[e]).to(h.dtype)

    # ---- attention
    def qk_prepare(self, qkv, q_out, batch, cache, *, num_heads, rotation, qk_norm, temperature):
        kv = cache.kv
        nkv, P, hd = kv.shape[2], kv.shape[3], kv.shape[4]
        nq = num_heads
        M = qkv.shape[0]
        x = qkv.to(self.acc).view(M, nq + 2 * nkv, hd)
        q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]
        pos = batch.positions.long()

        def norm(t, gain):
            t = t * (1.0 / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + qk_norm.eps))
            return t if gain is None else t * gain.to(t.device, self.acc)

        if qk_norm is not None and qk_norm.before_rotation:
            q, k = norm(q, qk_norm.q_gain), norm(k, qk_norm.k_gain)
        if rotation is not None:
            inv_freq = rotation.inv_freq.to(q.device)
            rd = rotation.rotary_dim or hd
            ang = (pos.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)).to(self.acc)
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

            def rot(t):
                o = t.clone()
                if rotation.pairing == "neighbours":
                    a, b = t[..., 0:rd:2], t[..., 1:rd:2]
                    o[..., 0:rd:2] = a * cos - b * sin
                    o[..., 1:rd:2] = a * sin + b * cos
                else:
                    a, b = t[..., :rd // 2], t[..., rd // 2:rd]
                    o[..., :rd // 2] = a * cos - b * sin
                    o[..., rd // 2:rd] = a * sin + b * cos
                return o
            q, k = rot(q), rot(k)
        if qk_norm is not None and not qk_norm.before_rotation:
            q, k = norm(q, qk_norm.q_gain), norm(k, qk_norm.k_gain)
        if temperature:
            floor, scale = temperature
            fl = torch.div(pos + 1, int(floor), rounding_mode="floor").to(self.acc)
            q = q * (torch.log(fl + 1.0) * scale + 1.0)[:, None, None]
        q_out.copy_(q.reshape(M, nq * hd).to(q_out.dtype))
        if cache.write:
            bt = batch.block_tables[cache.group]
            seg = batch.seg_of_token.long()
            for t in range(M):
                p = int(pos[t])
                page = int(bt[seg[t], p // P])
                assert page >= 0, "write into a page that is not held"
                kv[0, page, :, p % P, :] = k[t].to(kv.dtype)
                kv[1, page, :, p % P, :] = v[t].to(kv.dtype)

    def paged_attention(self, q, out, batch, cache, *, num_heads, window, softmax_scale, cache_settled=False):
        kv = cache.kv
        nkv, P, hd = kv.shape[2], kv.shape[3], kv.shape[4]
        nq = num_heads
        group = nq // nkv
        M = q.shape[0]
        bt = batch.block_tables[cache.group]
        pos = batch.positions.tolist()
        seg = batch.seg_of_token.tolist()
        qf = q.to(self.acc).view(M, nq, hd)
        for t in range(M):
            p = pos[t]
            lo = window.lowest_visible(p)
            js = torch.arange(lo, p + 1)
            pages = bt[seg[t]].long()[torch.div(js, P, rounding_mode="floor")]
            assert bool((pages >= 0).all()), "read from a page that was given back"
            K = kv[0, pages, :, js % P, :].to(self.acc)          # [n, nkv, hd]
            V = kv[1, pages, :, js % P, :].to(self.acc)
            for h in range(nq):
                s = (K[:, h // group, :] @ qf[t, h]) * softmax_scale
                w = torch.softmax(s, dim=0)
                out[t, h * hd:(h + 1) * hd] = (w @ V[:, h // group, :]).to(out.dtype)

    # ---- mixture of experts
    def moe_route(self, x, w_router, top_k, want_logits=False) -> Routing:
        logits = (x.to(torch.float32) @ w_router.to(torch.float32).T)
        order = torch.sort(logits, dim=-1, descending=True, stable=True)
        ids = order.indices[:, :top_k].T.contiguous().to(torch.int32)        # [k, M]
        w = (1.0 / (1.0 + torch.exp(-order.values[:, :top_k]))).T.contiguous()
        M, E = logits.shape
        offsets = torch.zeros((top_k, E + 1), dtype=torch.int32, device=x.device)
        rows = torch.zeros((top_k, M), dtype=torch.int32, device=x.device)
        for s in range(top_k):
            srt = torch.sort(ids[s].long(), stable=True)
            rows[s] = srt.indices.to(torch.int32)
            counts = torch.bincount(ids[s].long(), minlength=E)
            offsets[s, 1:] = torch.cumsum(counts, 0).to(torch.int32)
        return Routing(ids, w, offsets, rows, logits if want_logits else None)

    # ---- sampling
    def argmax(self, logits):
        V = logits.shape[1]
        flipped = torch.flip(logits, dims=[1])
        return (V - 1 - torch.argmax(flipped, dim=1)).to(torch.int32)

    def sample(self, logits, *, temperature, top_k=None, top_p=None, min_p=None, repetition_penalty=None,
               context=None, context_offsets=None, rng_state):
        from plain_llama4 import sample_plain
        out = torch.zeros(logits.shape[0], dtype=torch.int32)
        for r in range(logits.shape[0]):
            ctx = []
            if context is not None:
                ctx = context[int(context_offsets[r]):int(context_offsets[r + 1])].tolist()
            tok, st = sample_plain(
                logits[r].cpu(), ctx, temperature=float(temperature[r]),
                top_k=int(top_k[r]) if top_k is not None else 0,
                top_p=float(top_p[r]) if top_p is not None else 1.0,
                min_p=float(min_p[r]) if min_p is not None else 0.0,
                repetition_penalty=float(repetition_penalty[r]) if repetition_penalty is not None else 1.0,
                repeat_last_n=0, state=int(rng_state[r]) & ((1 << 64) - 1))
            out[r] = tok
            rng_state[r] = st - (1 << 64) if st >= (1 << 63) else st
        return out.to(logits.device)
