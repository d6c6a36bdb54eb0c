"""The tokens of one step, flattened for the device.

A step runs M tokens that belong to S segments, one segment per request in the
step: a portion of a prompt (two tokens or more) or a single decoded token.  All
integer inputs of the step are packed into one host buffer and copied to the
device in one transfer; the fields below are views into that copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class Segment:
    req_id: object
    slot: int          # the request's state slot
    start_pos: int     # absolute position of the segment's first token
    n_tokens: int
    offset: int        # row of its first token in the step's flattened arrays
    fresh: bool        # the request's first step: fixed-size state starts at zero


@dataclass
class StepBatch:
    n_tokens: int
    segments: list
    token_ids: torch.Tensor        # [M] int32
    positions: torch.Tensor        # [M] int32
    seg_of_token: torch.Tensor     # [M] int32
    cu_seqlens: torch.Tensor       # [S + 1] int32
    slots: torch.Tensor            # [S] int32
    logit_rows: torch.Tensor       # [R] int32 rows whose logits are wanted
    block_tables: list = field(default_factory=list)   # per group: [S, W] int32
    max_seg_len: int = 0
    context_bucket: int | None = None   # steps replayed from a CUDA graph: launch shapes are chosen for
                                        # this context length instead of the step's own


def build_step_batch(segments, tokens_per_segment, wants, tables_per_group, device, pin=True) -> StepBatch:
    """`tables_per_group[g][s]` is the block table (list of page ids, -1 for freed)
    of segment s in group g; `wants[s]` the indices within segment s whose logits are asked."""
    S = len(segments)
    M = sum(len(t) for t in tokens_per_segment)
    widths = [max(1, max((len(t) for t in tabs), default=1)) for tabs in tables_per_group]
    R = sum(len(w) for w in wants)
    total = 3 * M + (S + 1) + S + R + sum(S * w for w in widths)
    host = torch.empty(max(total, 1), dtype=torch.int32)
    if pin and torch.device(device).type == "cuda":
        host = host.pin_memory()
    buf = host.numpy()
    o = 0
    views = {}

    def take(name, n):
        nonlocal o
        views[name] = (o, n)
        o += n
        return buf[o - n:o]
    tok, pos, sot = take("tok", M), take("pos", M), take("sot", M)
    cu, sl, lr = take("cu", S + 1), take("slots", S), take("rows", R)
    cu[0] = 0
    r = 0
    for s, (seg, toks, want) in enumerate(zip(segments, tokens_per_segment, wants)):
        n = len(toks)
        a = seg.offset
        tok[a:a + n] = toks
        pos[a:a + n] = range(seg.start_pos, seg.start_pos + n)
        sot[a:a + n] = s
        cu[s + 1] = a + n
        sl[s] = seg.slot
        for w in want:
            lr[r] = a + w
            r += 1
    for g, tabs in enumerate(tables_per_group):
        w = widths[g]
        bt = take(f"bt{g}", S * w).reshape(S, w)
        bt[:] = -1
        for s, t in enumerate(tabs):
            bt[s, :len(t)] = t
    dev = host.to(device, non_blocking=True)

    def view(name):
        a, n = views[name]
        return dev[a:a + n]
    return StepBatch(
        n_tokens=M, segments=list(segments), token_ids=view("tok"), positions=view("pos"),
        seg_of_token=view("sot"), cu_seqlens=view("cu"), slots=view("slots"), logit_rows=view("rows"),
        block_tables=[view(f"bt{g}").view(S, widths[g]) for g in range(len(tables_per_group))],
        max_seg_len=max((len(t) for t in tokens_per_segment), default=0))


class StaticDecodeBatch:
    """The inputs of a decode step (one token per request) at fixed device addresses,
    so that the step's kernels can be captured once in a CUDA graph and replayed:
    only the contents of these buffers change from step to step.

    The batch has room for `n_requests` rows; a step of fewer requests fills the
    rest with copies of its first row.  A copy computes what the first row
    computes and writes the same keys and values to the same place, so it changes
    nothing and reads no weight or page that the step would not read anyway."""

    def __init__(self, n_requests: int, table_widths: list, device, context_bucket: int):
        S = self.S = n_requests
        self.widths = list(table_widths)
        total = 3 * S + (S + 1) + S + S + sum(S * w for w in self.widths)
        self.host = torch.empty(total, dtype=torch.int32)
        if torch.device(device).type == "cuda":
            self.host = self.host.pin_memory()
        self.dev = torch.empty(total, dtype=torch.int32, device=device)
        buf = self.host.numpy()
        o = 0

        def take(n):
            nonlocal o
            o += n
            return slice(o - n, o)
        self._tok, self._pos, sot = take(S), take(S), take(S)
        cu, self._slots, rows = take(S + 1), take(S), take(S)
        self._bt = [take(S * w) for w in self.widths]
        buf[sot] = range(S)
        buf[cu] = range(S + 1)
        buf[rows] = range(S)
        self.batch = StepBatch(
            n_tokens=S, segments=[], token_ids=self.dev[self._tok], positions=self.dev[self._pos],
            seg_of_token=self.dev[sot], cu_seqlens=self.dev[cu], slots=self.dev[self._slots],
            logit_rows=self.dev[rows],
            block_tables=[self.dev[sl].view(S, w) for sl, w in zip(self._bt, self.widths)],
            max_seg_len=1, context_bucket=context_bucket)
        self._copied = None

    def fill(self, segments, tokens, tables_per_group):
        """Write this step's tokens, positions, slots and block tables and start the copy."""
        if self._copied is not None:
            self._copied.synchronize()          # the last step's copy has read the host buffer
        n = len(segments)
        if not 1 <= n <= self.S:
            raise ValueError(f"a static batch of {self.S} rows cannot hold {n} requests")
        pad = self.S - n
        buf = self.host.numpy()
        buf[self._tok] = list(tokens) + [tokens[0]] * pad
        buf[self._pos] = [s.start_pos for s in segments] + [segments[0].start_pos] * pad
        buf[self._slots] = [s.slot for s in segments] + [segments[0].slot] * pad
        for sl, w, tabs in zip(self._bt, self.widths, tables_per_group):
            bt = buf[sl].reshape(self.S, w)
            bt[:] = -1
            for i, t in enumerate(tabs):
                bt[i, :len(t)] = t
            if pad:
                bt[n:] = bt[0]
        first = segments[0]
        self.batch.segments = list(segments) + [
            Segment(first.req_id, first.slot, first.start_pos, 1, n + i, first.fresh) for i in range(pad)]
        self.dev.copy_(self.host, non_blocking=True)
        if self.dev.is_cuda:
            self._copied = torch.cuda.Event()
            self._copied.record()
        return self.batch
