"""Each hot kernel alone at Llama-4-Scout layer shapes: time (CUDA events, L2 flushed
between iterations), achieved bandwidth or throughput, and the fraction of the measured
peak.  Also the small driver that `ncu` captures for the summaries under `profiles/`.

    python bench_kernels.py                      # all cases, one JSON line each
    python bench_kernels.py --only gemm_decode   # one family (for ncu: -k regex:...)
    python bench_kernels.py --small              # shapes a profiler can replay in seconds
    python bench_kernels.py --only gemm_decode --case "lm_head M=8"   # one case
    python bench_kernels.py --only gemm_decode,moe_decode --rows 4,6   # the decode families at other token counts

Families: gemm_decode (weight streaming, mma.sync), gemm_prefill (tcgen05/TMA),
moe_decode, moe_prefill (grouped products), attention_decode, attention_prefill,
small (norm, rotation + cache append, router, sampling).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main(argv=None):
    import torch
    from bench import peaks
    from spite_b200.cache import LayerCache, Window
    from spite_b200.engine.batch import Segment, build_step_batch
    from spite_b200.kernels.cuda import CudaKernels

    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--case", default="", help="run only the cases whose name contains this text")
    ap.add_argument("--experts", type=int, default=16, help="experts of the grouped products (128: Maverick's)")
    ap.add_argument("--rows", default="1,8,64", help="token counts of the decode families")
    args = ap.parse_args(argv)
    dev = "cuda:0"
    torch.cuda.set_device(0)
    ks = CudaKernels(torch.bfloat16, dev)
    pk, src = peaks()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)       # larger than L2
    bf = torch.bfloat16
    d, F, V, nq, nkv, hd, E = 5120, 8192, 202048, 40, 8, 128, args.experts
    if args.small:
        V = 32768
    rnd = lambda *s: (torch.randn(s, device=dev, dtype=torch.float32) * 0.05).to(bf)

    def _timed(fn, iters):
        """One launch between two events, L2 flushed before it.  Includes the launch latency:
        right for kernels of hundreds of microseconds, too pessimistic for short ones."""
        for _ in range(3):
            fn()
        ms = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        ms.sort()
        return ms[len(ms) // 2]

    def _timed_rotating(make, nbytes, iters):
        """Short kernels: `make()` builds a launch closure on fresh operands; enough copies are
        made that together they exceed L2 several times, and they run back to back between two
        events, so every launch finds its operands in HBM and no launch gap is counted."""
        n = max(2, min(24, -(-3 * 160 * 1024 * 1024 // max(nbytes, 1))))
        fns = [make() for _ in range(n)]
        for f in fns:
            f()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()              # replayed, so that the host's launch rate does not count
        with torch.cuda.graph(graph):
            for f in fns:
                f()
        best = []
        for _ in range(max(3, iters // 2)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            best.append(e0.elapsed_time(e1) / n)
        best.sort()
        return best[len(best) // 2]

    # the timers are lazy, so that a case filtered out by --case launches nothing
    timed = lambda fn, iters=args.iters: (lambda: _timed(fn, iters))
    timed_rotating = lambda make, nbytes, iters=args.iters: (lambda: _timed_rotating(make, nbytes, iters))

    def report(family, name, timer, nbytes=0, flops=0, **extra):
        if args.case and args.case not in name:
            return
        ms = timer()
        out = {"family": family, "case": name, "us": round(ms * 1e3, 2)}
        if nbytes:
            gbs = nbytes / (ms * 1e-3) / 1e9
            out.update(GBps=round(gbs, 1), hbm_frac=round(gbs / pk["hbm_gbs"], 3))
        if flops:
            tf = flops / (ms * 1e-3) / 1e12
            out.update(TFLOPs=round(tf, 1), bf16_frac=round(tf / pk["bf16_tflops"], 3))
        out.update(peaks=src, **extra)
        print(json.dumps(out), flush=True)

    want = lambda fam: not args.only or fam in args.only.split(",")

    # ---- plain products
    shapes = [("qkv", (nq + 2 * nkv) * hd, d), ("o_proj", d, nq * hd), ("shared_down", d, F), ("lm_head", V, d)]
    decode_rows = tuple(int(m) for m in args.rows.split(","))
    if want("gemm_decode"):
        for M in decode_rows:
            for name, N, K in shapes:
                def make(M=M, N=N, K=K, name=name):
                    x, w = rnd(M, K), rnd(N, K)
                    out = torch.empty((M, N), dtype=torch.float32 if name == "lm_head" else bf, device=dev)
                    return lambda: ks.linear(x, w, out)
                nbytes = 2 * N * K + 2 * M * K + (4 if name == "lm_head" else 2) * M * N
                report("gemm_decode", f"{name} M={M} N={N} K={K}", timed_rotating(make, nbytes), nbytes=nbytes)
            def make(M=M):
                x, w = rnd(M, d), rnd(2 * F, d)
                out = torch.empty((M, F), dtype=bf, device=dev)
                return lambda: ks.linear_swiglu(x, w, out)
            nbytes = 2 * 2 * F * d + 2 * M * d + 2 * M * F
            report("gemm_decode", f"shared_gate_up_swiglu M={M} N=2x{F} K={d}", timed_rotating(make, nbytes),
                   nbytes=nbytes)
    if want("gemm_prefill"):
        for M in ((512,) if args.small else (256, 2048, 8192)):
            for name, N, K in shapes[:3]:
                x, w = rnd(M, K), rnd(N, K)
                out = torch.empty((M, N), dtype=bf, device=dev)
                report("gemm_prefill", f"{name} M={M} N={N} K={K}", timed(lambda: ks.linear(x, w, out)),
                       flops=2 * M * N * K, nbytes=2 * (N * K + M * K + M * N))
                del w
            x, w = rnd(M, d), rnd(2 * F, d)
            out = torch.empty((M, F), dtype=bf, device=dev)
            report("gemm_prefill", f"shared_gate_up_swiglu M={M} N=2x{F} K={d}",
                   timed(lambda: ks.linear_swiglu(x, w, out)), flops=2 * M * 2 * F * d)
            del w
        assert ks.gemm_tc_error() == 0

    # ---- grouped products (experts)
    def routed(M):
        g = torch.Generator(device=dev).manual_seed(M)
        ids = torch.randint(0, E, (M,), device=dev, generator=g)
        order = torch.sort(ids, stable=True)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=dev)
        offsets[1:] = torch.cumsum(torch.bincount(ids, minlength=E), 0)
        return order.indices.to(torch.int32), offsets, int(ids.unique().numel())
    for fam, Ms in (("moe_decode", decode_rows), ("moe_prefill", (512,) if args.small else (256, 512, 1024, 2048, 8192))):
        if not want(fam):
            continue
        w_gu, w_dn = rnd(E, 2 * F, d), rnd(E, d, F)
        for M in Ms:
            rows, offsets, used = routed(M)
            used = E if M > 64 else used
            x, scale = rnd(M, d), torch.rand(M, device=dev)
            a = torch.empty((M, F), dtype=bf, device=dev)
            h = torch.zeros((M, d), dtype=torch.float32, device=dev)
            report(fam, f"experts_gate_up_swiglu M={M} experts_used={used}",
                   timed(lambda: ks.grouped_linear_swiglu(x, w_gu, rows, offsets, scale, a)),
                   nbytes=used * 2 * 2 * F * d, flops=2 * M * 2 * F * d)
            report(fam, f"experts_down_add M={M} experts_used={used}",
                   timed(lambda: ks.grouped_linear_accumulate(a, w_dn, rows, offsets, h)),
                   nbytes=used * 2 * F * d, flops=2 * M * F * d)
        del w_gu, w_dn

    # ---- attention over the paged cache
    P = 64
    def attention_case(fam, n_req, n_new, ctx, window):
        pages_per = -(-ctx // P)
        win = Window(*window)
        segs, tables, off = [], [], 0
        for r in range(n_req):
            segs.append(Segment(r, r, ctx - n_new, n_new, off, False))
            tables.append(list(range(r * pages_per, (r + 1) * pages_per)))
            off += n_new
        batch = build_step_batch(segs, [[0] * n_new] * n_req, [[]] * n_req, [tables], dev)
        def make():
            kv = (torch.randn((2, n_req * pages_per, nkv, P, hd), device=dev) * 0.5).to(bf)
            q, out = rnd(off, nq * hd), torch.empty((off, nq * hd), dtype=bf, device=dev)
            cache = LayerCache(0, kv, None, P, False)
            return lambda: ks.paged_attention(q, out, batch, cache, num_heads=nq, window=win,
                                              softmax_scale=1 / math.sqrt(hd))
        seen = sum(min(p + 1, ctx) - win.lowest_visible(p) for p in range(ctx - n_new, ctx)) / n_new
        if n_new == 1:
            # short launches: back to back over rotating copies of the cache, so no launch gap is counted
            nbytes = int(n_req * seen * 2 * nkv * hd * 2)
            report(fam, f"requests={n_req} context={ctx} window={window[0]}", timed_rotating(make, nbytes), nbytes=nbytes)
            return
        report(fam, f"tokens={n_new} context={ctx} window={window[0]}", timed(make()),
               flops=int(n_req * n_new * seen * 4 * nq * hd))
    if want("attention_decode"):
        for n_req in ((8,) if args.small else (1, 8, 64)):
            attention_case("attention_decode", n_req, 1, 2048 if args.small else 8192, ("full", 0))
    if want("attention_prefill"):
        attention_case("attention_prefill", 1, 512 if args.small else 2048, 512 if args.small else 2048, ("full", 0))
        if not args.small:
            attention_case("attention_prefill", 1, 2048, 8192, ("chunk", 8192))
            attention_case("attention_prefill", 1, 8192, 131072, ("full", 0))     # a late portion of a long prompt

    # ---- rotation + per-head norm + cache append, at decode and at prompt lengths
    if want("small"):
        from spite_b200.parts import QkNorm, Rotation
        for M in (8, 2048):
            pages_per = -(-M // P) + 1
            segs = [Segment(0, 0, 0, M, 0, True)]
            batch = build_step_batch(segs, [[0] * M], [[]], [[list(range(pages_per))]], dev)
            inv_freq = torch.tensor([500000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float32, device=dev)
            def make_prepare(M=M, batch=batch, pages_per=pages_per):
                qkv = rnd(M, (nq + 2 * nkv) * hd)
                q = torch.empty((M, nq * hd), dtype=bf, device=dev)
                kv = torch.zeros((2, pages_per, nkv, P, hd), dtype=bf, device=dev)
                cache = LayerCache(0, kv, None, P, True)
                return lambda: ks.qk_prepare(qkv, q, batch, cache, num_heads=nq, rotation=Rotation(inv_freq, "neighbours"),
                                             qk_norm=QkNorm(1e-5), temperature=None)
            nbytes = M * ((nq + 2 * nkv) * hd * 2 + (nq + 2 * nkv) * hd * 2)
            report("small", f"qk_prepare M={M}", timed_rotating(make_prepare, max(nbytes, 64 << 20) if M == 8 else nbytes), nbytes=nbytes)

    # ---- the small kernels of a decode step
    if want("small"):
        for M in (8, 64):
            def make_norm(M=M):
                h, gain = torch.randn((M, d), device=dev), torch.ones(d, device=dev)
                x = torch.empty((M, d), dtype=bf, device=dev)
                return lambda: ks.rms_norm(h, gain, 1e-5, x)
            report("small", f"rms_norm M={M}", timed_rotating(make_norm, 64 << 20), nbytes=M * d * 6)
            def make_route(M=M):
                x, wr = rnd(M, d), torch.randn((E, d), device=dev) * 0.05
                return lambda: ks.moe_route(x, wr, 1)
            report("small", f"router M={M}", timed_rotating(make_route, 64 << 20), nbytes=E * d * 4 + M * d * 2)
            def make_argmax(M=M):
                logits = torch.randn((M, V), device=dev)
                return lambda: ks.argmax(logits)
            report("small", f"argmax M={M} V={V}", timed_rotating(make_argmax, M * V * 4), nbytes=M * V * 4)
            def make_sample(M=M):
                logits = torch.randn((M, V), device=dev) * 3
                f32 = lambda v: torch.full((M,), v, dtype=torch.float32, device=dev)
                ctxt = torch.randint(0, V, (M * 64,), dtype=torch.int32, device=dev)
                offs = torch.arange(0, M * 64 + 1, 64, dtype=torch.int32, device=dev)
                state = torch.arange(M, dtype=torch.int64, device=dev)
                return lambda: ks.sample(logits, temperature=f32(0.7), top_k=torch.zeros(M, dtype=torch.int32, device=dev),
                                         top_p=f32(0.95), min_p=f32(0.0), repetition_penalty=f32(1.1), context=ctxt,
                                         context_offsets=offs, rng_state=state)
            report("small", f"sample (temperature 0.7, top-p 0.95, penalty 1.1) M={M} V={V}",
                   timed_rotating(make_sample, M * V * 4), nbytes=M * V * 4)
    return 0


if __name__ == "__main__":
    sys.exit(main())
