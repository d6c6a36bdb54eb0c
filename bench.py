"""Measurement: decode tokens per second of a Llama-4-Scout-shaped model with
random bfloat16 weights on one B200, plus prefill of 2,048 tokens, the decode
step's HBM roofline fraction, and decoding at batch 1 and 64.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Prints one JSON line.

Two further workloads print a line of the same kind (they are extra modes; the default line stays the one above):

    python bench.py --config maverick    # Llama-4-Maverick layer shapes, 4 layers (dense, MoE of 128 experts, dense, MoE):
                                         # 64 requests with prompts of 16 to 4,096 tokens through the scheduler
    python bench.py --config long        # Scout layer shapes, 8 layers: a prompt of 131,072 tokens in portions of
                                         # 8,192, then 256 decode steps at batch 1 and at batch 4
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-4-Scout layer shapes, 16 layers (the benchmark configuration)
SCOUT = dict(
    architectures=["Llama4ForCausalLM"], num_hidden_layers=16, hidden_size=5120, num_attention_heads=40,
    num_key_value_heads=8, head_dim=128, interleave_moe_layer_step=1, num_local_experts=16,
    num_experts_per_tok=1, intermediate_size=8192, intermediate_size_mlp=16384, vocab_size=202048,
    tie_word_embeddings=False, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=16.0, low_freq_factor=1.0, high_freq_factor=1.0,
                      original_max_position_embeddings=8192),
    attention_chunk_size=8192, no_rope_layer_interval=4, use_qk_norm=True, attn_temperature_tuning=True,
    floor_scale=8192, attn_scale=0.1, rms_norm_eps=1e-5, max_position_embeddings=131072)
FULL_LAYERS = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out, src = dict(FALLBACK_PEAKS), "fallback"
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            for k in out:
                if isinstance(raw.get(k), (int, float)) and raw[k] > 0:
                    out[k] = float(raw[k])
            src = "measured"
        except (OSError, ValueError):
            pass
    return out, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def decode_bytes(model, engine, contexts, distinct_experts):
    """Bytes a decode step has to read: every weight it uses once and the cache of the
    live requests (each layer reads the keys and values its window lets it see)."""
    from spite_b200.parts.feedforward import MoESigmoidPrescaled
    es = 2
    p = model.plan
    total = p.vocab_size * p.hidden_size * es                       # output head (embedding rows are negligible)
    for i, blk in enumerate(model.blocks):
        total += blk.mixer.weight_bytes() + blk.mixer_norm.weight_bytes() + blk.ffn_norm.weight_bytes()
        if isinstance(blk.ffn, MoESigmoidPrescaled):
            total += blk.ffn.active_weight_bytes(distinct_experts[i])
        else:
            total += blk.ffn.weight_bytes()
        win = blk.mixer.window
        for ctx in contexts:
            seen = ctx - win.lowest_visible(ctx - 1)
            total += seen * 2 * blk.mixer.nkv * blk.mixer.hd * es
    return total


def prefill_flops(cfg, T):
    d, hd, nq, nkv = cfg["hidden_size"], cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    f = cfg["intermediate_size"]
    per_layer = 2 * T * d * (nq + 2 * nkv) * hd + 2 * T * nq * hd * d        # projections
    per_layer += 2 * T * d * cfg["num_local_experts"]                          # router
    per_layer += 2 * (2 * T * d * 3 * f)                                       # routed + shared expert
    per_layer += 2 * 2 * nq * hd * T * (T + 1) // 2                            # causal attention
    return cfg["num_hidden_layers"] * per_layer + 2 * d * cfg["vocab_size"]    # one logits row


def prefill_roofline_ms(cfg, T, pk):
    """The time a prefill of T tokens cannot beat kernel by kernel: every product at the sustained bf16 rate or
    the time to read its weights once, whichever is longer, the attention at the bf16 rate, the head's weights."""
    d, hd, nq, nkv = cfg["hidden_size"], cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    f, E, k = cfg["intermediate_size"], cfg["num_local_experts"], cfg["num_experts_per_tok"]
    fl, bw = pk["bf16_tflops_sustained"] * 1e12, pk["hbm_gbs"] * 1e9
    both = lambda flops, nbytes: max(flops / fl, nbytes / bw)
    step = int(cfg.get("interleave_moe_layer_step", 1))
    total = 0.0
    for L in range(cfg["num_hidden_layers"]):
        total += both(2 * T * d * (nq + 2 * nkv) * hd, 2 * d * (nq + 2 * nkv) * hd) + both(2 * T * nq * hd * d, 2 * nq * hd * d)
        total += (2 * 2 * nq * hd * T * (T + 1) // 2) / fl
        if step > 0 and (L + 1) % step == 0:
            total += both(2 * T * d * 3 * f, 2 * 3 * d * f)                             # shared expert
            total += both(2 * T * k * d * 3 * f, 2 * 3 * d * f * min(E, T * k))         # routed experts
        else:
            fm = cfg["intermediate_size_mlp"]
            total += both(2 * T * d * 3 * fm, 2 * 3 * d * fm)
    return (total + 2 * d * cfg["vocab_size"] / bw) * 1e3


def build_model(cfgd):
    import torch
    from spite_b200.config import Llama4Config
    from spite_b200.engine import Model
    from spite_b200.kernels import build as kb
    torch.cuda.set_device(0)
    cfg = Llama4Config.from_dict(cfgd)
    model = Model.from_config(cfg, dtype="bfloat16", device="cuda:0")
    kb.ensure_built(model.kernel_libraries() + ["sampling"])
    model.init_random(seed=0, std=0.02)
    return cfg, model


def distinct_experts(model):
    """Per layer, how many experts the tokens of the last step used (0 for layers without experts)."""
    import torch
    out = []
    for blk in model.blocks:
        r = getattr(blk.ffn, "last_routing", None)
        out.append(torch.unique(r.expert_ids).numel() if r is not None else 0)
    return out


def base_line(metric, value, unit, steps, warmup, ms_per_step, config, data="synthetic (random token ids, random weights N(0,0.02))"):
    return {"metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": data, "config": config}


def run_maverick(args):
    """BASELINE configuration 4: sparse routing over 128 experts in mixed batches.  64 requests with prompts of 16
    to 4,096 random tokens and 32 new tokens each go through the public entry point (scheduler, portions of
    prompts beside decoded tokens under a budget of 4,096 tokens a step).  `value` is all tokens run (prompt and
    new) per second of device time; a "step" here is one step of the scheduler."""
    import random
    import torch
    from spite_b200.api import LLM
    cfgd = dict(SCOUT, num_hidden_layers=4, interleave_moe_layer_step=2, num_local_experts=128,
                intermediate_size_mlp=16384, rope_scaling=None)
    cfg, model = build_model(cfgd)
    n_req, new = 64, 32
    llm = LLM(model, ctx=8192, cache_tokens=n_req * 4224, max_requests=n_req, max_batch_tokens=4096)
    rng = random.Random(0)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(16, 4096))] for _ in range(n_req)]
    llm.generate(prompts, max_tokens=new, temperature=0.0)            # the same run once untimed: every kernel, shape and graph is warm
    pinned = [torch.tensor(p, dtype=torch.int32).pin_memory() for p in prompts]
    clocks = ClockSampler()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = model.kernels.launches
    with clocks:
        e0.record()
        outs = llm.generate([p.tolist() for p in pinned], max_tokens=new, temperature=0.0)
        e1.record()
        torch.cuda.synchronize()
    llm.engine.check()
    ms = e0.elapsed_time(e1)
    n_in, n_out = sum(map(len, prompts)), sum(map(len, outs))
    c = llm.last_counters
    line = base_line("tokens/s through the scheduler (Llama-4-Maverick-shaped, 64 requests, prompts 16-4096)",
                     (n_in + n_out) * 1e3 / ms, "tok/s", c["steps"], 1, ms / max(c["steps"], 1),
                     {"model": "llama4-maverick-shaped", "layers": 4, "layers_full": 48, "dense_layers": 2, "moe_layers": 2,
                      "hidden": 5120, "q_heads": 40, "kv_heads": 8, "head_dim": 128, "experts": 128, "top_k": 1,
                      "expert_ffn": 8192, "dense_ffn": 16384, "vocab": 202048, "requests": n_req,
                      "prompt_tokens": n_in, "new_tokens": n_out, "max_batch_tokens": 4096, "page_size": 64,
                      "parallelism": "single-gpu"})
    line.update({"gpu_launches": model.kernels.launches - l0, "clocks": clocks.summary(),
                 "scheduler": {"steps": c["steps"], "preemptions": c["preemptions"], "steps_ahead": c["steps_ahead"]},
                 "e2e": {"value": round((n_in + n_out) * 1e3 / ms, 2), "unit": "tok/s",
                         "h2d_bytes_per_step": round(4 * 4 * (n_in + n_out) / max(c["steps"], 1)), "d2h_bytes_per_step": 4 * n_req,
                         "note": "the whole run goes through LLM.generate: host token lists in, host token lists out"}})
    print(json.dumps(line))


def run_long(args):
    """BASELINE configuration 5: one request with a prompt of 131,072 tokens run in portions of 8,192 (many chunk
    windows on the chunked layers, the whole context on the layers without rotation), then 256 decode steps at
    batch 1, and the same at batch 4 (four such requests).  `value` is the decode rate at batch 1."""
    import torch
    from spite_b200.engine import Engine, StepEntry
    layers, C, portion, n_dec = args.layers if args.layers != FULL_LAYERS else 8, 131072, 8192, 256
    cfgd = dict(SCOUT, num_hidden_layers=layers, max_position_embeddings=C + 1024)
    cfg, model = build_model(cfgd)
    ks, pk = model.kernels, peaks()
    pk, pk_src = pk
    engine = Engine(model, cache_tokens=4 * (C + 1024), page_size=64, max_requests=4, max_positions=C + 1024)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg.vocab_size, (C,), generator=g, dtype=torch.int32).pin_memory()
    clocks = ClockSampler()

    def prefill(rid):
        ms = []
        for i in range(0, C, portion):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([StepEntry(rid, toks[i:i + portion].tolist(), [portion - 1] if i + portion == C else [])])
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        return ms

    def decode(rids, steps, warmup=3):
        ids = torch.randint(0, cfg.vocab_size, (steps + warmup, len(rids)), generator=g).tolist()
        for i in range(warmup):
            ks.argmax(engine.step([StepEntry(r, [ids[i][j]], [0]) for j, r in enumerate(rids)]))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            ks.argmax(engine.step([StepEntry(r, [ids[i][j]], [0]) for j, r in enumerate(rids)]))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        ctxs = [engine.cached_tokens(r) for r in rids]
        nbytes = decode_bytes(model, engine, ctxs, [float(n) for n in distinct_experts(model)])
        return ms, nbytes / (ms * 1e-3) / 1e9

    l0 = ks.launches
    with clocks:
        pre = prefill(0)
        ms1, gbs1 = decode([0], n_dec)
    for r in (1, 2, 3):
        prefill(r)
    ms4, gbs4 = decode([0, 1, 2, 3], n_dec)
    engine.check()
    line = base_line("decode tok/s at batch 1 after a 131,072-token prompt (Llama-4-Scout-shaped)", 1e3 / ms1, "tok/s",
                     n_dec, 3, ms1,
                     {"model": "llama4-scout-shaped", "layers": layers, "layers_full": 48, "hidden": 5120, "q_heads": 40,
                      "kv_heads": 8, "head_dim": 128, "experts": 16, "top_k": 1, "expert_ffn": 8192, "vocab": 202048,
                      "chunk": 8192, "nope_every": 4, "global_batch": 1, "seq_len": C, "portion": portion,
                      "page_size": 64, "parallelism": "single-gpu",
                      "l2": "inputs larger than L2 (weights and cache read per step exceed 126 MB)"})
    line.update({
        "gpu_launches": ks.launches - l0, "clocks": clocks.summary(),
        "prefill": {"value": round(C * 1e3 / sum(pre), 1), "tokens": C, "ms": round(sum(pre), 1),
                    "ms_first_portion": round(pre[0], 2), "ms_last_portion": round(pre[-1], 2)},
        "roofline": {"bound": "hbm", "achieved": round(gbs1, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs1 / pk["hbm_gbs"], 4), "peaks": pk_src},
        "points": {"decode_b1": round(1e3 / ms1, 1), "decode_b1_ms": round(ms1, 3), "decode_b1_hbm_frac": round(gbs1 / pk["hbm_gbs"], 4),
                   "decode_b4": round(4e3 / ms4, 1), "decode_b4_ms": round(ms4, 3), "decode_b4_hbm_frac": round(gbs4 / pk["hbm_gbs"], 4)},
        "e2e": {"value": round(1e3 / ms1, 2), "unit": "tok/s", "h2d_bytes_per_step": 4 * (6 + 2 * ((C + 1024) // 64 + 1)),
                "d2h_bytes_per_step": 0, "note": "token ids come from pinned host memory every step; the sampled ids stay on the device"}})
    print(json.dumps(line))


def run_ours(args):
    import torch
    from spite_b200.engine import Engine, StepEntry
    from spite_b200.engine.scheduler import Request, Scheduler
    from spite_b200.sampling import Sampler, SamplingParams

    dev = "cuda:0"
    cfgd = dict(SCOUT, num_hidden_layers=args.layers)
    cfg, model = build_model(cfgd)
    ks = model.kernels
    B, ctx = args.batch, args.context
    page = 64
    max_b = max(B, 64 if not args.skip_points else B)
    engine = Engine(model, cache_tokens=max_b * (ctx + page), page_size=page, max_requests=max_b,
                    max_positions=ctx + page, cuda_graphs=False if args.no_graphs else None)
    for kv in engine.storage.kv:                       # a cache as earlier steps would have left it
        kv.normal_(0.0, 1.0)
    g = torch.Generator().manual_seed(1)
    vocab = cfg.vocab_size

    def occupy(n_req, n_cached):
        for r in list(engine.cache.requests):
            engine.finish(r)
        for r in range(n_req):
            engine.cache.admit(r)
            engine.cache.reserve(r, n_cached)
            engine.cache.commit(r)

    def timed_decode(n_req, steps, warmup, clocks=None):
        start_ctx = ctx - (steps + warmup) - 1
        occupy(n_req, start_ctx)
        toks = torch.randint(0, vocab, (steps + warmup, n_req), generator=g).tolist()
        ids = None
        for i in range(warmup):
            ids = ks.argmax(engine.step([StepEntry(r, [toks[i][r]], [0]) for r in range(n_req)]))
        torch.cuda.synchronize()
        l0 = ks.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctxm = clocks if clocks is not None else _Null()
        with ctxm:
            e0.record()
            for i in range(warmup, warmup + steps):
                ids = ks.argmax(engine.step([StepEntry(r, [toks[i][r]], [0]) for r in range(n_req)]))
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        return ms / steps, ks.launches - l0, ids

    pk, pk_src = peaks()
    def measure_prefill():
        """Prefill of 2,048 tokens, logits of the last row."""
        T = 2048
        ptoks = torch.randint(0, vocab, (T,), generator=g).tolist()
        pre_ms = []
        for i in range(6):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([StepEntry("p", ptoks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            engine.finish("p")
            pre_ms.append(e0.elapsed_time(e1))
        pms = sorted(pre_ms[1:])[2]                       # the median of five runs after one warm-up
        pflops = prefill_flops(cfgd, T)
        if args.verbose:
            print("prefill runs (ms):", [round(x, 2) for x in pre_ms], file=sys.stderr)
        floor = prefill_roofline_ms(cfgd, T, pk)
        # frac: the step's flops / time / the sustained bf16 peak.  frac_kernel_roofline: the time the step's kernels
        # cannot beat one by one (the experts' weights make their products memory-bound at this length) / time
        return {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                "frac": round(pflops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                "roofline_ms": round(floor, 3), "frac_kernel_roofline": round(floor / pms, 4)}

    if args.only_prefill:
        print(json.dumps({"prefill": measure_prefill(), "layers": args.layers}))
        return
    clocks = ClockSampler()
    ms_step, launches, _ = timed_decode(B, args.steps, args.warmup, clocks)
    value = B * 1000.0 / ms_step
    def step_bytes(n_req):
        """Bytes a decode step of `n_req` requests at the end of the context has to read; the experts its tokens
        use, layer by layer, are the mean over a few more (untimed) steps of the same kind."""
        probe = 8
        occupy(n_req, ctx - probe - 1)
        ptoks = torch.randint(0, vocab, (probe, n_req), generator=g).tolist()
        distinct = [0.0] * len(model.blocks)
        for i in range(probe):
            engine.step([StepEntry(r, [ptoks[i][r]], [0]) for r in range(n_req)])
            for li, n in enumerate(distinct_experts(model)):
                distinct[li] += n / probe
        return decode_bytes(model, engine, [ctx - 1] * n_req, distinct)
    nbytes = step_bytes(B)
    achieved = nbytes / (ms_step * 1e-3) / 1e9
    engine.check()
    if args.only_decode:
        print(json.dumps({"decode_ms_per_step": round(ms_step, 4), "tok_per_s": round(value, 1), "batch": B,
                          "layers": args.layers, "launches": launches, "GBps": round(achieved, 1)}))
        return

    # end to end through the scheduler: host tokens in (pinned copy), sampled tokens out
    sched = Scheduler(engine, Sampler(ks), max_batch_tokens=4096, ctx=ctx + page)
    occupy(B, ctx - (args.steps + args.warmup) - 2)
    prompt_tail = torch.randint(0, vocab, (B,), generator=g).tolist()
    for r in range(B):
        req = Request(r, [0] * engine.cached_tokens(r) + [prompt_tail[r]],
                      SamplingParams(temperature=0.0, max_tokens=args.steps + args.warmup + 1))
        req.n_fed = engine.cached_tokens(r)
        req.state = req.state.__class__.PREFILLING
        req.rng_state = 0
        sched.running.append(req)
    for _ in range(args.warmup + 1):
        sched.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n_tok = 0
    for _ in range(args.steps - 1):
        n_tok += sum(1 for o in sched.step() if o.token is not None)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
    e2e = n_tok * 1000.0 / e2e_ms if e2e_ms > 0 else 0.0
    table_w = -(-(ctx + page) // page)
    h2d = 4 * (3 * B + (B + 1) + B + B + 2 * B * table_w)
    for r in list(engine.cache.requests):
        engine.finish(r)

    points = {}
    if not args.skip_points:
        for nb in (1, 64):
            pc = ClockSampler()
            # long enough for the clock sampler to see it: a step of one token takes a few milliseconds
            ms_b, _, _ = timed_decode(nb, max(4, args.steps * 4 if nb == 1 else args.steps // 2), 3, pc)
            gbs = step_bytes(nb) / (ms_b * 1e-3) / 1e9
            # each point with its own step time, fraction of the HBM roofline and clocks (flat: the record keeps one level)
            points.update({f"decode_b{nb}": round(nb * 1000.0 / ms_b, 1), f"decode_b{nb}_ms": round(ms_b, 4),
                           f"decode_b{nb}_GBps": round(gbs, 1), f"decode_b{nb}_hbm_frac": round(gbs / pk["hbm_gbs"], 4),
                           f"decode_b{nb}_sm_mhz": pc.summary()["sm_mhz"]})
        for r in list(engine.cache.requests):
            engine.finish(r)
    engine.check()

    prefill = measure_prefill()
    engine.check()

    line = {
        "metric": f"decode tok/s (Llama-4-Scout-shaped, batch {B}, context {ctx})",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random token ids, random weights N(0,0.02))",
        "config": {"model": "llama4-scout-shaped", "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": 5120, "q_heads": 40, "kv_heads": 8, "head_dim": 128, "experts": 16, "top_k": 1,
                   "expert_ffn": 8192, "shared_ffn": 8192, "vocab": 202048, "chunk": 8192, "nope_every": 4,
                   "global_batch": B, "seq_len": ctx, "page_size": page, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights read per step exceed 126 MB)",
                   "cache": "random-filled to context"},
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B,
                "ids_read": "one step late (decode steps are launched from the ids on the device)"
                if sched.counters["steps_ahead"] else "every step"},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes, "peaks": pk_src},
        "points": points,
    }
    print(json.dumps(line))


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def run_reference(args):
    # giveen/spite is a Rust workspace (Cargo.toml, no pyproject/setup.py): pip cannot install it, the
    # image has no cargo/rustc, and its Llama 4 path has no GPU kernel to run.
    print(json.dumps({"impl": "reference",
                      "unavailable": "giveen/spite is a Rust workspace without a Python package; "
                                     "no cargo/rustc offline, and its Llama 4 path is CPU-only"}))
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=["scout", "maverick", "long"], default="scout",
                    help="scout: the benchmark line; maverick, long: two further workloads, one line each")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step by itself")
    ap.add_argument("--only-decode", action="store_true", help="measure the decode step only (for profiling)")
    ap.add_argument("--only-prefill", action="store_true", help="measure the prefill step only (for profiling)")
    ap.add_argument("--verbose", action="store_true", help="print the single prefill timings to standard error")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this engine")
        return 2
    if args.config == "maverick":
        run_maverick(args)
        return 0
    if args.config == "long":
        run_long(args)
        return 0
    if args.warmup < 3:
        args.warmup = 3
    if args.steps < 1 or args.steps + args.warmup + 16 > args.context:
        print(f"bench.py: --steps {args.steps} with --warmup {args.warmup} does not fit the context of {args.context}")
        return 2
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
