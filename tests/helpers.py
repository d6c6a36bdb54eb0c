"""Shared fixtures of the tests: two tiny Llama 4 configurations that differ in
every size and option, model folders with random weights, token sequences, and
the four ways of cutting the same requests into steps."""
from __future__ import annotations

import functools
import random
from pathlib import Path

import torch

import plain_llama4 as plain
from spite_b200.config import Llama4Config
from spite_b200.weights import write_random_model

# 4 layers, all MoE, NoPE layer 3, chunk 32, qk-norm and temperature tuning on, untied head
CONFIG_A = dict(
    architectures=["Llama4ForCausalLM"], num_hidden_layers=4, hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, interleave_moe_layer_step=1, num_local_experts=4,
    num_experts_per_tok=1, intermediate_size=128, intermediate_size_mlp=256, vocab_size=512,
    tie_word_embeddings=False, rope_theta=10000.0, rope_scaling=None, attention_chunk_size=32,
    no_rope_layer_interval=4, use_qk_norm=True, attn_temperature_tuning=True, floor_scale=16,
    attn_scale=0.1, rms_norm_eps=1e-5, max_position_embeddings=4096)
STD_A = 0.02

# 6 layers, dense/MoE alternating, NoPE layers 2 and 5, chunk 16, one kv head, llama3 scaling, tied head
CONFIG_B = dict(
    architectures=["Llama4ForCausalLM"], num_hidden_layers=6, hidden_size=96, num_attention_heads=6,
    num_key_value_heads=1, head_dim=32, interleave_moe_layer_step=2, num_local_experts=8,
    num_experts_per_tok=1, intermediate_size=64, intermediate_size_mlp=192, vocab_size=1000,
    tie_word_embeddings=True, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
    attention_chunk_size=16, no_rope_layer_interval=3, use_qk_norm=False, attn_temperature_tuning=False,
    floor_scale=8192, attn_scale=0.1, rms_norm_eps=1e-6, max_position_embeddings=2048)
STD_B = 0.05

# Sizes that reach the tcgen05 kernels: head size 64, widths that are multiples of 8, three query heads
# per kv head; chunk 96 ends inside a 64-key tile; layer 1 has no rotation and sees every key
CONFIG_C = dict(
    architectures=["Llama4ForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=6,
    num_key_value_heads=2, head_dim=64, interleave_moe_layer_step=1, num_local_experts=3,
    num_experts_per_tok=1, intermediate_size=72, intermediate_size_mlp=144, vocab_size=300,
    tie_word_embeddings=False, rope_theta=10000.0, rope_scaling=None, attention_chunk_size=96,
    no_rope_layer_interval=2, use_qk_norm=True, attn_temperature_tuning=True, floor_scale=50,
    attn_scale=0.2, rms_norm_eps=1e-5, max_position_embeddings=4096)
STD_C = 0.03

# Awkward sizes: a width that is no multiple of 8, a head size that is no multiple of 16, seven query heads
# on one kv head, an odd vocabulary, five experts, a window shorter than a page
CONFIG_D = dict(
    architectures=["Llama4ForCausalLM"], num_hidden_layers=3, hidden_size=100, num_attention_heads=7,
    num_key_value_heads=1, head_dim=24, interleave_moe_layer_step=1, num_local_experts=5,
    num_experts_per_tok=1, intermediate_size=44, intermediate_size_mlp=60, vocab_size=301,
    tie_word_embeddings=True, rope_theta=1000.0, rope_scaling=None, attention_chunk_size=9,
    no_rope_layer_interval=3, use_qk_norm=True, attn_temperature_tuning=False, floor_scale=8192,
    attn_scale=0.1, rms_norm_eps=1e-4, max_position_embeddings=1024)
STD_D = 0.05

CONFIGS = {"A": (CONFIG_A, STD_A, 11), "B": (CONFIG_B, STD_B, 23), "C": (CONFIG_C, STD_C, 31),
           "D": (CONFIG_D, STD_D, 47)}


def write_model(folder, name: str, dtype=torch.bfloat16) -> Path:
    cfg, std, seed = CONFIGS[name]
    return write_random_model(folder, Llama4Config.from_dict(cfg), seed=seed, std=std, dtype=dtype)


@functools.lru_cache(maxsize=None)
def _folder_contents(folder: str):
    return plain.read_model_folder(folder)


_plain_cache: dict = {}


def plain_logits(folder, tokens) -> torch.Tensor:
    """Logits [T, vocab] of the plain implementation for one whole sequence (cached)."""
    key = (str(folder), tuple(tokens))
    if key not in _plain_cache:
        cfg, tensors = _folder_contents(str(folder))
        _plain_cache[key] = plain.forward(cfg, tensors, list(tokens))
    return _plain_cache[key]


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def decisive_tokens(folder, n: int, seed: int, min_margin: float) -> list[int]:
    """A token sequence in which every routing decision of the plain implementation
    is clear: the chosen expert's logit exceeds the next by `min_margin` at every MoE
    layer and position.  A comparison in bfloat16 is meaningless where rounding
    decides which expert runs; the sequence is grown token by token (the model is
    causal, so earlier margins do not change)."""
    cfg, tensors = _folder_contents(str(folder))
    rng = random.Random(seed)
    vocab = cfg["vocab_size"]
    toks: list[int] = []
    while len(toks) < n:
        for _ in range(200):
            cand = toks + [rng.randrange(vocab)]
            info = {}
            plain.forward(cfg, tensors, cand, collect=info)
            m = info["router_margins"]
            if m.numel() == 0 or float(m[:, -1].min()) >= min_margin:
                toks = cand
                break
        else:
            raise RuntimeError("no token with clear routing found")
    return toks


# ----------------------------------------------------------------------------
# cutting requests into steps
# ----------------------------------------------------------------------------
def _round64(n):
    return -(-n // 64) * 64


def steps_whole(requests: dict) -> list[dict]:
    """Each request alone and whole: one step with all its tokens."""
    return [{"step": i, "entries": [{"id": r, "tokens": list(t), "want": list(range(len(t)))}], "end": [r]}
            for i, (r, t) in enumerate(requests.items())]


def steps_last_decoded(requests: dict, n_last: int = 32) -> list[dict]:
    """Most of a request in one step, its last `n_last` tokens one by one."""
    steps = []
    for r, t in requests.items():
        cut = max(1, len(t) - n_last)
        steps.append({"entries": [{"id": r, "tokens": list(t[:cut]), "want": list(range(cut))}], "end": []})
        for i in range(cut, len(t)):
            steps.append({"entries": [{"id": r, "tokens": [t[i]], "want": [0]}],
                          "end": [r] if i == len(t) - 1 else []})
        if cut == len(t):
            steps[-1]["end"] = [r]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def steps_portions(requests: dict, seed: int = 0, sizes=(2, 3, 5, 7, 11, 16, 17, 29)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    steps = []
    for r, t in requests.items():
        i = 0
        while i < len(t):
            n = rng.choice(sizes)
            if len(t) - i - n == 1:          # never leave a single token for a "portion"
                n += 1
            n = min(n, len(t) - i)
            steps.append({"entries": [{"id": r, "tokens": list(t[i:i + n]), "want": list(range(n))}],
                          "end": [r] if i + n == len(t) else []})
            i += n
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def steps_mixed(requests: dict, n_prompt: dict, seed: int = 0, max_live: int = 4,
                sizes=(2, 3, 4, 6, 9, 14)) -> list[dict]:
    """Up to `max_live` live requests: portions of some prompts beside single decoded
    tokens of others; a request sometimes sits a step out.  The first `n_prompt[r]`
    tokens of request r come in portions, the rest one by one."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: dict = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            live[waiting.pop(0)] = 0
        entries, ends = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            i, t = live[r], requests[r]
            if i < n_prompt[r]:
                n = min(rng.choice(sizes), n_prompt[r] - i)
                if n_prompt[r] - i - n == 1:
                    n += 1
            else:
                n = 1
            n = min(n, len(t) - i)
            entries.append({"id": r, "tokens": list(t[i:i + n]), "want": list(range(n))})
            live[r] = i + n
            if live[r] == len(t):
                ends.append(r)
                del live[r]
        if entries:
            steps.append({"entries": entries, "end": ends})
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def max_tokens_of(steps) -> int:
    """Most tokens live requests hold at any time, each rounded up to 64."""
    held: dict = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(_round64(n) for n in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return worst


def run_steps(engine, steps, before_step=None) -> dict:
    """Drive `engine.step` with `steps`; returns {(request, position): logits row (CPU float32)}.
    `before_step(engine)`, if given, runs before every step."""
    from spite_b200.engine import StepEntry
    pos: dict = {}
    out = {}
    for s in steps:
        if before_step is not None:
            before_step(engine)
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = engine.step(entries).float().cpu()
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = logits[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        for r in s["end"]:
            engine.finish(r)
            pos.pop(r, None)
        engine.cache.check_invariants()
    return out


#: worst error seen per test (name of the running test -> (error, tolerance)); the summary at the end of a
#: run prints it, so that a tolerance can be set from what the runs show
WORST: dict = {}


def note_error(err: float, tol: float):
    import os
    test = os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0]
    if err > WORST.get(test, (-1.0, tol))[0]:
        WORST[test] = (err, tol)


def compare_with_plain(results: dict, folder, requests: dict, tol: float):
    """Every logits row against the plain implementation; the error is measured
    against the largest logit magnitude of the row's sequence.  Returns the worst
    relative error; raises AssertionError naming the first position beyond `tol`."""
    worst = 0.0
    for r, toks in requests.items():
        ref = plain_logits(folder, toks)
        scale = float(ref.abs().max())
        for p in range(len(toks)):
            if (r, p) not in results:
                continue
            err = float((results[(r, p)] - ref[p]).abs().max()) / scale
            worst = max(worst, err)
            assert err <= tol, (f"request {r!r}, position {p} (first wrong one): error {err:.3e} of the "
                                f"logit scale exceeds {tol:.1e} (worst before it: {worst:.3e})")
    note_error(worst, tol)
    return worst


def assert_cuts_identical(results_by_cut: dict):
    """float32 only: the logits of a (request, position) are the same bits whichever way the requests were
    cut into steps, whatever else was in the batch and whichever pages held the keys (every kernel's order
    of additions for one output element depends on that element's own data alone).  Names the first
    position that differs and by how much."""
    names = list(results_by_cut)
    base = results_by_cut[names[0]]
    compared = 0
    for other in names[1:]:
        res = results_by_cut[other]
        for key in sorted(base.keys() & res.keys(), key=lambda k: (str(k[0]), k[1])):
            compared += 1
            if not torch.equal(base[key], res[key]):
                diff = (base[key] - res[key]).abs()
                raise AssertionError(
                    f"request {key[0]!r}, position {key[1]} (first one that differs): {names[0]!r} and {other!r} "
                    f"disagree in {int((diff > 0).sum())} of {diff.numel()} logits, by up to {float(diff.max()):.3e}")
    assert compared > 0, "the cuts share no (request, position)"
    return compared
