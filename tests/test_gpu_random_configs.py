"""Random tiny configurations of the architecture (every size and option drawn anew: head sizes
in steps of 8, odd widths and vocabularies, one to sixteen query heads per kv head, windows that are
no multiple of a page, rope scaling on and off), each run through the engine in the four ways of
cutting and compared with the plain implementation.  The short ones have experts and run in both
precisions; the long ones (prompts of hundreds of tokens, portions of up to 260, so that the tcgen05
kernels and windows' edges deep inside a row tile are reached) have dense feed-forwards only, since
with random weights a router's near-tie would decide the comparison."""
import random

import pytest
import torch

import helpers as H
from spite_b200.config import Llama4Config
from spite_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def short_config(rng):
    nkv = rng.choice([1, 2, 3, 4])
    scaling = rng.choice([None, dict(rope_type="llama3", factor=rng.choice([2.0, 8.0, 16.0]), low_freq_factor=1.0,
                                     high_freq_factor=rng.choice([1.0, 4.0]),
                                     original_max_position_embeddings=rng.choice([32, 64, 256]))])
    return dict(architectures=["Llama4ForCausalLM"], num_hidden_layers=rng.choice([2, 3, 4, 5]),
                hidden_size=rng.choice([64, 72, 96, 100, 128, 136, 192, 200, 256]),
                num_attention_heads=nkv * rng.choice([1, 2, 3, 4, 5, 8]), num_key_value_heads=nkv,
                head_dim=rng.choice([16, 24, 32, 40, 48, 64, 80, 96, 128]), interleave_moe_layer_step=rng.choice([1, 1, 2, 3]),
                num_local_experts=rng.choice([2, 3, 4, 5, 8, 16]), num_experts_per_tok=1,
                intermediate_size=rng.choice([32, 48, 64, 72, 100, 128, 136]),
                intermediate_size_mlp=rng.choice([64, 96, 144, 200]), vocab_size=rng.choice([257, 300, 512, 1000, 1111]),
                tie_word_embeddings=rng.random() < 0.5, rope_theta=rng.choice([1000.0, 10000.0, 500000.0]),
                rope_scaling=scaling, attention_chunk_size=rng.choice([7, 16, 32, 48, 64, 96, 100, 128]),
                no_rope_layer_interval=rng.choice([2, 3, 4]), use_qk_norm=rng.random() < 0.5,
                attn_temperature_tuning=rng.random() < 0.5, floor_scale=rng.choice([8, 50, 8192]),
                attn_scale=rng.choice([0.1, 0.3]), rms_norm_eps=rng.choice([1e-5, 1e-6, 1e-4]),
                max_position_embeddings=4096)


def long_config(rng):
    nkv = rng.choice([1, 2, 3])
    return dict(short_config(rng), num_hidden_layers=rng.choice([2, 3]), hidden_size=rng.choice([64, 128, 136, 192, 256]),
                num_attention_heads=nkv * rng.choice([1, 2, 3, 5, 8, 16]), num_key_value_heads=nkv,
                head_dim=rng.choice([64, 128]), moe_layers=[], rope_scaling=None,
                attention_chunk_size=rng.choice([64, 96, 128, 200, 256, 300, 425, 1024]),
                no_rope_layer_interval=rng.choice([2, 3]), floor_scale=rng.choice([50, 200]))


def held_most(steps, page):
    """Most tokens live requests hold at any time, each rounded up to a page."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // page) * page for n in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return worst


def run_cuts(model, path, requests, cuts, tol, rng, pages):
    from spite_b200.engine import Engine
    results = {}
    for name, steps in cuts.items():
        page = rng.choice(pages)
        engine = Engine(model, cache_tokens=held_most(steps, page), page_size=page, max_requests=4)
        results[name] = H.run_steps(engine, steps)
        try:
            H.compare_with_plain(results[name], path, requests, tol)
        except AssertionError as e:
            raise AssertionError(f"{name}, pages of {page}: {e}") from None
    if model.dtype == torch.float32:
        H.assert_cuts_identical(results)          # not only close to the plain implementation: the same bits
    if model.dtype == torch.bfloat16:
        assert model.kernels.gemm_tc_error() == 0 and model.kernels.attention_tc_error() == 0


@pytest.mark.parametrize("seed", range(6))
def test_short_prompts_with_experts(seed, tmp_path):
    from spite_b200.engine import Model
    rng = random.Random(1000 + seed)
    config = short_config(rng)
    path = write_random_model(tmp_path / "m", Llama4Config.from_dict(config), seed=seed + 1, std=rng.choice([0.03, 0.05]),
                              dtype=torch.bfloat16)
    lengths = {"a": rng.randrange(60, 110), "b": rng.randrange(20, 80), "c": rng.randrange(33, 90), "d": rng.randrange(2, 40)}
    for dtype, margin in (("float32", 1e-4), ("bfloat16", 0.02)):
        requests = {r: H.decisive_tokens(path, n, seed * 10 + i, margin) for i, (r, n) in enumerate(lengths.items())}
        n_prompt = {r: max(2, len(t) - rng.randrange(0, 30)) for r, t in requests.items()}
        cuts = {"whole": H.steps_whole(requests), "last 32 one by one": H.steps_last_decoded(requests, 32),
                "portions": H.steps_portions(requests, seed), "mixed": H.steps_mixed(requests, n_prompt, seed=seed)}
        run_cuts(Model.from_folder(path, dtype=dtype, device="cuda:0"), path, requests, cuts, TOL[dtype], rng, [16, 32, 64])


@pytest.mark.parametrize("seed", range(6))
def test_long_prompts_dense(seed, tmp_path):
    from spite_b200.engine import Model
    rng = random.Random(2000 + seed)
    config = long_config(rng)
    path = write_random_model(tmp_path / "m", Llama4Config.from_dict(config), seed=seed + 1, std=0.04, dtype=torch.bfloat16)
    lengths = {"a": rng.randrange(300, 700), "b": rng.randrange(130, 400), "c": rng.randrange(20, 200)}
    requests = {r: H.random_tokens(config["vocab_size"], n, seed * 10 + i) for i, (r, n) in enumerate(lengths.items())}
    n_prompt = {r: max(2, len(t) - rng.randrange(0, 20)) for r, t in requests.items()}
    cuts = {"whole": H.steps_whole(requests), "last 32 one by one": H.steps_last_decoded(requests, 32),
            "portions": H.steps_portions(requests, seed, sizes=(2, 17, 64, 65, 128, 130, 200, 257)),
            "mixed": H.steps_mixed(requests, n_prompt, seed=seed, sizes=(2, 9, 40, 129, 150, 260)),
            "long decoding": H.steps_mixed(requests, {r: rng.randrange(2, 60) for r in requests}, seed=seed + 7, max_live=3)}
    for dtype in ("float32", "bfloat16"):
        run_cuts(Model.from_folder(path, dtype=dtype, device="cuda:0"), path, requests, cuts, TOL[dtype], rng, [16, 64, 64, 128])
