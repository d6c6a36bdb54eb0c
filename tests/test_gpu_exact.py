"""float32 exactness.

1. The four ways of cutting the same requests into steps give the same bits: prefill == incremental as
   crates/spite-models/src/llama/llama4.rs:377-389 asserts it (`==`, not "close"), batched == sequential as
   tools/verify/verify_batch.py:131-206 does.  For the four fixed tiny configurations (the random ones
   assert the same in test_gpu_random_configs.py).
2. Layer sizes of Llama-4-Scout (width 5120, 40/8 heads of 128, 16 experts of 8192, vocabulary 202048) with
   two layers, one rotary with a chunk of 128 and one without rotation, in true float32 against the plain
   implementation, cut in every way; and the bfloat16 engine on the same weights.
"""
import random

import pytest
import torch

import helpers as H
import plain_llama4 as plain

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------- 1. the same bits under every cut
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_float32_logits_do_not_depend_on_the_cut(name, tmp_path):
    from spite_b200.engine import Engine, Model
    path = H.write_model(tmp_path / name, name)
    model = Model.from_folder(path, dtype="float32", device="cuda:0")
    vocab = model.plan.vocab_size
    lengths = {"a": 150, "b": 40, "c": 77, "d": 66, "e": 21} if name != "C" else {"a": 300, "b": 130, "c": 97, "d": 45}
    requests = {r: H.random_tokens(vocab, n, 900 + i) for i, (r, n) in enumerate(lengths.items())}
    big = (2, 5, 43, 64, 90, 128)
    cuts = {
        "whole": (H.steps_whole(requests), 16),
        "whole, pages of 64": (H.steps_whole(requests), 64),
        "last 32 one by one": (H.steps_last_decoded(requests, 32), 16),
        "portions": (H.steps_portions(requests, 5), 16),
        "large portions": (H.steps_portions(requests, 6, sizes=big), 64),
        "mixed, pages used again": (H.steps_mixed(requests, {r: max(2, len(t) - 12) for r, t in requests.items()}, 7), 16),
        "mixed, long decoding": (H.steps_mixed(requests, {r: 2 + i for i, r in enumerate(requests)}, 8, max_live=3), 32),
    }
    results = {}
    for cut, (steps, page) in cuts.items():
        eng = Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page, max_requests=4)
        results[cut] = H.run_steps(eng, steps)
    assert H.assert_cuts_identical(results) >= 6 * sum(lengths.values())
    H.compare_with_plain(results["whole"], path, requests, 2e-5)


# ---------------------------------------------------------------------------- 2. Scout layer sizes
SCOUT_2_LAYERS = dict(
    architectures=["Llama4ForCausalLM"], num_hidden_layers=2, hidden_size=5120, num_attention_heads=40,
    num_key_value_heads=8, head_dim=128, interleave_moe_layer_step=1, num_local_experts=16,
    num_experts_per_tok=1, intermediate_size=8192, intermediate_size_mlp=16384, vocab_size=202048,
    tie_word_embeddings=False, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=16.0, low_freq_factor=1.0, high_freq_factor=1.0,
                      original_max_position_embeddings=8192),
    attention_chunk_size=128,            # small enough to be crossed by a prompt the plain implementation can afford
    no_rope_layer_interval=2,            # layer 0 rotary + chunked, layer 1 without rotation, global, temperature
    use_qk_norm=True, attn_temperature_tuning=True, floor_scale=50, attn_scale=0.1, rms_norm_eps=1e-5,
    max_position_embeddings=8192)
MARGIN = 0.05         # router logit margin that bfloat16 rounding of a 5120-wide sum cannot flip


def _clear_routing_tokens(model, n, seed, min_margin):
    """A token sequence whose routing decisions all have a clear margin, grown token by token with the
    float32 engine: candidate t is kept if, run as the last token of tokens[:t] + [candidate], the two
    best router logits of both layers differ by `min_margin`."""
    from spite_b200.engine import Engine
    rng = random.Random(seed)
    vocab = model.plan.vocab_size
    moes = [b.ffn for b in model.blocks]
    for m in moes:
        m.keep_router_logits = True
    toks = []
    eng = Engine(model, cache_tokens=-(-(n + 1) // 64) * 64, page_size=64, max_requests=2, cuda_graphs=False)
    while len(toks) < n:
        for _ in range(50):
            cand = toks + [rng.randrange(vocab)]
            eng.step([("probe", cand, [])])
            eng.finish("probe")
            worst = min(float((lambda top: top[0] - top[1])(m.last_routing.logits[-1].topk(2).values)) for m in moes)
            if worst >= min_margin:
                toks = cand
                break
        else:
            raise RuntimeError("no token with clear routing found")
    for m in moes:
        m.keep_router_logits = False
    return toks


@pytest.fixture(scope="module")
def scout():
    """Checkpoint tensors of the two Scout-sized layers, made on the device (12.6 GB in bfloat16; a folder
    of that size is not worth writing), the float32 model bound to them, and the plain implementation's
    copies on the host."""
    from spite_b200.config import Llama4Config
    from spite_b200.engine import Model
    from spite_b200.weights import random_checkpoint_tensors
    config = Llama4Config.from_dict(SCOUT_2_LAYERS)
    tensors = random_checkpoint_tensors(config, seed=7, std=0.02, dtype=torch.bfloat16, device="cuda:0")
    model32 = Model.from_tensors(config, tensors, dtype="float32", device="cuda:0")
    main = _clear_routing_tokens(model32, 168, 1, MARGIN)           # crosses the chunk edge at 128
    other = _clear_routing_tokens(model32, 70, 2, MARGIN)
    host = {k: v.cpu() for k, v in tensors.items()}
    cfg = dict(SCOUT_2_LAYERS)
    info = {}
    refs = {"m": plain.forward(cfg, host, main, collect=info), "o": plain.forward(cfg, host, other)}
    assert float(info["router_margins"].min()) >= MARGIN / 2        # the plain implementation sees the same margins
    del host
    return dict(config=config, tensors=tensors, model32=model32, requests={"m": main, "o": other}, refs=refs)


def _cuts(requests):
    m, o = requests["m"], requests["o"]
    portions = []
    i = 0
    for n in (64, 100, 2, 2):                                        # 64 / 100 / 2 / the rest, as the contract names them
        portions.append({"entries": [{"id": "m", "tokens": m[i:i + n], "want": list(range(n))}], "end": []})
        i += n
    assert i == len(m)
    portions[-1]["end"] = ["m"]
    mixed = [
        {"entries": [{"id": "m", "tokens": m[:120], "want": list(range(120))}], "end": []},
        {"entries": [{"id": "m", "tokens": m[120:160], "want": list(range(40))},            # crosses the chunk edge
                     {"id": "o", "tokens": o[:50], "want": list(range(50))}], "end": []},
    ]
    for j in range(8):                                               # m decodes beside o's portions and decodes
        e = [{"id": "m", "tokens": [m[160 + j]], "want": [0]}]
        if j < 5:
            e.append({"id": "o", "tokens": o[50 + 4 * j:54 + 4 * j], "want": [0, 1, 2, 3]})
        mixed.append({"entries": e, "end": ["m"] if j == 7 else []})
    mixed.append({"entries": [], "end": ["o"]})
    # portions of 6 to 40 tokens: the sizes of larger decode batches, which the weight-streaming products take with
    # tiles of fewer rows (k slices) and with 16 or 32 token columns
    medium, i = [], 0
    for n in (8, 12, 24, 30, 6, 16, 32, 40):
        medium.append({"entries": [{"id": "m", "tokens": m[i:i + n], "want": list(range(n))}], "end": []})
        i += n
    assert i == len(m)
    medium[-1]["end"] = ["m"]
    cuts = {"whole": H.steps_whole(requests), "last 8 one by one": H.steps_last_decoded(requests, 8),
            "portions 64/100/2/2": portions, "mixed beside a second request": mixed,
            "portions of 6 to 40": medium}
    for steps in cuts.values():
        for k, s in enumerate(steps):
            s["step"] = k
    return cuts


def _compare(results, refs, requests, tol, what):
    worst = 0.0
    for (r, p), row in results.items():
        ref = refs[r]
        err = float((row - ref[p]).abs().max()) / float(ref.abs().max())
        worst = max(worst, err)
        assert err <= tol, f"{what}: request {r!r}, position {p}: error {err:.3e} of the logit scale exceeds {tol:.1e}"
    H.note_error(worst, tol)
    return worst


def test_scout_layer_sizes_in_float32(scout):
    from spite_b200.engine import Engine
    results = {}
    for cut, steps in _cuts(scout["requests"]).items():
        eng = Engine(scout["model32"], cache_tokens=H.max_tokens_of(steps), page_size=64, max_requests=2)
        results[cut] = H.run_steps(eng, steps)
        worst = _compare(results[cut], scout["refs"], scout["requests"], 2e-5, cut)
        print(f"scout float32, {cut}: worst error {worst:.2e} of the logit scale")
    H.assert_cuts_identical(results)
    assert len(results["whole"]) == 168 + 70


def test_scout_layer_sizes_in_bfloat16_on_the_same_weights(scout):
    """The serving kernels (tcgen05 products and attention for the portions, weight streaming and split-key
    attention for the decoded tokens) at the sizes they were written for, against the plain implementation."""
    from spite_b200.engine import Engine, Model
    scout["model32"] = None                                          # 25 GB back before the next model
    torch.cuda.empty_cache()
    model = Model.from_tensors(scout["config"], scout["tensors"], dtype="bfloat16", device="cuda:0")
    for cut, steps in _cuts(scout["requests"]).items():
        eng = Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=64, max_requests=2)
        worst = _compare(H.run_steps(eng, steps), scout["refs"], scout["requests"], 4e-2, cut)
        print(f"scout bfloat16, {cut}: worst error {worst:.2e} of the logit scale")
    assert model.kernels.errors() == {}
    used = model.kernels.launches_by_library
    assert all(used[lib] > 0 for lib in ("gemm_tc", "gemm_stream", "attention_tc", "attention_decode")), dict(used)
