"""The engine's host logic (cache manager, block tables, batches, step function,
trace replay) without a GPU: the kernels are replaced by their plain torch
restatements (`reference_kernels.py`), everything else is the product code.
The results are compared with the plain whole-sequence implementation."""
import io
import json

import numpy as np
import pytest
import torch

import helpers as H
from reference_kernels import TorchReferenceKernels
from spite_b200.cache import OutOfPages
from spite_b200.engine import Engine, Model
from spite_b200.engine.trace import replay

TOL = 2e-5


@pytest.fixture(scope="module", params=["A", "B"])
def setup(request, tmp_path_factory):
    folder = H.write_model(tmp_path_factory.mktemp(f"model{request.param}"), request.param)
    model = Model.from_folder(folder, dtype="float32", device="cpu",
                              kernels=TorchReferenceKernels(torch.float32, "cpu"))
    vocab = model.plan.vocab_size
    requests = {"a": H.random_tokens(vocab, 83, 1), "b": H.random_tokens(vocab, 40, 2),
                "c": H.random_tokens(vocab, 37, 3), "d": H.random_tokens(vocab, 66, 4),
                "e": H.random_tokens(vocab, 21, 5)}
    return folder, model, requests


def _engine(model, steps, page_size):
    return Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page_size, max_requests=4)


@pytest.mark.parametrize("page_size", [16, 64])
def test_whole(setup, page_size):
    folder, model, requests = setup
    steps = H.steps_whole(requests)
    res = H.run_steps(_engine(model, steps, page_size), steps)
    assert len(res) == sum(len(t) for t in requests.values())
    H.compare_with_plain(res, folder, requests, TOL)


def test_last_tokens_decoded(setup):
    folder, model, requests = setup
    steps = H.steps_last_decoded(requests, 32)
    H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), folder, requests, TOL)


@pytest.mark.parametrize("seed", [0, 1])
def test_portions(setup, seed):
    folder, model, requests = setup
    steps = H.steps_portions(requests, seed)
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) == 2
    H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), folder, requests, TOL)


@pytest.mark.parametrize("seed,page_size", [(0, 16), (1, 16), (2, 64)])
def test_mixed_with_page_reuse(setup, seed, page_size):
    folder, model, requests = setup
    n_prompt = {r: max(2, len(t) - 12) for r, t in requests.items()}
    steps = H.steps_mixed(requests, n_prompt, seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    eng = _engine(model, steps, page_size)
    total = sum(H._round64(len(t)) for t in requests.values())
    assert eng.n_pages * page_size < total, "the pool must be too small to hold all requests at once"
    res = H.run_steps(eng, steps)
    H.compare_with_plain(res, folder, requests, TOL)
    assert eng.cache.free_pages() == [eng.n_pages] * len(eng.cache.pools)


def test_window_pages_are_given_back(setup):
    folder, model, requests = setup
    eng = Engine(model, cache_tokens=128, page_size=16, max_requests=2)
    chunk = model.config.attention_chunk_size
    toks = requests["a"]
    eng.step([("x", toks[:chunk * 2 + 3], [])])
    kinds = [k.window.kind for k in eng.cache.groups]
    g_chunk, g_full = kinds.index("chunk"), kinds.index("full")
    held = lambda g: sum(p >= 0 for p in eng.cache.block_table("x", g))
    assert held(g_full) == -(-(chunk * 2 + 3) // 16)
    first_live = (chunk * 2) // 16
    assert held(g_chunk) == -(-(chunk * 2 + 3) // 16) - first_live
    eng.finish("x")
    eng.cache.check_invariants()


def test_step_is_all_or_nothing(setup):
    folder, model, requests = setup
    eng = Engine(model, cache_tokens=64, page_size=16, max_requests=4)
    eng.step([("x", requests["a"][:40], [])])
    before = (eng.cache.free_pages(), eng.cached_tokens("x"))
    with pytest.raises(OutOfPages):
        eng.step([("x", requests["a"][40:48], []), ("y", requests["b"][:30], [])])
    assert (eng.cache.free_pages(), eng.cached_tokens("x")) == before
    assert not eng.is_live("y")
    eng.cache.check_invariants()
    out = eng.step([("x", requests["a"][40:48], [7])])
    ref = H.plain_logits(folder, requests["a"][:48])[47]
    assert float((out[0] - ref).abs().max()) <= TOL * float(ref.abs().max()) * 10


def test_trace_replay_writes_logits(setup, tmp_path):
    folder, model, requests = setup
    reqs = {k: requests[k] for k in ("b", "c")}
    steps = H.steps_mixed(reqs, {r: len(t) - 5 for r, t in reqs.items()}, seed=3)
    steps[1]["entries"][0]["want"] = []          # a step part of which wants nothing
    eng = _engine(model, steps, 16)
    log = io.StringIO()
    replay(eng, [json.dumps(s) for s in steps], tmp_path, log=log)
    assert log.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    vocab = model.plan.vocab_size
    pos = {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        f = tmp_path / f"{s['step']}.f32"
        if not n_want:
            assert not f.exists()
            continue
        data = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(n_want, vocab))
        row = 0
        for e in s["entries"]:
            ref = H.plain_logits(folder, reqs[e["id"]])
            for w in e["want"]:
                p = pos.get(e["id"], 0) + w
                assert float((data[row] - ref[p]).abs().max()) <= TOL * float(ref.abs().max())
                row += 1
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
