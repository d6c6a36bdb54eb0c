"""The engine on the GPU, in float32 and in bfloat16, against the plain
implementation: each request alone and whole; most of it in one step and the last
32 tokens one by one; portions of changing size down to two tokens; mixed batches
of up to four live requests with so few pages that they are used again; long
decoding; the first tokens of a sequence; and `bin/trace_run` as a program."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# float32: sums in another order than the plain implementation's.  bfloat16: 8 bits of
# mantissa at some thirty rounding points between the embedding and the logits.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
MARGIN = {"A": 0.012, "B": 0.03}      # router logit margin that bfloat16 rounding cannot flip


@pytest.fixture(scope="module", params=["A", "B"])
def folder(request, tmp_path_factory):
    return H.write_model(tmp_path_factory.mktemp(f"model{request.param}"), request.param), request.param


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, folder):
    from spite_b200.engine import Model
    path, name = folder
    dtype = request.param
    model = Model.from_folder(path, dtype=dtype, device="cuda:0")
    vocab = model.plan.vocab_size
    lengths = {"a": 83, "b": 40, "c": 37, "d": 66, "e": 21}
    if dtype == "float32":
        requests = {r: H.random_tokens(vocab, n, i) for i, (r, n) in enumerate(lengths.items())}
    else:
        requests = {r: H.decisive_tokens(path, n, i, MARGIN[name]) for i, (r, n) in enumerate(lengths.items())}
    return path, model, requests, TOL[dtype]


def _engine(model, steps, page_size):
    from spite_b200.engine import Engine
    return Engine(model, cache_tokens=H.max_tokens_of(steps), page_size=page_size, max_requests=4)


@pytest.mark.parametrize("page_size", [16, 64])
def test_whole(setup, page_size):
    path, model, requests, tol = setup
    steps = H.steps_whole(requests)
    H.compare_with_plain(H.run_steps(_engine(model, steps, page_size), steps), path, requests, tol)


def test_last_32_tokens_one_by_one(setup):
    path, model, requests, tol = setup
    steps = H.steps_last_decoded(requests, 32)
    H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), path, requests, tol)


@pytest.mark.parametrize("seed", [0, 1])
def test_portions_down_to_two_tokens(setup, seed):
    path, model, requests, tol = setup
    steps = H.steps_portions(requests, seed)
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) == 2
    H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), path, requests, tol)


@pytest.mark.parametrize("seed,page_size", [(0, 16), (1, 16), (2, 64)])
def test_mixed_batches_reusing_pages(setup, seed, page_size):
    path, model, requests, tol = setup
    n_prompt = {r: max(2, len(t) - 12) for r, t in requests.items()}
    steps = H.steps_mixed(requests, n_prompt, seed)
    eng = _engine(model, steps, page_size)
    assert eng.n_pages * page_size < sum(H._round64(len(t)) for t in requests.values())
    H.compare_with_plain(H.run_steps(eng, steps), path, requests, tol)
    assert eng.cache.free_pages() == [eng.n_pages] * len(eng.cache.pools)


def poison_free_pages(engine):
    """Every page that no request holds gets NaN in every cache: what a request whose activations
    overflowed may leave behind when it ends."""
    for g, pool in enumerate(engine.cache.pools):
        if pool._free:
            engine.storage.kv[g][:, :, torch.tensor(pool._free, device=engine.storage.kv[g].device)] = float("nan")


def test_what_a_page_held_before_is_never_seen(setup):
    """Free pages are filled with NaN before every step, so every page a request receives (its first, the
    ones it grows into, the ones it gets again after its window let them go) arrives poisoned.  The logits
    stay those of the plain implementation: a masked key's zero weight never meets the old contents."""
    path, model, requests, tol = setup
    n_prompt = {r: max(2, len(t) - 12) for r, t in requests.items()}
    steps = H.steps_mixed(requests, n_prompt, 3)
    eng = _engine(model, steps, 16)
    results = H.run_steps(eng, steps, before_step=poison_free_pages)
    assert all(bool(torch.isfinite(v).all()) for v in results.values())
    H.compare_with_plain(results, path, requests, tol)


def test_first_tokens_of_a_sequence(setup):
    """Positions 0..3 alone: one key, the first rotation angles, a page's first rows."""
    path, model, requests, tol = setup
    toks = requests["a"][:4]
    steps = [{"step": i, "entries": [{"id": "s", "tokens": [t], "want": [0]}], "end": []}
             for i, t in enumerate(toks)]
    steps[-1]["end"] = ["s"]
    H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), path, {"s": toks}, tol)


def test_long_decoding(setup):
    """A short prompt, then 200 tokens one by one: several chunks and many pages pass."""
    path, model, requests, tol = setup
    vocab = model.plan.vocab_size
    if tol < 1e-3:
        toks = H.random_tokens(vocab, 216, 77)
    else:
        name = "A" if vocab == H.CONFIG_A["vocab_size"] else "B"
        toks = H.decisive_tokens(path, 216, 77, MARGIN[name])
    steps =[{"entries": [{"id": "l", "tokens": toks[:16], "want": list(range(16))}], "end": []}]
    steps += [{"entries": [{"id": "l", "tokens": [t], "want": [0]}], "end": []} for t in toks[16:]]
    steps[-1]["end"] = ["l"]
    for i, s in enumerate(steps):
        s["step"] = i
    H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), path, {"l": toks}, tol)


def test_sizes_of_the_tcgen05_kernels(tmp_path):
    """A third configuration whose head size, widths and prompt lengths reach the tcgen05 attention and
    product kernels (the two tiny ones stay below them): whole prompts, large portions beside small ones,
    and mixed batches with pages of 64 used again; a chunk edge inside a 64-key tile, a layer that sees all."""
    from spite_b200.engine import Model
    path = H.write_model(tmp_path / "modelC", "C")
    model = Model.from_folder(path, dtype="bfloat16", device="cuda:0")
    lengths = {"a": 300, "b": 130, "c": 97, "d": 64, "e": 45}
    requests = {r: H.decisive_tokens(path, n, 40 + i, 0.02) for i, (r, n) in enumerate(lengths.items())}
    steps = H.steps_whole(requests)
    H.compare_with_plain(H.run_steps(_engine(model, steps, 64), steps), path, requests, TOL["bfloat16"])
    assert model.kernels.attention_tc_error() == 0 and model.kernels.gemm_tc_error() == 0
    by_library = model.kernels.launches_by_library
    assert by_library["attention_tc"] > 0 and by_library["gemm_tc"] > 0, dict(by_library)
    steps = H.steps_portions(requests, 3, sizes=(2, 5, 43, 64, 90, 128))
    H.compare_with_plain(H.run_steps(_engine(model, steps, 64), steps), path, requests, TOL["bfloat16"])
    n_prompt = {r: len(t) - 8 for r, t in requests.items()}
    steps = H.steps_mixed(requests, n_prompt, 5, sizes=(2, 9, 50, 70))
    eng = _engine(model, steps, 64)
    assert eng.n_pages * 64 < sum(H._round64(len(t)) for t in requests.values())
    # free pages hold NaN before every step: the rows of a live page behind a request's last position,
    # inside the 64-key tile that the tensor cores multiply, must have been cleared when the page was handed out
    results = H.run_steps(eng, steps, before_step=poison_free_pages)
    assert all(bool(torch.isfinite(v).all()) for v in results.values())
    H.compare_with_plain(results, path, requests, TOL["bfloat16"])
    assert model.kernels.attention_tc_error() == 0 and model.kernels.gemm_tc_error() == 0
    assert all(by_library[lib] > 0 for lib in ("attention_tc", "attention_rows", "attention_decode", "gemm_stream"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_awkward_sizes(tmp_path, dtype):
    """Sizes that the fast kernels refuse (width 100, head size 24, seven heads on one kv head, vocabulary
    301): the general kernels take over, in both precisions, with the same answers."""
    from spite_b200.engine import Model
    path = H.write_model(tmp_path / "modelD", "D")
    model = Model.from_folder(path, dtype=dtype, device="cuda:0")
    lengths = {"a": 70, "b": 33}
    if dtype == "float32":
        requests = {r: H.random_tokens(301, n, 60 + i) for i, (r, n) in enumerate(lengths.items())}
    else:
        requests = {r: H.decisive_tokens(path, n, 60 + i, 0.03) for i, (r, n) in enumerate(lengths.items())}
    for steps in (H.steps_whole(requests), H.steps_last_decoded(requests, 20), H.steps_portions(requests, 1)):
        H.compare_with_plain(H.run_steps(_engine(model, steps, 16), steps), path, requests, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folder, dtype, tmp_path):
    """`bin/trace_run` as a user runs it: JSON lines in, `done <step>` lines and .f32 files out."""
    path, name = folder
    cfg = json.loads((Path(path) / "config.json").read_text())
    vocab = cfg["vocab_size"]
    if dtype == "float32":
        reqs = {"p": H.random_tokens(vocab, 45, 5), "q": H.random_tokens(vocab, 30, 6)}
    else:
        reqs = {"p": H.decisive_tokens(path, 45, 5, MARGIN[name]), "q": H.decisive_tokens(path, 30, 6, MARGIN[name])}
    steps = H.steps_mixed(reqs, {"p": 40, "q": 20}, seed=4)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(path), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(H.max_tokens_of(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    pos, results = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in s["entries"]:
            for w in e["want"]:
                results[(e["id"], pos.get(e["id"], 0) + w)] = torch.from_numpy(data[row].copy())
                row += 1
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
    H.compare_with_plain(results, path, reqs, TOL[dtype])


def test_trace_run_step_by_step(folder, tmp_path):
    """`bin/trace_run` driven as a caller that waits for every `done`: a request with an integer id, steps in
    which nothing is wanted, a request that sits a step out, a step that only ends a request, the end of an
    unknown request, wanted places out of order, step numbers with gaps."""
    path, name = folder
    vocab = json.loads((Path(path) / "config.json").read_text())["vocab_size"]
    a, b, c = H.random_tokens(vocab, 70, 1), H.random_tokens(vocab, 40, 2), H.random_tokens(vocab, 9, 3)
    steps = [
        {"step": 0, "entries": [{"id": 1, "tokens": a[:33], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": 1, "tokens": a[33:35], "want": [1]},
                                {"id": "b", "tokens": b[:2], "want": [0, 1]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:40], "want": [37]}], "end": []},
        {"step": 3, "entries": [], "end": ["b"]},
        {"step": 4, "entries": [{"id": 1, "tokens": a[35:36], "want": [0]},
                                {"id": "c", "tokens": c, "want": [8, 0]}], "end": ["c", "nobody"]},
        {"step": 7, "entries": [{"id": 1, "tokens": a[36:70], "want": [33]}], "end": [1]},
    ]
    out = tmp_path / "out"
    proc = subprocess.Popen(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(path), "--dtype", "float32",
         "--out", str(out), "--max-tokens", "192"],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    assert sorted(p.name for p in out.iterdir()) == ["1.f32", "2.f32", "4.f32", "7.f32"]
    refs = {"a": H.plain_logits(path, a), "b": H.plain_logits(path, b), "c": H.plain_logits(path, c)}
    wanted = {1: [("a", 34), ("b", 0), ("b", 1)], 2: [("b", 39)], 4: [("a", 35), ("c", 8), ("c", 0)], 7: [("a", 69)]}
    for step, rows in wanted.items():
        data = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab)
        for i, (r, p) in enumerate(rows):
            err = float((torch.from_numpy(data[i].copy()) - refs[r][p]).abs().max()) / float(refs[r].abs().max())
            assert err <= TOL["float32"], f"step {step}, row {i}: error {err:.3e}"
