"""The scheduler's own schedules with the CUDA kernels below it (tests/test_scheduler.py runs the same
decisions on the CPU stand-in): sampling with a temperature from a fixed seed in mixed batches, preemption
and recomputation when pages run out, and a batch that drains request by request through more decode
shapes than the engine keeps CUDA graphs for.

Counterparts: the scheduler's contract in crates/spite-scheduler/src/lib.rs:8-13,126-152, the sampler's
order of operations and generator in crates/spite-sampling/src/lib.rs:273-296,343-348."""
import random

import pytest
import torch

import helpers as H
import plain_llama4 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from spite_b200.engine import Model
    out = {}
    for name in ("A", "B"):
        path = H.write_model(tmp_path_factory.mktemp(f"sched{name}"), name)
        out[name] = (path, Model.from_folder(path, dtype="float32", device=DEV))
    return out


def plain_sampled(path, prompt, n, *, temperature, seed, top_p=0.95, repetition_penalty=1.1):
    """What `spite run --temperature T` would produce: the plain forward pass and the plain sampler."""
    cfg, W = H._folder_contents(str(path))
    ids, state, out = list(prompt), seed & ((1 << 64) - 1), []
    for _ in range(n):
        logits = plain.forward(cfg, W, ids)[-1]
        tok, state = plain.sample_plain(logits, ids, temperature=temperature, top_p=top_p,
                                        repetition_penalty=repetition_penalty, repeat_last_n=64, state=state)
        ids.append(tok)
        out.append(tok)
    return out


def scheduler(model, *, cache_tokens=512, page_size=16, max_requests=4, cuda_graphs=None, max_graphs=32, **kw):
    from spite_b200.engine import Engine
    from spite_b200.engine.scheduler import Scheduler
    from spite_b200.sampling import Sampler
    eng = Engine(model, cache_tokens=cache_tokens, page_size=page_size, max_requests=max_requests,
                 cuda_graphs=cuda_graphs, max_graphs=max_graphs)
    return Scheduler(eng, Sampler(model.kernels), **kw)


def test_three_requests_in_portions_of_eight_sampled_at_temperature(models):
    """Prompts of 37, 5 and 20 tokens, a budget of 8 tokens a step (portions of prompts beside decoded tokens),
    temperature 0.7 with the `run` command's sampler settings, a fixed seed per request: the tokens are the
    plain implementation's, and they are the same for other budgets and arrival orders."""
    from spite_b200.engine.scheduler import FinishReason, Request
    from spite_b200.sampling.sampler import run_sampling_params
    path, model = models["B"]
    prompts = [H.random_tokens(1000, n, 40 + i) for i, n in enumerate((37, 5, 20))]
    seeds = [0x1234_5678_9ABC_DEF0, 17, 2 ** 63 + 5]
    want = [plain_sampled(path, p, 10, temperature=0.7, seed=s) for p, s in zip(prompts, seeds)]
    assert len({tuple(w) for w in want}) == 3

    def run(budget, order):
        s = scheduler(model, max_batch_tokens=budget, max_requests=3)
        for i in order:
            s.submit(Request(i, prompts[i], run_sampling_params(0.7, seed=seeds[i], max_tokens=10)))
        mixed = 0
        while s.active_count():
            n_before = s.counters["steps"]
            s.step()
            s.engine.cache.check_invariants()
        assert all(r.finish_reason is FinishReason.MAX_TOKENS for r in s.finished.values())
        assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2
        return [s.finished[i].output for i in range(3)], s.counters
    got, counters = run(8, (0, 1, 2))
    assert got == want
    assert counters["steps"] >= (37 + 5 + 20) // 8                     # the prompts really came in portions
    for budget, order in ((24, (2, 0, 1)), (2048, (1, 2, 0)), (8, (2, 1, 0)), (3, (0, 2, 1))):
        assert run(budget, order)[0] == want, (budget, order)


def test_a_request_preempted_for_want_of_pages_is_recomputed_to_the_same_tokens(models):
    from spite_b200.engine.scheduler import Request
    from spite_b200.sampling import SamplingParams
    path, model = models["A"]
    cfg, W = H._folder_contents(str(path))
    a = H.random_tokens(512, 44, 0)
    c = H.random_tokens(512, 25, 2)

    def run(cache_tokens, **params):
        s = scheduler(model, cache_tokens=cache_tokens, max_batch_tokens=64)
        s.submit(Request("a", a, SamplingParams(max_tokens=12, seed=5, **params)))
        s.submit(Request("c", c, SamplingParams(max_tokens=12, seed=6, **params)))
        while s.active_count():
            s.step()
            s.engine.cache.check_invariants()
        assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2
        return s
    for params in (dict(temperature=0.0), dict(temperature=0.8, top_p=0.9, repetition_penalty=1.1)):
        tight, roomy = run(96, **params), run(1024, **params)
        assert tight.counters["preemptions"] >= 1 and roomy.counters["preemptions"] == 0
        assert tight.finished["c"].preemptions >= 1 and tight.finished["a"].preemptions == 0
        for r in ("a", "c"):
            assert tight.finished[r].output == roomy.finished[r].output, (r, params)
    assert roomy.finished["a"].output == plain_sampled(path, a, 12, temperature=0.8, seed=5, top_p=0.9)
    greedy = run(96, temperature=0.0)
    assert greedy.finished["c"].output == plain.generate_greedy(cfg, W, c, 12)


@pytest.mark.parametrize("n_requests,max_graphs", [(20, 4), (64, 32)])
def test_a_draining_batch_walks_through_more_shapes_than_graphs_are_kept(models, n_requests, max_graphs):
    """Requests that end after different numbers of tokens: the number of live requests falls one by one, so
    the decode step changes shape again and again while steps are launched ahead of the reading of their
    ids.  With few graphs kept (the least recently used goes) and with many, the tokens are those of the
    engine without CUDA graphs, and the number of captures stays small because request counts share rows."""
    from spite_b200.engine.scheduler import FinishReason, Request
    from spite_b200.sampling import SamplingParams
    path, model = models["A"]
    rng = random.Random(n_requests)
    prompts = [H.random_tokens(512, rng.randint(3, 14), 300 + i) for i in range(n_requests)]
    limits = list(range(3, 3 + n_requests))
    rng.shuffle(limits)

    def run(cuda_graphs):
        s = scheduler(model, cache_tokens=n_requests * 96, max_requests=n_requests, max_batch_tokens=4096,
                      cuda_graphs=cuda_graphs, max_graphs=max_graphs)
        for i in range(n_requests):
            s.submit(Request(i, prompts[i], SamplingParams(temperature=0.0, max_tokens=limits[i])))
        done = s.run_until_done()
        assert all(done[i].finish_reason is FinishReason.MAX_TOKENS and len(done[i].output) == limits[i]
                   for i in range(n_requests))
        assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2
        return s
    eager, graphs = run(False), run(True)
    for i in range(n_requests):
        assert graphs.finished[i].output == eager.finished[i].output, i
    eng = graphs.engine
    shapes = {eng.decode_rows(n) for n in range(1, n_requests + 1)}
    assert graphs.counters["steps_ahead"] > 0 and eng.graph_replays > 0
    assert len(eng._graphs) <= max_graphs
    if max_graphs >= len(shapes):
        assert eng.graph_captures <= len(shapes)                          # 64 -> 1 requests: 20 graphs, not 64
    else:
        assert eng.graph_captures > max_graphs                            # graphs were dropped and made again
    cfg, W = H._folder_contents(str(path))
    for i in (0, n_requests // 2):
        assert graphs.finished[i].output == plain.generate_greedy(cfg, W, prompts[i], limits[i])


def test_a_long_portion_beside_a_decoded_token_needs_little_scratch(tmp_path):
    """A step of one decoded token and a portion of 500: the split-key attention's partial results are kept
    for the decoded token's rows only, not for every token of the step."""
    from spite_b200.engine import Engine, Model
    path = H.write_model(tmp_path / "C", "C")
    model = Model.from_folder(path, dtype="bfloat16", device=DEV)
    eng = Engine(model, cache_tokens=2048, page_size=64, max_requests=2)
    short, long = H.random_tokens(300, 700, 1), H.random_tokens(300, 500, 2)
    eng.step([("s", short, [])])
    model.kernels.attention_scratch_bytes = 0
    eng.step([("s", [5], [0]), ("l", long, [499])])
    per_row = 6 * 64 * 4 + 6 * 2 * 4                                      # six heads of 64, maximum and sum
    assert 0 < model.kernels.attention_scratch_bytes <= 32 * 8 * per_row   # a few rows times the splits
