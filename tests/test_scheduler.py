"""The scheduler's decisions: admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out.  The step function
below it is the product's, with the kernels replaced by their plain torch
restatements so that the test runs without a GPU."""
import pytest
import torch

import helpers as H
import plain_llama4 as plain
from reference_kernels import TorchReferenceKernels
from spite_b200.engine import ContextOverflow, Engine, Model
from spite_b200.engine.scheduler import FinishReason, Request, RequestState, Scheduler
from spite_b200.sampling import Sampler, SamplingParams


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    folder = H.write_model(tmp_path_factory.mktemp("modelA"), "A")
    m = Model.from_folder(folder, dtype="float32", device="cpu", kernels=TorchReferenceKernels())
    m.folder = folder
    return m


def make(model, *, cache_tokens=512, page_size=16, max_requests=4, **kw):
    eng = Engine(model, cache_tokens=cache_tokens, page_size=page_size, max_requests=max_requests)
    return Scheduler(eng, Sampler(model.kernels), **kw)


def greedy(n=8, **kw):
    return SamplingParams(temperature=0.0, max_tokens=n, **kw)


def plain_greedy(model, prompt, n):
    cfg, tensors = H._folder_contents(str(model.folder))
    return plain.generate_greedy(cfg, tensors, prompt, n)


PROMPTS = [H.random_tokens(512, n, s) for s, n in enumerate((48, 5, 20, 33))]


def test_portions_follow_the_token_budget_and_decodes_come_first(model):
    s = make(model, max_batch_tokens=16)
    s.submit(Request("a", PROMPTS[0], greedy(4)))
    s.submit(Request("b", PROMPTS[1], greedy(4)))
    plan = s.plan_step()
    assert [(r.id, len(t), w) for r, t, w in plan.entries] == [("a", 16, False)]
    s = make(model, max_batch_tokens=16)
    s.submit(Request("a", PROMPTS[0], greedy(4)))
    s.submit(Request("b", PROMPTS[1], greedy(4)))
    sizes = []
    for _ in range(6):
        plan_sizes = None
        outs = s.step()
        sizes.append(s.counters["tokens"])
    # 48-token prompt in portions of 16; the 5-token prompt joins the step in which budget is left
    assert sizes[:3] == [16, 32, 48]
    assert s.finished == {} or all(r.state is RequestState.DONE for r in s.finished.values())
    s.run_until_done()
    assert s.finished["a"].output == plain_greedy(model, PROMPTS[0], 4)
    assert s.finished["b"].output == plain_greedy(model, PROMPTS[1], 4)
    assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2 and s.engine.cache.slots.n_free == 4


def test_mixed_step_has_decodes_beside_a_portion(model):
    s = make(model, max_batch_tokens=12)
    s.submit(Request("b", PROMPTS[1], greedy(6)))
    s.step()                                              # b's whole prompt, first token sampled
    s.submit(Request("a", PROMPTS[0], greedy(2)))
    plan = s.plan_step()
    assert [(r.id, len(t), w) for r, t, w in plan.entries] == [("b", 1, True), ("a", 11, False)]


@pytest.mark.parametrize("budget,pages,order", [(2048, 512, (0, 1, 2, 3)), (7, 512, (3, 2, 1, 0)),
                                                (24, 160, (1, 3, 0, 2)), (2, 128, (0, 1, 2, 3))])
def test_outputs_do_not_depend_on_budget_pool_or_arrival(model, budget, pages, order):
    s = make(model, max_batch_tokens=budget, cache_tokens=pages, max_requests=3)
    for i in order:
        s.submit(Request(i, PROMPTS[i], greedy(6)))
    done = s.run_until_done()
    for i in order:
        assert done[i].output == plain_greedy(model, PROMPTS[i], 6), i
        assert done[i].finish_reason is FinishReason.MAX_TOKENS
    s.engine.cache.check_invariants()
    assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2


def test_running_out_of_pages_preempts_the_latest_admitted(model):
    # 6 pages of 16: a (48 tokens) takes 3... both decode until a page is missing
    s = make(model, max_batch_tokens=64, cache_tokens=96, page_size=16)
    s.submit(Request("a", PROMPTS[0][:44], greedy(12)))
    s.submit(Request("c", PROMPTS[2] + PROMPTS[1], greedy(12)))     # 25 tokens
    preempted = []
    while s.active_count():
        before = s.counters["preemptions"]
        s.step()
        if s.counters["preemptions"] > before:
            preempted.append([r.id for r in s.waiting])
        s.engine.cache.check_invariants()
    assert s.counters["preemptions"] >= 1
    assert preempted[0] == ["c"]                                    # the most recently admitted one
    assert s.finished["c"].preemptions >= 1 and s.finished["a"].preemptions == 0
    assert s.finished["a"].output == plain_greedy(model, PROMPTS[0][:44], 12)
    assert s.finished["c"].output == plain_greedy(model, PROMPTS[2] + PROMPTS[1], 12)
    assert s.engine.cache.free_pages() == [6, 6]


def test_a_lone_request_that_fills_the_cache_ends(model):
    s = make(model, cache_tokens=32, page_size=16)
    s.submit(Request("a", PROMPTS[2], greedy(40)))                   # 20 tokens, room for 32
    done = s.run_until_done()
    r = done["a"]
    assert r.finish_reason is FinishReason.CACHE_FULL
    assert len(PROMPTS[2]) + len(r.output) == 33                     # 32 cached + the token not yet fed
    assert r.output == plain_greedy(model, PROMPTS[2], len(r.output))
    assert s.engine.cache.free_pages() == [2, 2]
    with pytest.raises(ContextOverflow):
        s.submit(Request("big", PROMPTS[0], greedy(1)))              # 48 tokens can never fit 2 pages


def test_finish_reasons(model):
    ref = plain_greedy(model, PROMPTS[1], 6)
    s = make(model, eos_token_ids=[ref[3]])
    s.submit(Request("e", PROMPTS[1], greedy(6)))
    s.submit(Request("s", PROMPTS[1], greedy(6, stop_token_ids=(ref[2],))))
    s.submit(Request("z", PROMPTS[1], greedy(0)))
    outs = []
    while s.active_count():
        outs += s.step()
    first = ref.index(ref[3])
    assert s.finished["e"].output == ref[:first] and s.finished["e"].finish_reason is FinishReason.EOS_TOKEN
    assert s.finished["s"].finish_reason in (FinishReason.STOP_TOKEN, FinishReason.EOS_TOKEN)
    assert s.finished["s"].output == ref[:min(ref.index(ref[2]), first)]
    assert s.finished["z"].output == [] and s.finished["z"].finish_reason is FinishReason.MAX_TOKENS
    ended = [o for o in outs if o.done and o.request_id == "e"]
    assert len(ended) == 1 and ended[0].token is None                # the end token is not emitted
    s = make(model, ctx=8)
    s.submit(Request("c", PROMPTS[1], greedy(50)))
    s.run_until_done()
    assert s.finished["c"].finish_reason is FinishReason.CONTEXT_FULL and len(s.finished["c"].output) == 3
    with pytest.raises(ContextOverflow):
        s.submit(Request("x", PROMPTS[0], greedy(1)))
    with pytest.raises(ValueError):
        s.submit(Request("y", [], greedy(1)))


def test_sampling_is_reproducible_and_independent_of_batching(model):
    def run(ids, budget):
        s = make(model, max_batch_tokens=budget)
        for i in ids:
            s.submit(Request(i, PROMPTS[i], SamplingParams(temperature=0.7, top_p=0.9, repetition_penalty=1.1,
                                                          seed=100 + i, max_tokens=8)))
        return {i: r.output for i, r in s.run_until_done().items()}
    together = run([0, 1, 2], 2048)
    assert together == run([0, 1, 2], 2048)
    assert together == run([2, 1, 0], 9)
    assert run([1], 2048)[1] == together[1]
    assert len({tuple(v) for v in together.values()}) == 3
    # the plain sampler with the same per-request state gives the same tokens
    cfg, tensors = H._folder_contents(str(model.folder))
    ids, state, out = list(PROMPTS[1]), 101, []
    for _ in range(8):
        logits = plain.forward(cfg, tensors, ids)[-1]
        tok, state = plain.sample_plain(logits, ids, temperature=0.7, top_p=0.9, repetition_penalty=1.1,
                                        repeat_last_n=64, state=state)
        ids.append(tok)
        out.append(tok)
    assert out == together[1]


def test_no_slot_means_waiting_not_failing(model):
    s = make(model, max_requests=1)
    for i in (1, 2):
        s.submit(Request(i, PROMPTS[i], greedy(3)))
    s.step()
    assert [r.id for r in s.running] == [1] and [r.id for r in s.waiting] == [2]
    done = s.run_until_done()
    assert done[2].output == plain_greedy(model, PROMPTS[2], 3)


@pytest.mark.parametrize("budget,pages,slots", [(2048, 512, 4), (24, 160, 3), (64, 96, 4), (7, 512, 2)])
def test_decoding_ahead_produces_the_same_tokens(model, budget, pages, slots):
    """With the sampled ids read one step late (decode steps launched from the ids on the device), every
    request ends with the same tokens and reason as with the plain loop: ends by count, by an
    end-of-generation and a stop token (which cost one discarded step), preemption when pages run out,
    and requests that wait for a slot."""
    ref = plain_greedy(model, PROMPTS[1], 12)

    def run(ahead):
        s = make(model, max_batch_tokens=budget, cache_tokens=pages, max_requests=slots,
                 eos_token_ids=[ref[7]], decode_ahead=ahead)
        s.submit(Request(0, PROMPTS[0][:40], greedy(14)))
        s.submit(Request(1, PROMPTS[1], greedy(12)))                               # ends on the eos token
        s.submit(Request(2, PROMPTS[2], greedy(9, stop_token_ids=(ref[4],))))
        s.submit(Request(3, PROMPTS[1], greedy(5)))
        s.submit(Request(4, PROMPTS[3], greedy(3)))
        outs = []
        while s.active_count():
            outs += s.step()
            s.engine.cache.check_invariants()
        assert s._in_flight is None
        assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2
        emitted = {i: [o.token for o in outs if o.request_id == i and o.token is not None] for i in range(5)}
        return s, emitted

    plain_run, plain_emitted = run(False)
    ahead_run, ahead_emitted = run(True)
    assert plain_run.counters["steps_ahead"] == 0 and ahead_run.counters["steps_ahead"] > 0
    for i in range(5):
        assert ahead_run.finished[i].output == plain_run.finished[i].output, i
        assert ahead_run.finished[i].finish_reason is plain_run.finished[i].finish_reason, i
        assert ahead_emitted[i] == plain_emitted[i] == plain_run.finished[i].output, i
    assert plain_run.finished[1].finish_reason is FinishReason.EOS_TOKEN


@pytest.mark.parametrize("seed", range(16))
def test_decoding_ahead_random_scenarios(model, seed):
    """Random prompts, limits, stop tokens, budgets and pool sizes: reading the ids one step late never
    changes what a request produces or why it ends, and every page comes back."""
    import random
    rng = random.Random(seed)
    n_req = rng.randint(2, 6)
    prompts = [H.random_tokens(512, rng.randint(2, 40), 100 * seed + i) for i in range(n_req)]
    limits = [rng.randint(1, 14) for _ in range(n_req)]
    probe = plain_greedy(model, prompts[0], limits[0])
    eos = [probe[rng.randrange(len(probe))]] if rng.random() < 0.7 else []
    stops = [tuple(rng.sample(range(512), 3)) if rng.random() < 0.5 else () for _ in range(n_req)]
    budget, slots = rng.choice([3, 16, 64, 2048]), rng.randint(1, 4)
    pages = rng.choice([96, 160, 512])

    # every other scenario samples: a temperature, filters, a repetition penalty over the last few tokens (which
    # has to find the token that the host has not read yet), one generator state per request; some rows greedy
    from spite_b200.sampling import SamplingParams
    def params(i):
        if seed % 2 == 0 or rng_of[i] < 0.25:
            return greedy(limits[i], stop_token_ids=stops[i])
        return SamplingParams(temperature=0.5 + rng_of[i], top_p=0.9, top_k=40 if i % 2 else 0, min_p=0.0,
                              repetition_penalty=1.0 if i % 3 == 0 else 1.3, repeat_last_n=4 + i, seed=1000 + 17 * i,
                              max_tokens=limits[i], stop_token_ids=stops[i])
    rng_of = [rng.random() for _ in range(n_req)]

    def run(ahead):
        s = make(model, max_batch_tokens=budget, cache_tokens=pages, max_requests=slots, eos_token_ids=eos,
                 decode_ahead=ahead)
        for i in range(n_req):
            s.submit(Request(i, prompts[i], params(i)))
        s.run_until_done(max_steps=2000)
        assert not s.active_count() and s._in_flight is None
        s.engine.cache.check_invariants()
        assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2
        return s

    a, b = run(False), run(True)
    for i in range(n_req):
        assert b.finished[i].output == a.finished[i].output, (seed, i)
        assert b.finished[i].finish_reason is a.finished[i].finish_reason, (seed, i)
    if any(limits[i] > 2 for i in range(n_req)):
        assert b.counters["steps_ahead"] > 0 or pages == 96 or budget == 3, seed


def test_two_prompts_in_a_tight_pool_do_not_block_each_other(model):
    """Two 120-token prompts that each fit a pool of 160 tokens alone, portions of 32 under a budget of 64:
    whatever is admitted, every step runs something and both requests end with the right tokens."""
    a, b = H.random_tokens(512, 120, 70), H.random_tokens(512, 120, 71)
    s = make(model, cache_tokens=160, page_size=16, max_batch_tokens=64, max_portion=32)
    s.submit(Request("a", a, greedy(4)))
    s.submit(Request("b", b, greedy(4)))
    while s.active_count():
        before = s.counters["steps"]
        s.step()
        assert s.counters["steps"] == before + 1
        s.engine.cache.check_invariants()
    assert s.finished["a"].output == plain_greedy(model, a, 4)
    assert s.finished["b"].output == plain_greedy(model, b, 4)
    assert all(r.finish_reason is FinishReason.MAX_TOKENS for r in s.finished.values())
    assert s.counters["preemptions"] == 0                 # b waited for a instead of taking its pages
    assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2


def test_prompts_in_progress_give_way_when_none_can_go_on(model):
    """The state that greedy admission could reach: two requests in the middle of their prompts hold all the
    pages between them.  The later one is preempted, the earlier one goes on."""
    a, b = H.random_tokens(512, 120, 70), H.random_tokens(512, 120, 71)
    s = make(model, cache_tokens=160, page_size=16, max_batch_tokens=64, max_portion=32)
    s.submit(Request("a", a, greedy(3)))
    s.submit(Request("b", b, greedy(3)))
    ra, rb = s.waiting.popleft(), s.waiting.popleft()
    for r, n in ((ra, 96), (rb, 64)):                       # 6 + 4 pages of 10: nothing is free
        s.engine.step([(r.id, r.prompt[:n], [])])
        r.n_fed, r.state = n, RequestState.PREFILLING
        s.running.append(r)
    assert s.engine.cache.free_pages() == [10, 0]           # (chunked, full): the chunked group let the passed chunks go
    s.step()
    assert [r.id for r in s.waiting] == ["b"] and rb.preemptions == 1 and rb.n_fed == 0
    assert ra.n_fed == 120 and len(ra.output) == 1          # a ran the rest of its prompt in that step
    done = s.run_until_done()
    assert done["a"].output == plain_greedy(model, a, 3) and done["b"].output == plain_greedy(model, b, 3)
    assert done["b"].preemptions == 1
    assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2


@pytest.mark.parametrize("seed", range(12))
def test_random_pools_and_budgets_always_make_progress(model, seed):
    """Random prompts, portions, budgets and pools down to the size of the longest request: every step runs
    something, nobody ends for want of pages that the pool has, the tokens are the plain implementation's."""
    import random
    rng = random.Random(1000 + seed)
    n_req = rng.randint(2, 5)
    prompts = [H.random_tokens(512, rng.randint(2, 90), 50 * seed + i) for i in range(n_req)]
    limits = [rng.randint(1, 6) for _ in range(n_req)]
    longest = max(len(p) + n for p, n in zip(prompts, limits))
    pages = -(-longest // 16) * 16 + 16 * rng.choice([0, 0, 1, 3, 8])
    budget = rng.choice([2, 5, 16, 40, 64, 2048])
    portion = rng.choice([None, 3, 16, 32])
    s = make(model, cache_tokens=pages, page_size=16, max_batch_tokens=budget, max_portion=portion,
             max_requests=rng.randint(2, 4))
    for i in range(n_req):
        s.submit(Request(i, prompts[i], greedy(limits[i])))
    steps = 0
    while s.active_count():
        before = (s.counters["steps"], len(s.finished))
        s.step()
        assert (s.counters["steps"], len(s.finished)) != before
        s.engine.cache.check_invariants()
        steps += 1
        assert steps < 3000
    for i in range(n_req):
        assert s.finished[i].finish_reason is FinishReason.MAX_TOKENS, (seed, i)
        assert s.finished[i].output == plain_greedy(model, prompts[i], limits[i]), (seed, i)
    assert s.engine.cache.free_pages() == [s.engine.n_pages] * 2


def test_a_kernel_that_gave_up_waiting_stops_the_step_and_nothing_is_lost(model):
    """The kernel set reports that a kernel gave up a bounded wait (here: a stand-in that says so once).
    The scheduler raises the typed error at the point where it has the ids, keeps none of them, sends the
    running requests back to the queue with their pages freed, and the next calls produce the right tokens."""
    from spite_b200.engine import KernelTimeout

    class GivesUpOnce(TorchReferenceKernels):
        pending = {}

        def errors(self):
            out, self.pending = self.pending, {}
            return out

    kernels = GivesUpOnce()
    m = Model.from_folder(model.folder, dtype="float32", device="cpu", kernels=kernels)
    for ahead in (False, True):
        eng = Engine(m, cache_tokens=512, page_size=16, max_requests=4)
        s = Scheduler(eng, Sampler(kernels), max_batch_tokens=64, decode_ahead=ahead)
        for i in (1, 2):
            s.submit(Request(i, PROMPTS[i], greedy(6)))
        s.step(); s.step(); s.step()
        before = {i: list(r.output) for i, r in ((r.id, r) for r in s.running)}
        kernels.pending = {"gemm_tc": 2}
        with pytest.raises(KernelTimeout, match="gemm_tc .code 2."):
            while True:
                s.step()
        assert not s.running and [r.id for r in s.waiting] == [1, 2] and s._in_flight is None
        assert {r.id: r.output for r in s.waiting} == before             # nothing of the bad step was kept
        assert eng.cache.free_pages() == [eng.n_pages] * 2 and eng.cache.slots.n_free == 4
        done = s.run_until_done()
        for i in (1, 2):
            assert done[i].output == plain_greedy(model, PROMPTS[i], 6) and done[i].preemptions == 1
    # sampled requests: the draw of a token that was in flight is lost with it, so that what follows is what an
    # undisturbed run samples
    from spite_b200.sampling import SamplingParams
    sampled = lambda i: SamplingParams(temperature=0.9, top_p=0.9, repetition_penalty=1.2, seed=40 + i, max_tokens=7)
    eng = Engine(m, cache_tokens=512, page_size=16, max_requests=4)
    calm = Scheduler(eng, Sampler(kernels), max_batch_tokens=64, decode_ahead=True)
    for i in (1, 2):
        calm.submit(Request(i, PROMPTS[i], sampled(i)))
    want = {i: r.output for i, r in calm.run_until_done().items()}
    eng = Engine(m, cache_tokens=512, page_size=16, max_requests=4)
    s = Scheduler(eng, Sampler(kernels), max_batch_tokens=64, decode_ahead=True)
    for i in (1, 2):
        s.submit(Request(i, PROMPTS[i], sampled(i)))
    s.step(); s.step(); s.step(); s.step()
    kernels.pending = {"gemm_stream": 1}
    with pytest.raises(KernelTimeout):
        while True:
            s.step()
    assert {i: r.output for i, r in s.run_until_done().items()} == want
