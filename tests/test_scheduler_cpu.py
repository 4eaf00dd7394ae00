"""The scheduler's decisions, on the CPU with the kernels' plain PyTorch statements as ops:
admission under a token budget, portions, mixed batches, finishing and freeing, and what happens
when pages run out (retraction; refusal of what can never fit)."""

import tempfile

import pytest
import torch

import plain_impl
import tiny_models
from harness import make_runner, model_dir
from lily_b200.engine.scheduler import Scheduler
from lily_b200.sampling.params import SamplingParams
from lily_b200.sampling.sampler import uniform_for


@pytest.fixture(scope="module")
def setup():
    cfg = tiny_models.TINY_QWEN3
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 51, tmp)
        yield cfg, weights, path


def scheduler(path, max_tokens=1024, page_size=16, max_requests=8, **kw):
    runner = make_runner(path, max_tokens=max_tokens, page_size=page_size, max_requests=max_requests)
    return Scheduler(runner, random_seed=7, **kw)


def run(s, prompts, n, **params):
    for i, p in enumerate(prompts):
        s.add_request(f"r{i}", p, SamplingParams(max_new_tokens=n, ignore_eos=True, **params))
    s.run_to_completion()
    return [s.results[f"r{i}"].output_ids for i in range(len(prompts))]


def prompts(cfg, lens, seed=0):
    return [tiny_models.random_tokens(n, cfg["vocab_size"], seed + i) for i, n in enumerate(lens)]


def test_greedy_equals_plain_and_batching_changes_nothing(setup):
    cfg, weights, path = setup
    ps = prompts(cfg, [1, 7, 33, 64])
    want = [plain_impl.greedy_generate(cfg, weights, p, 16) for p in ps]
    single = []
    for p in ps:
        single += run(scheduler(path, max_requests=1), [p], 16)
    assert single == want
    s = scheduler(path)
    assert run(s, ps, 16) == want
    assert s.runner.cache.held_pages() == [0] and s.runner.cache.slots.available == 8
    assert s.prefill_tokens_computed == sum(len(p) for p in ps) and s.decode_steps == 4 * 15


def test_chunked_prefill_equals_unchunked(setup):
    cfg, weights, path = setup
    long = prompts(cfg, [150], seed=5)
    chunked = scheduler(path, chunked_prefill_size=64)
    seen = []
    orig = chunked.runner.step
    chunked.runner.step = lambda entries: (seen.append([len(e.tokens) for e in entries]), orig(entries))[1]
    assert run(chunked, long, 8) == run(scheduler(path), long, 8)
    assert chunked.prefill_tokens_computed == 150
    assert seen[:3] == [[64], [64], [22]]


def test_last_portion_fits_the_page_already_held(setup):
    """All pages are held after two portions; the rest of the prompt still fits the last of them
    and must be taken, not refused."""
    cfg, weights, path = setup
    p = prompts(cfg, [94], seed=9)
    whole = scheduler(path, max_tokens=96)
    want = run(whole, p, 2)
    assert whole.results["r0"].finish_reason == {"type": "length"} and len(want[0]) == 2
    chunked = scheduler(path, max_tokens=96, chunked_prefill_size=45)
    taken = []
    chunked.add_request("r0", p[0], SamplingParams(max_new_tokens=2, ignore_eos=True))
    while chunked.has_work():
        assert chunked.step()
        if chunked.last_batch.get("prefill_tokens"):
            taken.append(chunked.last_batch["prefill_tokens"])
            chunked.last_batch = {}
    assert taken == [45, 45, 4]
    assert chunked.results["r0"].output_ids == want[0] == plain_impl.greedy_generate(cfg, weights, p[0], 2)
    assert chunked.runner.cache.held_pages() == [0]


def test_budget_portions_and_mixed_batches(setup):
    cfg, weights, path = setup
    s = scheduler(path, chunked_prefill_size=40, max_running_requests=3)
    ps = prompts(cfg, [30, 30, 30, 10], seed=9)
    for i, p in enumerate(ps):
        s.add_request(f"r{i}", p, SamplingParams(max_new_tokens=4, ignore_eos=True))
    s.step()                        # 30 of r0 and 10 of r1: the budget of 40 is spent
    assert s.last_batch == {"decode": 0, "prefill_requests": 2, "prefill_tokens": 40}
    assert [r.rid for r in s.running] == ["r0"] and s.waiting_queue[0].rid == "r1" and s.waiting_queue[0].seq_len == 10
    s.step()                        # r0 decodes beside the rest of r1 and a portion of r2 (3 requests at most)
    assert s.last_batch == {"decode": 1, "prefill_requests": 2, "prefill_tokens": 40}
    assert [r.rid for r in s.running] == ["r0", "r1"] and s.waiting_queue[0].rid == "r2"
    s.step()                        # no slot for r3 while three requests are live
    assert s.last_batch == {"decode": 2, "prefill_requests": 1, "prefill_tokens": 10}
    s.run_to_completion()
    want = [plain_impl.greedy_generate(cfg, weights, p, 4) for p in ps]
    assert [s.results[f"r{i}"].output_ids for i in range(4)] == want
    assert all(s.results[f"r{i}"].finish_reason == {"type": "length"} for i in range(4))


def test_pages_run_out_retraction_keeps_outputs(setup):
    cfg, weights, path = setup
    ps = prompts(cfg, [20, 25, 18, 30, 22, 27, 19, 24], seed=20)
    want = [plain_impl.greedy_generate(cfg, weights, p, 12) for p in ps]
    s = scheduler(path, max_tokens=13 * 16, page_size=16)          # 13 pages for 8 requests of up to 42 tokens
    assert run(s, ps, 12) == want
    assert s.retractions > 0
    assert s.runner.cache.held_pages() == [0] and s.runner.cache.slots.available == 8


def test_what_can_never_fit_is_refused_and_a_lone_request_ends(setup):
    cfg, weights, path = setup
    s = scheduler(path, max_tokens=4 * 16, page_size=16)
    s.add_request("big", tiny_models.random_tokens(70, 256, 1), SamplingParams(max_new_tokens=4))
    assert s.results["big"].finish_reason["type"] == "abort" and "KV pool" in s.results["big"].finish_reason["message"]
    s.add_request("ctx", tiny_models.random_tokens(256, 256, 1), SamplingParams(max_new_tokens=4))
    assert "context" in s.results["ctx"].finish_reason["message"]
    s.add_request("bad", [5, 999], None)
    assert "vocabulary" in s.results["bad"].finish_reason["message"]
    assert not s.has_work()
    s.add_request("lone", tiny_models.random_tokens(60, 256, 2), SamplingParams(max_new_tokens=50, ignore_eos=True))
    s.run_to_completion()
    r = s.results["lone"]
    assert r.finish_reason == {"type": "length", "message": "KV cache exhausted"} and len(r.output_ids) == 5
    assert s.runner.cache.held_pages() == [0]


def test_finish_on_eos_stop_ids_context_and_abort(setup):
    cfg, weights, path = setup
    p = prompts(cfg, [12], seed=30)[0]
    free_run = plain_impl.greedy_generate(cfg, weights, p, 10)
    s = scheduler(path, eos_token_ids=[free_run[3]])
    s.add_request("a", p, SamplingParams(max_new_tokens=10))
    s.add_request("b", p, SamplingParams(max_new_tokens=10, ignore_eos=True))
    s.add_request("c", p, SamplingParams(max_new_tokens=10, stop_token_ids=[free_run[1]], ignore_eos=False))
    s.run_to_completion()
    first = free_run.index(free_run[3])
    assert s.results["a"].output_ids == free_run[:first + 1]
    assert s.results["a"].finish_reason == {"type": "stop", "value": free_run[3]}
    assert s.results["b"].output_ids == free_run
    assert s.results["c"].output_ids == free_run[:free_run.index(free_run[1]) + 1]
    s = scheduler(path)
    s.add_request("x", tiny_models.random_tokens(250, 256, 3), SamplingParams(max_new_tokens=50, ignore_eos=True))
    s.add_request("y", p, SamplingParams(max_new_tokens=50, ignore_eos=True))
    s.step()
    s.step()
    s.abort_request("y")
    s.run_to_completion()
    assert s.results["x"].finish_reason == {"type": "length", "message": "context length reached"}
    assert len(s.results["x"].output_ids) == 6
    assert s.results["y"].finish_reason["type"] == "abort"
    assert s.runner.cache.held_pages() == [0] and s.runner.cache.slots.available == 8


def test_temperature_seeds(setup):
    cfg, weights, path = setup
    p = prompts(cfg, [9], seed=40)[0]
    s = scheduler(path)
    kw = dict(max_new_tokens=12, temperature=0.7, ignore_eos=True)
    s.add_request("a", p, SamplingParams(seed=3, **kw))
    s.add_request("b", p, SamplingParams(seed=3, **kw))
    s.add_request("c", p, SamplingParams(seed=4, top_k=20, top_p=0.9, **kw))
    s.add_request("d", p, SamplingParams(seed=3, logprobs=True, **kw))
    s.run_to_completion()
    a, b, c, d = (s.results[k] for k in "abcd")
    assert a.output_ids == b.output_ids == d.output_ids and a.output_ids != c.output_ids
    assert len(d.logprobs) == 12 and all(lp <= 0 for lp in d.logprobs)
    # the same request alone draws the same tokens: the draw does not depend on the batch
    s2 = scheduler(path)
    s2.add_request("a", p, SamplingParams(seed=3, **kw))
    s2.run_to_completion()
    assert s2.results["a"].output_ids == a.output_ids
    # and follows the plain sampler step by step
    ids = list(p)
    for i, tok in enumerate(a.output_ids):
        probs = plain_impl.filtered_probs(plain_impl.all_logits(cfg, weights, ids)[-1], 0.7)
        assert plain_impl.inverse_cdf_pick(probs, uniform_for(3, i)) == tok
        ids.append(tok)


def test_overlap_schedule_changes_no_output(setup):
    """Launching a step before the tokens of the one before are read: same tokens, finish reasons
    and bookkeeping as reading them first, through mixed batches, chunked prompts, stop tokens
    (whose extra token in flight is dropped), length limits (known ahead: no extra step), abort,
    temperature with seeds and log-probabilities, penalties and retraction (both fall back to
    reading first)."""
    cfg, weights, path = setup
    ps = prompts(cfg, [1, 7, 33, 64, 150, 20], seed=60)
    # a seeded random run (greedy runs of this tiny model repeat one token) and a token that first
    # appears in the middle of it, to stop on
    drawn = dict(temperature=1.0, seed=11)
    free_run = run(scheduler(path), [ps[2]], 14, **drawn)[0]
    k = next(i for i in range(3, 14) if free_run[i] not in free_run[:i])

    def scenario(overlap, **kw):
        s = scheduler(path, overlap=overlap, chunked_prefill_size=64, eos_token_ids=[free_run[k]], **kw)
        s.add_request("plain", ps[0], SamplingParams(max_new_tokens=9, ignore_eos=True))
        s.add_request("one", ps[1], SamplingParams(max_new_tokens=1, ignore_eos=True))
        s.add_request("eos", ps[2], SamplingParams(max_new_tokens=14, **drawn))
        s.add_request("stop", ps[2], SamplingParams(max_new_tokens=14, stop_token_ids=[free_run[k - 1]], **drawn))
        s.add_request("temp", ps[3], SamplingParams(max_new_tokens=11, temperature=0.8, top_p=0.9, seed=5, logprobs=True,
                                                    ignore_eos=True))
        s.add_request("long", ps[4], SamplingParams(max_new_tokens=6, ignore_eos=True))
        for _ in range(3):
            s.step()
        s.add_request("late", ps[5], SamplingParams(max_new_tokens=12, ignore_eos=True))
        s.add_request("gone", ps[5], SamplingParams(max_new_tokens=30, ignore_eos=True))
        for _ in range(3):
            s.step()
        s.abort_request("gone")
        s.add_request("pen", ps[1], SamplingParams(max_new_tokens=8, repetition_penalty=1.3, ignore_eos=True))
        s.run_to_completion()
        assert not s.has_work() and s.runner.cache.held_pages() == [0] and s.runner.cache.slots.available == 8
        return s

    a, b = scenario(False), scenario(True)
    assert b.overlapped_steps > 10 and a.overlapped_steps == 0
    for rid in ("plain", "one", "eos", "stop", "temp", "long", "late", "pen"):
        ra, rb = a.results[rid], b.results[rid]
        assert ra.output_ids == rb.output_ids and ra.finish_reason == rb.finish_reason, rid
    assert a.results["temp"].logprobs == pytest.approx(b.results["temp"].logprobs)
    assert b.results["eos"].output_ids == free_run[:k + 1] and b.results["eos"].finish_reason["type"] == "stop"
    assert b.results["stop"].output_ids == free_run[:free_run.index(free_run[k - 1]) + 1]
    assert b.results["gone"].finish_reason["type"] == "abort"
    assert b.results["plain"].output_ids == plain_impl.greedy_generate(cfg, weights, ps[0], 9)
    # only the requests that ended on a stop token (and the aborted one) got a step beyond their last token
    assert a.decode_steps <= b.decode_steps <= a.decode_steps + 3
    # retraction under overlap: tokens are read first whenever the pool runs short
    ps2 = prompts(cfg, [20, 25, 18, 30, 22, 27, 19, 24], seed=20)
    want = [plain_impl.greedy_generate(cfg, weights, p, 12) for p in ps2]
    s = scheduler(path, max_tokens=13 * 16, page_size=16, overlap=True)
    assert run(s, ps2, 12) == want and s.retractions > 0 and s.overlapped_steps > 0
    assert s.runner.cache.held_pages() == [0] and s.runner.cache.slots.available == 8


def test_slots_count_requests_whose_last_token_is_in_flight(setup):
    """With every slot taken and requests ending by their length limit while others wait, a new
    request is admitted only when a slot has really come back (the ending request keeps its slot
    until its last token is read)."""
    cfg, weights, path = setup
    ps = prompts(cfg, [5, 9, 3, 12, 7, 4, 8, 6, 10, 2], seed=70)
    outs = {}
    for overlap in (False, True):
        s = scheduler(path, max_requests=2, overlap=overlap)
        for i, p in enumerate(ps):
            s.add_request(f"r{i}", p, SamplingParams(max_new_tokens=1 + i % 3, ignore_eos=True))
        s.run_to_completion()
        assert s.runner.cache.slots.available == 2 and s.runner.cache.held_pages() == [0]
        outs[overlap] = {k: (v.output_ids, v.finish_reason) for k, v in s.results.items()}
        assert all(len(outs[overlap][f"r{i}"][0]) == 1 + i % 3 for i in range(len(ps)))
    assert outs[False] == outs[True]


def test_a_prompt_still_filling_gives_its_pages_back_before_a_running_request_ends(setup):
    """One request decodes, another waits with part of its prompt cached and holds the rest of the
    pool: the decoding one is not cut short ("KV cache exhausted" is for a request that is alone);
    the filling one starts again later and both end as asked."""
    cfg, weights, path = setup
    a, b = prompts(cfg, [14, 120], seed=71)
    s = scheduler(path, max_tokens=160, page_size=16, chunked_prefill_size=32)
    s.add_request("a", a, SamplingParams(max_new_tokens=60, ignore_eos=True))
    s.step()
    s.add_request("b", b, SamplingParams(max_new_tokens=4, ignore_eos=True))
    s.run_to_completion()
    assert s.retractions >= 1
    for rid, p, n in (("a", a, 60), ("b", b, 4)):
        r = s.results[rid]
        assert r.finish_reason == {"type": "length"} and r.output_ids == plain_impl.greedy_generate(cfg, weights, p, n), rid
    assert s.runner.cache.held_pages() == [0]


@pytest.mark.parametrize("seed", [2, 4, 14])
def test_random_arrivals_overlap_equals_reading_first(setup, seed):
    """Random workloads (staggered arrivals, every kind of sampling parameters, small pools, few
    slots, prompt portions of several sizes): launching ahead changes no token and no finish
    reason, nothing is left held, and no request is refused a slot."""
    import random
    cfg, weights, path = setup

    def one(overlap):
        rnd = random.Random(seed)
        s = scheduler(path, max_tokens=rnd.choice([160, 320, 1024]), max_requests=rnd.choice([4, 8, 16]),
                      overlap=overlap, chunked_prefill_size=rnd.choice([32, 64, 128, 8192]))
        reqs = []
        for i in range(rnd.randint(20, 50)):
            p = tiny_models.random_tokens(rnd.choice([1, 2, 3, 5, 17, 40, 100, 150]), cfg["vocab_size"], seed * 1000 + i)
            kind = rnd.random()
            kw = dict(max_new_tokens=rnd.choice([1, 2, 5, 17, 40]), seed=i)
            if 0.3 <= kind < 0.6:
                kw.update(temperature=rnd.choice([0.5, 1.0, 1.5]), top_p=rnd.choice([1.0, 0.9]), top_k=rnd.choice([-1, 20]))
            elif 0.6 <= kind < 0.7:
                kw.update(repetition_penalty=1.2)
            elif 0.7 <= kind < 0.8:
                kw.update(temperature=1.0, logprobs=True)
            elif 0.8 <= kind < 0.9:
                kw.update(top_logprobs=3)
            elif kind >= 0.9:
                kw.update(temperature=1.0, stop_token_ids=[rnd.randrange(cfg["vocab_size"]) for _ in range(40)])
            if rnd.random() < 0.8:
                kw["ignore_eos"] = kind < 0.9
            reqs.append((f"r{i}", p, SamplingParams(**kw)))
        waiting = list(reqs)
        for _ in range(20000):
            for _ in range(rnd.randint(0, 3)):
                if waiting:
                    s.add_request(*waiting.pop(0))
            if not s.step() and not waiting:
                break
        assert not s.has_work() and not waiting and s.runner.cache.held_pages() == [0]
        assert s.runner.cache.slots.available == s.runner.max_requests
        return {rid: (s.results[rid].output_ids, s.results[rid].finish_reason) for rid, _, _ in reqs}, s

    (a, sa), (b, sb) = one(False), one(True)
    assert a == b
    assert sb.overlapped_steps > 20 and sa.overlapped_steps == 0


def test_top_logprobs_follow_the_plain_log_softmax(setup):
    cfg, weights, path = setup
    p = prompts(cfg, [9], seed=45)[0]
    s = scheduler(path, overlap=True)
    s.add_request("a", p, SamplingParams(max_new_tokens=5, top_logprobs=3, logprobs=True, ignore_eos=True))
    s.add_request("b", p, SamplingParams(max_new_tokens=5, ignore_eos=True))
    s.run_to_completion()
    a, b = s.results["a"], s.results["b"]
    assert a.output_ids == b.output_ids and b.top_logprobs is None and len(a.top_logprobs) == 5
    ids = list(p)
    for tok, lp, top in zip(a.output_ids, a.logprobs, a.top_logprobs):
        want = torch.log_softmax(plain_impl.all_logits(cfg, weights, ids)[-1].double(), -1)
        best = torch.topk(want, 3)
        assert [t for t, _ in top] == best.indices.tolist() and top[0][0] == tok       # greedy: the chosen token leads
        assert all(abs(v - float(w)) < 1e-4 for (_, v), w in zip(top, best.values)) and abs(lp - top[0][1]) < 1e-5
        ids.append(tok)


def test_sampling_params_checks():
    with pytest.raises(ValueError, match="top_logprobs"):
        SamplingParams(top_logprobs=0)
    assert SamplingParams(top_logprobs=5).top_logprobs == 5
    for kw in ({"max_new_tokens": 0}, {"temperature": -1}, {"top_p": 0}, {"top_k": 0}, {"min_p": 1.0},
               {"repetition_penalty": 0}, {"stop": "x"}, {"top_logprobs": 65}, {"n": 2}):
        with pytest.raises(ValueError):
            SamplingParams(**kw)
    assert SamplingParams().greedy and SamplingParams(temperature=1.0, top_k=1).greedy
    assert not SamplingParams(temperature=0.5).greedy
    assert SamplingParams(logit_bias={"3": 1}).logit_bias == {3: 1.0}
    us = [uniform_for(1, i) for i in range(1000)]
    assert all(0 <= u < 1 for u in us) and 0.45 < sum(us) / 1000 < 0.55 and uniform_for(1, 5) != uniform_for(2, 5)
