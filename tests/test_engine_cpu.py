"""The engine's host side (packing, cache, schedule walking, replay order) on the CPU.

The kernels are replaced by their plain PyTorch statements (tests/kernel_refs.py), so what is
tested here is everything around them: that logits do not depend on how a request is cut into
steps, on what else is in the batch, or on which pages are used.
"""

import tempfile

import pytest
import torch

import plain_impl
import tiny_models
from harness import make_runner, model_dir, run_mixed, run_portions, run_whole

TOL = 2e-5


@pytest.fixture(scope="module", params=["tiny_qwen3", "tiny_llama", "odd_qwen3", "odd_llama"])
def setup(request):
    cfg = tiny_models.CONFIGS[request.param]
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 21, tmp)
        yield cfg, weights, path


def test_whole_portions_and_decode_match_plain(setup):
    cfg, weights, path = setup
    ids = tiny_models.random_tokens(75, cfg["vocab_size"], 3)
    want = plain_impl.all_logits(cfg, weights, ids)
    runner = make_runner(path, page_size=16, max_tokens=160)
    assert float((run_whole(runner, ids) - want).abs().max()) < TOL
    assert float((run_portions(runner, ids, [43] + [1] * 32) - want).abs().max()) < TOL
    assert float((run_portions(runner, ids, [8, 2, 30, 17, 2, 3]) - want).abs().max()) < TOL
    assert runner.cache.held_pages() == [0] * len(runner.cache.groups)


def test_mixed_batches_reuse_pages(setup):
    cfg, weights, path = setup
    v = cfg["vocab_size"]
    reqs = {"a": tiny_models.random_tokens(50, v, 5), "b": tiny_models.random_tokens(37, v, 6),
            "c": tiny_models.random_tokens(20, v, 7), "d": tiny_models.random_tokens(41, v, 8),
            "e": tiny_models.random_tokens(30, v, 9)}
    plan = [{"a": 30}, {"a": 1, "b": 20}, {"b": 17, "a": 1, "c": 20}, {"a": 18, "d": 2}, {"d": 39, "e": 7},
            {"e": 1}, {"e": 22}]
    ends = {2: ["c", "b"], 3: ["a"], 4: ["d"]}
    runner = make_runner(path, page_size=16, max_tokens=9 * 16)
    got = run_mixed(runner, reqs, plan, ends)
    for name, ids in reqs.items():
        want = plain_impl.all_logits(cfg, weights, ids)
        assert float((got[name] - want).abs().max()) < TOL, name
    assert runner.cache.held_pages() == [0] * len(runner.cache.groups)


def test_wanted_rows_come_in_the_given_order(setup):
    cfg, weights, path = setup
    from lily_b200.engine.batch import StepEntry
    v = cfg["vocab_size"]
    a, b = tiny_models.random_tokens(9, v, 1), tiny_models.random_tokens(5, v, 2)
    runner = make_runner(path)
    sa, sb = runner.open_request(), runner.open_request()
    runner.step([StepEntry(sa, a[:8], [])])
    # a brings one token (runs first inside the batch), b a portion; the output keeps the given order
    out = runner.step([StepEntry(sb, b, [4, 0]), StepEntry(sa, a[8:], [0])]).float()
    la, lb = plain_impl.all_logits(cfg, weights, a), plain_impl.all_logits(cfg, weights, b)
    want = torch.stack([lb[4], lb[0], la[8]])
    assert float((out - want).abs().max()) < TOL
