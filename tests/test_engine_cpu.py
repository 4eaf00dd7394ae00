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


@pytest.fixture(scope="module", params=["tiny_qwen3", "tiny_llama", "odd_qwen3", "odd_llama", "partial_qwen3", "partial_llama"])
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


def test_decode_splits_follow_the_clusters_that_fit():
    """With the kernel's answer on how many clusters of s blocks fit (a B200's, head size 128), the most ranges
    whose clusters are all resident; without it, or with more rows than clusters of two, the wave rule."""
    from lily_b200.csrc.ops import choose_decode_splits
    room = {2: 222, 3: 142, 4: 104, 5: 82, 6: 71, 7: 56, 8: 48, 9: 45, 10: 41, 11: 31, 12: 31, 13: 28, 14: 24, 15: 24, 16: 21}
    pick = lambda b, ctx=4096: choose_decode_splits(b, 8, ctx, clusters=lambda s: room.get(s, 0))
    assert [pick(b) for b in (1, 2, 3, 4, 6, 8, 12, 16, 24)] == [16, 16, 13, 10, 8, 6, 4, 3, 2]
    assert pick(1, 1024) == 4 and pick(8, 1024) == 4 and pick(8, 300) == 1            # at least 256 keys a range
    assert pick(32) == choose_decode_splits(32, 8, 4096) == 7 and pick(64) == 4       # no cluster fits: the wave rule
    assert choose_decode_splits(8, 8, 4096) == 6 and choose_decode_splits(0, 8, 4096) == 1
    # a few long rows: a cluster's 16 blocks leave the device idle, one full wave through scratch does not
    assert [pick(1, ctx) for ctx in (8192, 16384, 24576, 32768, 131072)] == [16, 32, 48, 55, 55]
    assert [pick(2, ctx) for ctx in (12288, 16384, 24576, 131072)] == [16, 27, 27, 27]
    assert [pick(4, ctx) for ctx in (8192, 16384, 131072)] == [10, 13, 13]
    assert [pick(b, 131072) for b in (5, 6, 8, 16)] == [9, 8, 6, 3]                    # the clusters fill the device already


def test_whole_rows_rule():
    """One block a (request, kv head) with three stages: from three quarters of the 296 places up to three and a half
    rounds of them, unless the last round would be less than 45 % full."""
    from lily_b200.csrc.ops import whole_rows_pay
    pays = lambda requests: whole_rows_pay(requests * 8)
    assert not pays(1) and not pays(8) and not pays(20) and not pays(27)
    assert pays(28) and pays(32) and pays(37)                      # 224 to 296 blocks: one round
    assert not pays(38) and not pays(48) and pays(56) and pays(64) and pays(74)
    assert not pays(80) and pays(96) and pays(128) and not pays(130) and not pays(148) and not pays(256)


def test_rows_are_even():
    from lily_b200.engine.batch import rows_are_even
    assert rows_are_even([4096] * 32) and rows_are_even([4000, 4096, 4200, 3900]) and rows_are_even([7])
    assert not rows_are_even([]) and not rows_are_even([100, 4096]) and not rows_are_even([3000] * 31 + [4096])
    assert rows_are_even([3700] * 31 + [4096])


def test_gate_up_rule_sends_badly_filled_rounds_to_the_library(monkeypatch):
    """129 to 256 tokens are one pair of row blocks: the fused kernel pays only if its column tiles fill the block pairs."""
    from lily_b200.csrc import ops
    monkeypatch.setattr(ops, "sm_count", lambda: 148)
    pays = ops.gate_up_fused_pays
    assert not pays(64, 24576) and pays(65, 24576) and pays(128, 24576) and pays(257, 24576) and pays(2048, 24576)
    assert not pays(129, 24576) and not pays(256, 24576)          # 96 tiles on 74 pairs: the second round is a third full
    assert not pays(200, 28672)                                   # 112 tiles: half full
    assert pays(200, 51200) and pays(200, 2 * 18944)              # 200 and 148 tiles: 0.9 and all of three and two rounds


def test_both_forms_of_the_decode_step_agree(setup, monkeypatch):
    """A step in which every request brings one token may start its attention from the qkv product or run the
    norm / rotation / cache-write kernel first: same logits, same cache."""
    import kernel_refs
    cfg, weights, path = setup
    ids = tiny_models.random_tokens(60, cfg["vocab_size"], 4)
    want = plain_impl.all_logits(cfg, weights, ids)
    for fused in (True, False):
        monkeypatch.setattr(kernel_refs, "FUSE_DECODE", fused)
        runner = make_runner(path, page_size=16, max_tokens=160)
        assert float((run_portions(runner, ids, [30] + [1] * 30) - want).abs().max()) < TOL, fused


def test_bfloat16_layouts_on_the_host(setup):
    """In bfloat16 the fused gate/up matrix alternates runs of gate and up rows when the kernels ask for it, and
    a few tokens' products come as partial sums: the plain statements follow, so the packing is checked here."""
    cfg, weights, path = setup
    ids = tiny_models.random_tokens(90, cfg["vocab_size"], 6)
    want = plain_impl.all_logits(cfg, weights, ids)
    runner = make_runner(path, dtype="bfloat16", page_size=16, max_tokens=160)
    scale = float(want.abs().max())
    for got in (run_whole(runner, ids), run_portions(runner, ids, [70, 3] + [1] * 17)):
        err = (got - want).abs()
        assert float(err.max()) < 2e-2 * scale and float(err.mean()) < 3e-3 * scale


def test_one_capture_serves_both_kinds_of_batch_unless_a_part_plans_by_evenness(setup, monkeypatch):
    """The table of captured decode steps, with a stand-in for the capture itself: a step whose parts did not plan by
    the rows' evenness is stored for even and for uneven batches; one whose parts did is captured once for each."""
    from lily_b200.engine import runner as runner_module
    cfg, weights, path = setup
    runner = make_runner(path)
    made = []

    class Captured:
        def __init__(self, owner, bucket, cls, even):
            self.key, self.even_matters = (bucket, cls, even), bucket >= 32
            made.append(self.key)
    monkeypatch.setattr(runner_module, "_DecodeGraph", Captured)
    small = runner._graph_for(8, 8192, True)
    assert runner._graph_for(8, 8192, False) is small and made == [(8, 8192, True)]
    large = runner._graph_for(32, 8192, False)
    other = runner._graph_for(32, 8192, True)
    assert other is not large and runner._graph_for(32, 8192, False) is large and runner._graph_for(32, 8192, True) is other
    assert made == [(8, 8192, True), (32, 8192, False), (32, 8192, True)]
    assert sorted(runner._graphs) == [(8, 8192, False), (8, 8192, True), (32, 8192, False), (32, 8192, True)]


def test_step_checks_catch_what_the_kernels_would_trust(setup):
    """With LILY_B200_CHECK_STEPS on (the tests switch it on) a page id beyond the pool, a page held twice, a
    request whose length the cache manager does not know of, and a stale row are refused before anything runs."""
    from lily_b200.engine import check
    from lily_b200.engine.batch import StepEntry
    assert check.ENABLED
    cfg, _, path = setup
    v = cfg["vocab_size"]
    runner = make_runner(path, page_size=16, max_tokens=160)
    a, b = runner.open_request(), runner.open_request()
    runner.step([StepEntry(a, tiny_models.random_tokens(20, v, 1), []), StepEntry(b, tiny_models.random_tokens(5, v, 2), [])])
    pages_a = runner.cache.groups[0].tables.tables[a].pages
    pages_b = runner.cache.groups[0].tables.tables[b].pages
    kept = pages_a[0]
    pages_a[0] = runner.cache.num_pages + 7
    with pytest.raises(check.StepCheckError, match="page id"):
        runner.step([StepEntry(a, [1], [0])])
    pages_a[0] = pages_b[0]
    with pytest.raises(check.StepCheckError, match="held by slots"):
        runner.step([StepEntry(a, [1], [0])])
    pages_a[0] = kept
    runner.seq_lens[b] += 40                     # the step function believes in positions nobody cached
    with pytest.raises(check.StepCheckError, match="cache manager holds pages"):
        check.check_entries(runner, [StepEntry(b, [1], [0])])
    runner.seq_lens[b] -= 40
    out = runner.step([StepEntry(a, [1], [0]), StepEntry(b, [2, 3], [1])])
    assert out.shape == (2, v)
