"""The engine on the GPU against the plain implementation, in float32 and in bfloat16: whole
requests, most of a request in one step and the last 32 tokens one by one, portions of changing
size down to two tokens, and mixed batches over so few pages that they are used again."""

import os
import tempfile

import pytest
import torch

import plain_impl
import tiny_models
from harness import make_runner, model_dir, run_mixed, run_portions, run_whole
from lily_b200.engine.batch import StepEntry

pytestmark = pytest.mark.gpu

# float32: rounding only, absolute (logits are of order one).  bfloat16: activations carry 8 bits; the bounds are
# relative to the largest logit of the sequence, about three times what correct kernels give (largest error
# 0.2 to 0.6 % of it, mean 0.03 to 0.13 %), so a defect worth a hundredth of a logit fails.
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
MEAN_TOL = {"float32": 1e-5, "bfloat16": 3e-3}


def rounded(weights, dtype):
    """What the engine holds: matrices in the compute dtype, float32 gains kept."""
    if dtype == "float32":
        return weights
    return {k: (v if v.dim() == 1 and "bias" not in k else v.bfloat16().float()) for k, v in weights.items()}


def close(got, want, dtype, what=""):
    err = (got - want).abs()
    scale = float(want.abs().max()) if dtype == "bfloat16" else 1.0
    assert float(err.max()) < TOL[dtype] * scale, \
        f"{what}: max error {float(err.max()):.3e} at {int(err.argmax()) // want.shape[1]} (logits up to {scale:.2f})"
    assert float(err.mean()) < MEAN_TOL[dtype] * scale, f"{what}: mean error {float(err.mean()):.3e} (logits up to {scale:.2f})"


@pytest.fixture(scope="module", params=["tiny_qwen3", "tiny_llama", "odd_qwen3", "odd_llama", "partial_qwen3", "partial_llama"])
def setup(request):
    cfg = tiny_models.CONFIGS[request.param]
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 31, tmp)
        yield cfg, weights, path


@pytest.mark.parametrize("head_dim", [128, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_size_128_paths_inside_the_engine(dtype, head_dim):
    """Head size 128 (and 64), widths in multiples of 128, page size 64: tensor-core attention (tcgen05 for
    portions of 128 tokens and more, mma.sync below that and for split-key decode through graphs),
    the tcgen05 gate/up kernel and the weight-streaming decode product, all through the step
    function, against the plain implementation."""
    cfg = dict(tiny_models.MID_QWEN3, head_dim=head_dim)
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 33, tmp)
        v = cfg["vocab_size"]
        ids = tiny_models.random_tokens(700, v, 4)
        want = plain_impl.all_logits(cfg, rounded(weights, dtype), ids)
        runner = make_runner(path, dtype=dtype, device="cuda", page_size=64, max_tokens=2048 + 512)
        close(run_whole(runner, ids), want, dtype, "whole")
        close(run_portions(runner, ids, [668] + [1] * 32), want, dtype, "last 32 one by one")
        close(run_portions(runner, ids, [130, 2, 300, 65, 3, 129]), want, dtype, "portions")
        reqs = {k: tiny_models.random_tokens(n, v, 50 + i) for i, (k, n) in enumerate({"a": 400, "b": 330, "c": 200, "d": 90}.items())}
        plan = [{"a": 300, "b": 70}, {"a": 1, "b": 200, "c": 2}, {"a": 1, "b": 1, "c": 198, "d": 66}] + [{k: 1 for k in "abd"}] * 24
        got = run_mixed(runner, reqs, plan)
        for name, toks in reqs.items():
            full = plain_impl.all_logits(cfg, rounded(weights, dtype), toks)
            close(got[name], full[:got[name].shape[0]], dtype, name)
        assert runner.graph_steps > 0 and runner.cache.held_pages() == [0]
        if dtype == "bfloat16":
            from lily_b200.csrc import ops
            assert ops.uses_tcgen05_attention(torch.bfloat16, cfg["head_dim"], 64, 130)     # the portions of 130 tokens and more
            assert ops.attention_tc_status() == 0 and ops.gemm_tc_status() == 0          # no bounded wait gave up


def test_decode_graphs_captured_ahead():
    """Capturing the decode graphs while a request is half way through its prompt disturbs neither its cache nor what
    it decodes afterwards, and the steps that follow find their graphs there."""
    cfg = tiny_models.MID_QWEN3
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 35, tmp)
        ids = tiny_models.random_tokens(200, cfg["vocab_size"], 7)
        want = plain_impl.all_logits(cfg, rounded(weights, "bfloat16"), ids)
        runner = make_runner(path, dtype="bfloat16", device="cuda", page_size=64, max_tokens=1024)
        slot = runner.open_request()
        first = runner.step([StepEntry(slot, ids[:150], list(range(150)))])
        assert runner.capture_decode_graphs([1, 3]) == [1, 4] and runner.capture_decode_graphs([2, 4]) == [2]
        graphs = dict(runner._graphs)
        rest = [runner.step([StepEntry(slot, [t], [0])]).clone() for t in ids[150:]]     # a graph's logits live until its next replay
        assert runner.graph_steps == 50 and runner._graphs == graphs            # nothing was captured on the way
        close(torch.cat([first] + rest).cpu(), want, "bfloat16", "captured ahead")
        runner.close_request(slot)
        assert runner.cache.held_pages() == [0]
        assert len(runner.capture_decode_graphs()) == len(runner.graph_buckets) - 3


def test_decode_graphs_come_in_classes_of_length():
    """With a context past 8 k positions the captured decode steps come in classes of sequence length, each planned
    for its own bound: a short request decodes through the first class (key ranges merged inside clusters), one that
    has passed 16 k positions through the third (one full wave of ranges), and both agree with the plain implementation
    on the device."""
    cfg = dict(tiny_models.MID_QWEN3, num_attention_heads=8, num_key_value_heads=8, max_position_embeddings=40000)
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 37, tmp)
        runner = make_runner(path, dtype="bfloat16", device="cuda", page_size=64, max_tokens=20000, context_length=40000)
        assert runner.length_classes == [8192, 16384, 32768, 40000]
        dev_weights = {k: v.cuda() for k, v in rounded(weights, "bfloat16").items()}
        plans = {}
        for n in (300, 16500):
            ids = tiny_models.random_tokens(n + 6, cfg["vocab_size"], n)
            want = plain_impl.all_logits(cfg, dev_weights, ids)[-6:]
            slot = runner.open_request()
            runner.step([StepEntry(slot, ids[:n], [])])
            got = torch.cat([runner.step([StepEntry(slot, [t], [0])]).clone() for t in ids[n:]])
            runner.close_request(slot)
            close(got.cpu(), want.cpu(), "bfloat16", f"{n} positions")
            cls = runner._length_class(n + 6)
            graph = runner._graphs[(1, cls, True)]
            assert graph is runner._graphs[(1, cls, False)] and not graph.even_matters     # one row: nothing to plan by
            plans[cls] = next(iter(graph.batch.plans.values())).decode
        assert sorted({k[:2] for k in runner._graphs}) == [(1, 8192), (1, 32768)] and runner.graph_steps == 12
        clusters = os.environ.get("LILY_B200_DECODE_CLUSTER") != "0"
        assert plans[8192].arm == ("cluster" if clusters else "wave") and plans[32768].arm == "wave"
        assert plans[32768].splits > plans[8192].splits if clusters else plans[32768].splits >= plans[8192].splits
        assert runner.capture_decode_graphs([1], max_len=33000) == [1] and (1, 40000, False) in runner._graphs
        assert runner.cache.held_pages() == [0]


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configurations_in_every_cutting(seed, dtype):
    """Configurations drawn at random (head counts and groups, head sizes in steps of 16, widths and vocabularies
    that are no power of two, page sizes 16 to 64): whole, last 32 one by one, random portions down to two tokens,
    and mixed over a pool so small that pages are used again."""
    import random
    cfg = tiny_models.random_config(seed)
    r = random.Random(seed + 999)
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, seed, tmp)
        v = cfg["vocab_size"]
        n, page = r.choice([70, 150, 260]), r.choice([16, 32, 64])
        ids = tiny_models.random_tokens(n, v, seed)
        others = {k: tiny_models.random_tokens(m, v, seed * 7 + i) for i, (k, m) in enumerate((("b", 60), ("c", 45), ("d", 70)))}
        w = rounded(weights, dtype)
        want = plain_impl.all_logits(cfg, w, ids)
        pool = (-(-n // page) - (-60 // page) - (-45 // page) + 1) * page     # "d" fits only in what "b" gives back
        runner = make_runner(path, dtype=dtype, device="cuda", page_size=page, max_tokens=pool, max_requests=4, context_length=1024)
        close(run_whole(runner, ids), want, dtype, "whole")
        close(run_portions(runner, ids, [n - 32] + [1] * 32), want, dtype, "last 32 one by one")
        close(run_portions(runner, ids, [r.choice([2, 3, 5, 16, 17, 31, 64]) for _ in range(40)]), want, dtype, "portions")
        plan = [{"a": n // 2, "b": 20}, {"a": n // 4, "b": 2, "c": 30}, {"a": 1, "b": 38, "c": 1}] + [{"a": 1, "c": 1, "d": 4}] * 14 + \
               [{"a": n, "c": 9, "d": 14}]
        got = run_mixed(runner, {"a": ids, **others}, plan, ends={2: ["b"]})
        close(got["a"], want, dtype, "a")
        for k, toks in others.items():
            close(got[k], plain_impl.all_logits(cfg, w, toks)[:got[k].shape[0]], dtype, k)
        assert runner.cache.held_pages() == [0]


def test_pages_whose_offset_passes_two_to_the_31_elements():
    """A pool of 8.9 GB in which the request's pages lie past element 2^31 of a layer's cache (16 requests that only
    hold pages fill the front of the pool): the same logits, bit for bit, as in a small pool, through the
    tcgen05 and the mma.sync attention kernels, the cache write and the decode graphs.  A 32-bit offset
    anywhere would read or write the wrong page."""
    cfg = dict(tiny_models.MID_QWEN3, num_attention_heads=16, num_key_value_heads=8, hidden_size=512)
    with tempfile.TemporaryDirectory() as tmp:
        path, _ = model_dir(cfg, 34, tmp)
        ids = tiny_models.random_tokens(700, cfg["vocab_size"], 5)

        def logits_of(runner):
            whole = run_whole(runner, ids[:600])[-3:]
            cut = run_portions(runner, ids, [300, 130, 2, 200, 60] + [1] * 8)[-12:]
            return torch.cat([whole, cut])

        # the same context length in both, so that the decode graphs cut the keys into the same ranges
        small = make_runner(path, dtype="bfloat16", device="cuda", page_size=64, max_tokens=4096, context_length=65536)
        want = logits_of(small)
        del small
        torch.cuda.empty_cache()
        pages = 17000
        big = make_runner(path, dtype="bfloat16", device="cuda", page_size=64, max_tokens=pages * 64, max_requests=20,
                          context_length=65536)
        held = []
        for _ in range(16):                                   # 16 x 1024 pages: the front of the pool
            slot = big.cache.open_request()
            big.cache.grow(slot, 65536)
            held.append(slot)
        probe = big.cache.open_request()
        big.cache.grow(probe, 64)
        first = big.cache.block_table(0, probe)[0]
        big.cache.close_request(probe)
        elements_per_page = 2 * cfg["num_key_value_heads"] * 64 * cfg["head_dim"]
        assert first * elements_per_page > 2 ** 31, first
        got = logits_of(big)
        assert torch.equal(got, want)
        for slot in held:
            big.cache.close_request(slot)
        assert big.cache.held_pages() == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decode_and_portions(setup, dtype):
    cfg, weights, path = setup
    ids = tiny_models.random_tokens(150, cfg["vocab_size"], 3)
    want = plain_impl.all_logits(cfg, rounded(weights, dtype), ids)
    runner = make_runner(path, dtype=dtype, device="cuda", page_size=16, max_tokens=160)
    close(run_whole(runner, ids), want, dtype, "whole")
    close(run_portions(runner, ids, [118] + [1] * 32), want, dtype, "last 32 one by one")
    close(run_portions(runner, ids, [8, 2, 30, 17, 2, 3, 40, 2, 5]), want, dtype, "portions")
    close(run_portions(runner, ids, [1, 1, 1, 2, 1]), want, dtype, "first tokens")
    assert runner.cache.held_pages() == [0] * len(runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages(setup, dtype):
    cfg, weights, path = setup
    v = cfg["vocab_size"]
    reqs = {"a": tiny_models.random_tokens(50, v, 5), "b": tiny_models.random_tokens(37, v, 6),
            "c": tiny_models.random_tokens(20, v, 7), "d": tiny_models.random_tokens(41, v, 8),
            "e": tiny_models.random_tokens(30, v, 9)}
    plan = [{"a": 30}, {"a": 1, "b": 20}, {"b": 17, "a": 1, "c": 20}, {"a": 18, "d": 2}, {"d": 39, "e": 7},
            {"e": 1}, {"e": 22}]
    ends = {2: ["c", "b"], 3: ["a"], 4: ["d"]}
    runner = make_runner(path, dtype=dtype, device="cuda", page_size=16, max_tokens=9 * 16)
    got = run_mixed(runner, reqs, plan, ends)
    for name, ids in reqs.items():
        close(got[name], plain_impl.all_logits(cfg, rounded(weights, dtype), ids), dtype, name)
    assert runner.cache.held_pages() == [0] * len(runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_four_live_requests(setup, dtype):
    cfg, weights, path = setup
    v, ctx = cfg["vocab_size"], cfg["max_position_embeddings"]
    n = min(ctx, 230)
    reqs = {k: tiny_models.random_tokens(n - 7 * i, v, 40 + i) for i, k in enumerate("abcd")}
    plan = [{"a": 3, "b": 64, "c": 2, "d": 17}] + [{k: 1 for k in "abcd"}] * (n - 3)
    runner = make_runner(path, dtype=dtype, device="cuda", page_size=16, max_tokens=4 * 240)
    got = run_mixed(runner, reqs, plan)
    for name, ids in reqs.items():
        close(got[name], plain_impl.all_logits(cfg, rounded(weights, dtype), ids), dtype, name)


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "eager"])
@pytest.mark.parametrize("live", [20, 70])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["mid_8kv", "random"])
def test_many_live_requests(which, dtype, live, graphs, monkeypatch):
    """20 and 70 requests of ragged lengths (5 to 560 tokens) decoding side by side for 44 steps, through captured
    graphs and without them; a third of them end on the way and others take their slots and pages.  Every decoded
    row is held to the plain implementation, and the forms the attention took are the ones meant for these sizes:
    graph buckets past 8, products of 17 to 64 tokens, key ranges merged inside clusters or through scratch and a
    combine kernel, the attention started from the qkv product or behind the rotation kernel."""
    import random
    from lily_b200.csrc import ops
    from lily_b200.engine.batch import StepEntry
    if which == "mid_8kv":
        cfg = dict(tiny_models.MID_QWEN3, num_attention_heads=16, num_key_value_heads=8)
    else:
        cfg = dict(tiny_models.random_config(0), max_position_embeddings=1024)     # 20 heads over 4, width 328
    r = random.Random(live)
    v = cfg["vocab_size"]
    plans = []
    real_plan = ops.plan_decode_attention

    def recorded(*a, even=False):
        plan = real_plan(*a, even=even)
        if not even:                    # the rows here are ragged: the plan for even rows is asked for only to compare
            plans.append(plan)
        return plan
    monkeypatch.setattr(ops, "plan_decode_attention", recorded)
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 35, tmp)
        dev_weights = {k: t.cuda() for k, t in rounded(weights, dtype).items()}
        steps, swap_at = 44, 15
        first = [r.choice([5, 17, 64, 130, 300, 517, 560]) + r.randint(0, 3) for _ in range(live)]
        later = [r.choice([9, 70, 200]) for _ in range(live // 3)]
        seqs = [tiny_models.random_tokens(n + steps, v, 1000 + i) for i, n in enumerate(first)]
        newcomers = [tiny_models.random_tokens(n + steps - swap_at, v, 5000 + i) for i, n in enumerate(later)]
        leaving = list(range(0, live, 3))[:len(newcomers)]
        need = lambda group: sum(-(-len(ids) // 64) for ids in group)
        # the pool holds the first set whole, or those who stay and the newcomers: what the leavers give back is
        # what the newcomers get (the free list hands out the page given back last)
        pages = max(need(seqs), need([ids for i, ids in enumerate(seqs) if i not in leaving] + newcomers))
        runner = make_runner(path, dtype=dtype, device="cuda", page_size=64, max_tokens=pages * 64, max_requests=live,
                             context_length=1024, disable_cuda_graph=not graphs)
        slots = [runner.open_request() for _ in seqs]
        for at in range(0, live, 7):                                # prompts go in seven requests a step
            runner.step([StepEntry(slots[i], seqs[i][:first[i]], []) for i in range(at, min(at + 7, live))])
        at_pos = list(first)
        rows = [[] for _ in seqs]
        for s in range(steps):
            entries = [StepEntry(slots[i], [seqs[i][at_pos[i]]], [0]) for i in range(len(seqs)) if slots[i] is not None]
            index = [i for i in range(len(seqs)) if slots[i] is not None]
            if s == swap_at:
                # every third request ends; as many new ones bring their prompts beside the others' decoded tokens
                for i in leaving:
                    runner.close_request(slots[i])
                    slots[i] = None
                entries = [e for e, i in zip(entries, index) if slots[i] is not None]
                index = [i for i in index if slots[i] is not None]
                for j, ids in enumerate(newcomers):
                    seqs.append(ids)
                    slots.append(runner.open_request())
                    at_pos.append(0)
                    rows.append([])
                    entries.append(StepEntry(slots[-1], ids[:later[j]], [later[j] - 1]))
                    index.append(len(seqs) - 1)
            out = runner.step(entries).float()
            for row, (i, e) in enumerate(zip(index, entries)):
                rows[i].append((at_pos[i] + len(e.tokens) - 1, out[row].clone()))
                at_pos[i] += len(e.tokens)
        for i, slot in enumerate(slots):
            if slot is not None:
                runner.close_request(slot)
        assert runner.cache.held_pages() == [0] and runner.cache.slots.available == live
        for i, ids in enumerate(seqs):
            want = plain_impl.all_logits(cfg, dev_weights, ids)
            got = torch.stack([t for _, t in rows[i]])
            close(got.cpu(), want[[p for p, _ in rows[i]]].cpu(), dtype, f"request {i}")
        assert (runner.graph_steps == steps - 1) if graphs else (runner.graph_steps == 0)      # all but the mixed step
        decode = [p for p in plans if p.arm != "single"]
        assert decode, plans
        if which == "mid_8kv":            # 8 kv heads: 160 and 560 (request, kv head) pairs
            arms = {p.arm for p in decode}
            if dtype == "bfloat16" and live == 20 and os.environ.get("LILY_B200_DECODE_CLUSTER") != "0":
                assert arms == {"cluster"}, arms                                   # merged inside clusters
            else:
                assert arms == {"wave"} and all(p.scratch_floats > 0 for p in decode), arms     # scratch and the combine kernel
            if live == 70:
                assert not any(p.fused for p in decode)                            # too many blocks: the rotation kernel runs first
            elif dtype == "bfloat16":
                assert any(p.fused for p in decode)
