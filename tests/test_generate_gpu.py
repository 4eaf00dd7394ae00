"""Generation through the Python entry point and the command line on the GPU."""

import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

import plain_impl
import tiny_models
from harness import model_dir
from test_engine_gpu import rounded

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(path, dtype, **kw):
    from lily_b200 import Engine, EngineConfig
    return Engine(EngineConfig(path, dtype=dtype, max_total_tokens=kw.pop("max_total_tokens", 2048),
                               max_running_requests=kw.pop("max_running_requests", 8), server_args=kw or None))


def greedy_with_gaps(cfg, weights, prompt, n):
    """Plain greedy tokens with the runner-up and the top-2 gap at each position
    (the reference's tie-tolerant compare, tests/util.py:50-112 there)."""
    ids, toks, second, gaps = list(prompt), [], [], []
    for _ in range(n):
        top = torch.topk(plain_impl.all_logits(cfg, weights, ids)[-1], 2)
        toks.append(int(top.indices[0])); second.append(int(top.indices[1])); gaps.append(float(top.values[0] - top.values[1]))
        ids.append(toks[-1])
    return toks, second, gaps


def matches_up_to_tie_flip(got, ref, second, gaps, tie_gap):
    for i, (g, r) in enumerate(zip(got, ref)):
        if g != r:
            assert gaps[i] < tie_gap and g == second[i], f"position {i}: {g} vs {r}, gap {gaps[i]:.4f}"
            return i
    return len(ref)


@pytest.mark.parametrize("name", ["tiny_qwen3", "tiny_llama"])
def test_greedy_generation_float32_equals_plain(name):
    cfg = tiny_models.CONFIGS[name]
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 61, tmp)
        eng = engine(path, "float32", page_size=16)
        lens = [1, 7, 33, 64] if name == "tiny_qwen3" else [3, 17, 50, 100, 200, 300]
        prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 70 + i) for i, n in enumerate(lens)]
        want = [plain_impl.greedy_generate(cfg, weights, p, 16) for p in prompts]
        from lily_b200 import SamplingParams
        got = eng.generate(prompts, SamplingParams(max_new_tokens=16, ignore_eos=True))
        assert [g["output_ids"] for g in got] == want
        assert eng.generate_greedy(prompts[1], 16) == want[1]
        free = eng.kv_available()
        logits = eng.all_prefill_logits(prompts[2]).cpu()
        assert float((logits - plain_impl.all_logits(cfg, weights, prompts[2])).abs().max()) < 1e-4
        assert torch.equal(eng.prefill_logits(prompts[2]).cpu(), logits[-1])
        assert eng.kv_available() == free, "pages leaked"


def test_greedy_generation_bfloat16_up_to_tie_flips():
    cfg = tiny_models.TINY_LLAMA
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 62, tmp)
        eng = engine(path, "bfloat16", page_size=16)
        w = rounded(weights, "bfloat16")
        for i, n in enumerate([5, 40, 130]):
            p = tiny_models.random_tokens(n, cfg["vocab_size"], 80 + i)
            ref, second, gaps = greedy_with_gaps(cfg, w, p, 24)
            assert matches_up_to_tie_flip(eng.generate_greedy(p, 24), ref, second, gaps, tie_gap=0.03) >= 3


def test_temperature_generation_follows_the_plain_sampler():
    # tiny-llama workload of the benchmark description: temperature 0.7 under a fixed seed, page size 16
    cfg = tiny_models.TINY_LLAMA
    from lily_b200 import SamplingParams
    from lily_b200.sampling.sampler import uniform_for
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 63, tmp)
        eng = engine(path, "float32", page_size=16, chunked_prefill_size=128)
        prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 90 + i) for i, n in enumerate([3, 17, 50, 100, 200, 300])]
        params = [SamplingParams(max_new_tokens=24, temperature=0.7, seed=100 + i, ignore_eos=True) for i in range(6)]
        got = eng.generate(prompts, params)
        for i, (p, g) in enumerate(zip(prompts, got)):
            ids = list(p)
            for j, tok in enumerate(g["output_ids"]):
                probs = plain_impl.filtered_probs(plain_impl.all_logits(cfg, weights, ids)[-1], 0.7).double()
                cum = torch.cumsum(probs, 0)
                u = uniform_for(100 + i, j)
                assert float(cum[tok] - probs[tok]) - 1e-4 <= u < float(cum[tok]) + 1e-4, (i, j)
                ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlap_schedule_on_the_gpu_changes_no_token(dtype):
    """Steps launched before the tokens of the step before are read (graphs, the table of future
    tokens on the device, asynchronous copies) give the tokens of steps that read first."""
    cfg = tiny_models.TINY_LLAMA
    from lily_b200 import SamplingParams
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 65, tmp)
        prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 120 + i) for i, n in enumerate([3, 17, 50, 100, 200])]
        params = [SamplingParams(max_new_tokens=20 + i, temperature=0.9, seed=7 + i, ignore_eos=True) for i in range(5)]
        plain = engine(path, dtype, page_size=16, chunked_prefill_size=128, disable_overlap_schedule=True)
        first = plain.generate(prompts, params)
        assert plain.last_scheduler.overlapped_steps == 0
        # a token that appears in the middle of a run, to stop on: the extra token in flight is dropped
        run = first[2]["output_ids"]
        k = next(i for i in range(3, len(run)) if run[i] not in run[:i])
        params[2] = SamplingParams(max_new_tokens=22, temperature=0.9, seed=9, stop_token_ids=[run[k]])
        want = plain.generate(prompts, params)
        assert want[2]["output_ids"] == run[:k + 1] and want[2]["finish_reason"]["type"] == "stop"
        eng = engine(path, dtype, page_size=16, chunked_prefill_size=128)
        got = eng.generate(prompts, params)
        assert [g["output_ids"] for g in got] == [w["output_ids"] for w in want]
        assert [g["finish_reason"] for g in got] == [w["finish_reason"] for w in want]
        assert eng.last_scheduler.overlapped_steps > 15 and eng.runner.graph_steps > 15
        assert eng.kv_available() == 2048


def test_top_logprobs_on_the_gpu():
    cfg = tiny_models.TINY_LLAMA
    from lily_b200 import SamplingParams
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 66, tmp)
        eng = engine(path, "float32", page_size=16)
        p = tiny_models.random_tokens(40, cfg["vocab_size"], 130)
        out = eng.generate([p, p], [SamplingParams(max_new_tokens=6, top_logprobs=4, logprobs=True, ignore_eos=True),
                                    SamplingParams(max_new_tokens=6, temperature=0.8, seed=2, top_logprobs=2, ignore_eos=True)])
        for o, k in zip(out, (4, 2)):
            ids = list(p)
            assert len(o["top_logprobs"]) == 6
            for tok, top in zip(o["output_ids"], o["top_logprobs"]):
                want = torch.log_softmax(plain_impl.all_logits(cfg, weights, ids)[-1].double(), -1)
                best = torch.topk(want, k)
                assert [t for t, _ in top] == best.indices.tolist()
                assert all(abs(v - float(w)) < 1e-4 for (_, v), w in zip(top, best.values))
                ids.append(tok)
        assert out[0]["top_logprobs"][0][0][0] == out[0]["output_ids"][0] and abs(out[0]["logprobs"][0] - out[0]["top_logprobs"][0][0][1]) < 1e-5


def test_small_pool_retracts_on_the_gpu():
    cfg = tiny_models.TINY_QWEN3
    from lily_b200 import SamplingParams
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 64, tmp)
        prompts = [tiny_models.random_tokens(n, 256, 110 + i) for i, n in enumerate([20, 25, 18, 30, 22, 27, 19, 24])]
        want = [plain_impl.greedy_generate(cfg, weights, p, 12) for p in prompts]
        eng = engine(path, "float32", page_size=16, max_total_tokens=13 * 16)
        got = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
        assert [g["output_ids"] for g in got] == want
        assert eng.last_scheduler.retractions > 0 and eng.kv_available() == 13 * 16


def test_command_line_generates():
    cfg = tiny_models.TINY_QWEN3
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 65, tmp)
        p = tiny_models.random_tokens(9, 256, 5)
        out = subprocess.run([sys.executable, "-m", "lily_b200", "generate", "--model-path", path, "--dtype", "float32",
                              "--max-total-tokens", "256", "--page-size", "16", "--prompt-ids",
                              ",".join(map(str, p)), "--max-new-tokens", "6", "--ignore-eos"],
                             cwd=ROOT, capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        assert json.loads(out.stdout.strip().splitlines()[-1])["output_ids"] == plain_impl.greedy_generate(cfg, weights, p, 6)


def test_the_step_profile_names_this_packages_kernels(monkeypatch):
    """LILY_B200_PROFILE_BS arms the step function: after the window a table says where a decode step's time went."""
    monkeypatch.setenv("LILY_B200_PROFILE_BS", "3")
    monkeypatch.setenv("LILY_B200_PROFILE_STEPS", "6")
    cfg = tiny_models.MID_QWEN3
    with tempfile.TemporaryDirectory() as tmp:
        monkeypatch.setenv("LILY_B200_PROFILE_OUT", tmp)
        path, _ = model_dir(cfg, 5, tmp)
        from lily_b200 import SamplingParams
        eng = engine(path, "bfloat16", max_total_tokens=1024)
        prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], n) for n in (20, 33, 41)]
        eng.generate(prompts, SamplingParams(max_new_tokens=16, ignore_eos=True))
        table = eng.runner.profiler.tables[3]
        assert open(os.path.join(tmp, "decode_step_bs3.txt")).read().strip() == table.strip()
    lines = table.splitlines()
    assert "batch 3" in lines[0] and "over 6 steps" in lines[0]
    assert any("attention_mma_kernel" in ln for ln in lines) and any("add_rmsnorm" in ln for ln in lines)
    per_step = float(lines[2].split()[0])
    assert 10 < per_step < 5000                     # microseconds of device time a step


def test_a_long_request_beside_short_ones_through_the_engine():
    """A prompt of more than 16 k positions beside short ones (context 40 k, 8 kv heads): the scheduler's decode steps
    take the graphs of the long request's class of sequence length while it is among them (its attention one full wave
    of key ranges) and those of the first class for the short ones alone, and every generated token is still the
    prefill path's argmax."""
    from lily_b200 import SamplingParams
    from lily_b200.bench.check_greedy import check_greedy
    cfg = dict(tiny_models.MID_QWEN3, num_attention_heads=8, num_key_value_heads=8, max_position_embeddings=40000)
    with tempfile.TemporaryDirectory() as tmp:
        path, _ = model_dir(cfg, 65, tmp)
        from lily_b200 import Engine, EngineConfig
        eng = Engine(EngineConfig(path, dtype="bfloat16", max_total_tokens=24000, max_running_requests=4, context_length=40000))
        prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 400 + n) for n in (300, 16500, 40)]
        outs = [o["output_ids"] for o in eng.generate(prompts, SamplingParams(max_new_tokens=32, ignore_eos=True))]
        report = check_greedy(eng, prompts, outs)
        long_classes = sorted({cls for _, cls, _ in eng.runner._graphs})
        short = [prompts[0], prompts[2]]                   # the short ones alone: the first class's graphs
        again = [o["output_ids"] for o in eng.generate(short, SamplingParams(max_new_tokens=32, ignore_eos=True))]
        classes = sorted({cls for _, cls, _ in eng.runner._graphs})
    assert report["tokens"] == 3 * 32 and report["max_gap"] < 3e-2, report
    assert long_classes == [32768] and classes == [8192, 32768], (long_classes, classes)
    # beside the long request or alone, through either class of graphs: the same tokens up to near-ties
    assert sum(a != b for x, y in zip(again, (outs[0], outs[2])) for a, b in zip(x, y)) <= 2


def test_many_rows_of_one_length_take_whole_rows_and_uneven_ones_keep_their_ranges():
    """32 requests over 8 kv heads: while they are about equally long a block of the decode attention takes a whole
    row (three stages, no scratch), and with one much longer request among them the rows keep their key ranges; each
    kind of batch has its own graph, and every generated token is the prefill path's argmax either way."""
    from lily_b200 import Engine, EngineConfig, SamplingParams
    from lily_b200.bench.check_greedy import check_greedy
    from lily_b200.csrc import ops
    if not ops._WHOLE_ROWS:
        pytest.skip("whole rows are switched off")
    cfg = dict(tiny_models.MID_QWEN3, num_attention_heads=16, num_key_value_heads=8)
    even = ops.plan_decode_attention(torch.bfloat16, 32, 16, 8, 128, 8192, even=True)
    uneven = ops.plan_decode_attention(torch.bfloat16, 32, 16, 8, 128, 8192)
    assert (even.arm, even.splits, even.stages, even.scratch_floats, even.fused) == ("whole rows", 1, 3, 0, True)
    assert uneven.arm == "wave" and uneven.splits > 1 and uneven.stages == 0
    with tempfile.TemporaryDirectory() as tmp:
        path, _ = model_dir(cfg, 66, tmp)
        eng = Engine(EngineConfig(path, dtype="bfloat16", max_total_tokens=32 * 512 + 2048, max_running_requests=32))
        prompts = [tiny_models.random_tokens(190 + n % 7, cfg["vocab_size"], 500 + n) for n in range(32)]
        outs = [o["output_ids"] for o in eng.generate(prompts, SamplingParams(max_new_tokens=24, ignore_eos=True))]
        report = check_greedy(eng, prompts, outs)
        cls = eng.runner.length_classes[0]
        kinds = sorted(k for k in eng.runner._graphs if k[0] == 32)
        assert kinds == [(32, cls, True)] and eng.runner._graphs[kinds[0]].even_matters, kinds
        prompts[5] = tiny_models.random_tokens(700, cfg["vocab_size"], 77)
        outs2 = [o["output_ids"] for o in eng.generate(prompts, SamplingParams(max_new_tokens=24, ignore_eos=True))]
        report2 = check_greedy(eng, prompts, outs2)
        kinds2 = sorted(k for k in eng.runner._graphs if k[0] == 32)
    assert report["tokens"] == 32 * 24 and report["max_gap"] < 3e-2, (report, [len(o) for o in outs])
    assert report2["tokens"] == 32 * 24 and report2["max_gap"] < 3e-2, (report2, [len(o) for o in outs2])
    assert kinds2 == [(32, cls, False), (32, cls, True)], kinds2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generated_tokens_are_the_prefill_paths_argmax(dtype):
    """What the decode path generated (graphs, split-key attention, the decode products) against one teacher-forced
    pass of the prefill path over the same tokens (lily_b200/bench/check_greedy.py): in float32 every token is the
    argmax up to rounding, in bfloat16 a token may differ only where the two best logits are nearly tied."""
    from lily_b200 import SamplingParams
    from lily_b200.bench.check_greedy import check_greedy
    cfg = tiny_models.MID_QWEN3
    with tempfile.TemporaryDirectory() as tmp:
        path, _ = model_dir(cfg, 64, tmp)
        eng = engine(path, dtype, max_total_tokens=4096)
        prompts = [tiny_models.random_tokens(n, cfg["vocab_size"], 300 + n) for n in (5, 130, 200, 64, 333)]
        outs = [o["output_ids"] for o in eng.generate(prompts, SamplingParams(max_new_tokens=48, ignore_eos=True))]
        report = check_greedy(eng, prompts, outs)
    assert report["tokens"] == 5 * 48
    assert report["max_gap"] < (1e-4 if dtype == "float32" else 3e-2), report
