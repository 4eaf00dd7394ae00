"""The engine at the layer sizes of the benchmark configurations (Qwen3-8B, Llama-3.1-8B, Qwen3-32B), with two
layers each, against the plain implementation evaluated on the device in float64: float32 (bound 1e-4 on logits
up to 7) and bfloat16 (bounds relative to the largest logit), in every way of cutting the work.  The weights are
the engine's own random-weights mode on the device; the plain implementation gets the same tensors by name.

The reference holds its engine to a library model on real checkpoints of its sizes (tests/test_engine.py:68-84
there); without checkpoints, the layer sizes with random weights are what can be held here.
"""

import pytest
import torch

import plain_impl
import tiny_models
from lily_b200.config.registry import resolve_architecture
from lily_b200.config.server_args import ServerArgs
from lily_b200.engine.batch import StepEntry
from lily_b200.engine.runner import ModelRunner
from lily_b200.weights.random_init import RandomSource, expected_tensors

pytestmark = pytest.mark.gpu

LAYERS = 2          # of 36, 32 and 64: the layer sizes are the configurations', the depth is not
SIZES = {
    "qwen3_8b": {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": LAYERS, "hidden_size": 4096,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
        "max_position_embeddings": 4096, "hidden_act": "silu"},
    "llama31_8b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": LAYERS, "hidden_size": 4096,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
        "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192, "hidden_act": "silu"},
    "qwen3_32b": {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": LAYERS, "hidden_size": 5120,
        "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 25600,
        "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
        "max_position_embeddings": 16384, "hidden_act": "silu"},
}
BOUNDS = {"float32": (1e-4, 1e-5, False), "bfloat16": (2e-2, 3e-3, True)}       # max, mean, relative to the largest logit


def check(got, want, dtype, what):
    top, mean, relative = BOUNDS[dtype]
    err = (got.double() - want).abs()
    scale = float(want.abs().max()) if relative else 1.0
    assert float(err.max()) < top * scale, f"{what}: max error {float(err.max()):.3e} (logits up to {float(want.abs().max()):.2f})"
    assert float(err.mean()) < mean * scale, f"{what}: mean error {float(err.mean()):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", sorted(SIZES))
def test_layer_sizes_of_the_benchmark_configurations(size, dtype):
    cfg = dict(SIZES[size], torch_dtype=dtype)
    v = cfg["vocab_size"]
    args = ServerArgs(dtype=dtype, device="cuda", context_length=1024, page_size=64, max_total_tokens=12 * 64,
                      max_running_requests=4)
    runner = ModelRunner.from_random(cfg, seed=7, args=args, gain_jitter=0.05)
    arch = resolve_architecture(cfg["architectures"])
    config = arch.config_from_dict(cfg, {}, architecture=arch.name)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    source = RandomSource(expected_tensors(config, arch), 7, store, "cuda", 0.02, 0.05)
    weights = {name: source.get(name) for name in source.specs}          # the engine's tensors, by checkpoint name

    def plain(ids):
        with plain_impl.precision(torch.float64):
            return plain_impl.all_logits(cfg, weights, ids)

    def step(entries):
        return runner.step([StepEntry(slot, toks, list(range(len(toks)))) for slot, toks in entries])

    def portions(ids, cuts):
        slot, rows, done = runner.open_request(), [], 0
        for n in list(cuts) + [len(ids)]:
            n = min(n, len(ids) - done)
            if n > 0:
                rows.append(step([(slot, ids[done:done + n])]).clone())
                done += n
        runner.close_request(slot)
        return torch.cat(rows)

    a = tiny_models.random_tokens(300, v, 1)
    want = plain(a)
    check(portions(a, [300]), want, dtype, "whole")
    check(portions(a, [268] + [1] * 32), want, dtype, "last 32 one by one")
    check(portions(a, [130, 2, 65, 3, 40, 2, 17]), want, dtype, "portions")
    # mixed: four live requests, portions of some beside decoded tokens of others, over 12 pages of 64: what "b"
    # gives back when it ends is what "d" takes
    reqs = {"a": a, "b": tiny_models.random_tokens(120, v, 2), "c": tiny_models.random_tokens(190, v, 3),
            "d": tiny_models.random_tokens(128, v, 4)}
    plan = [({"a": 140, "b": 50}, []), ({"a": 1, "b": 68, "c": 2}, []), ({"a": 1, "b": 2, "c": 150}, ["b"])] + \
           [({"a": 1, "c": 1, "d": 8}, [])] * 16 + [({"a": 142, "c": 22}, [])]
    slots, done, rows = {}, {k: 0 for k in reqs}, {k: [] for k in reqs}
    for portion, ends in plan:
        entries, names = [], []
        for k, n in portion.items():
            slots.setdefault(k, None)
            if slots[k] is None:
                slots[k] = runner.open_request()
            toks = reqs[k][done[k]:done[k] + n]
            if toks:
                entries.append((slots[k], toks))
                names.append(k)
                done[k] += len(toks)
        out, at = step(entries), 0
        for k, (_, toks) in zip(names, entries):
            rows[k].append(out[at:at + len(toks)].clone())
            at += len(toks)
        for k in ends:
            runner.close_request(slots.pop(k))
    for k in list(slots):
        runner.close_request(slots.pop(k))
    assert done == {k: len(ids) for k, ids in reqs.items()}
    for k, ids in reqs.items():
        check(torch.cat(rows[k]), want if k == "a" else plain(ids), dtype, f"mixed, request {k}")
    assert runner.graph_steps >= 32 and runner.cache.held_pages() == [0]
