"""The plain implementation against the reference's own outputs (tests/golden) and against itself."""

import os

import pytest
import torch
from safetensors.torch import load_file

import plain_impl
import tiny_models
from golden.make_golden import SEEDS

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(tiny_models.CONFIGS))
def test_plain_matches_reference_outputs(name):
    cfg = tiny_models.CONFIGS[name]
    gold = load_file(os.path.join(GOLDEN, f"{name}.safetensors"))
    weights = tiny_models.make_weights(cfg, SEEDS[name])
    logits = plain_impl.all_logits(cfg, weights, gold["ids"].tolist())
    assert logits.shape == gold["logits"].shape
    assert float((logits - gold["logits"]).abs().max()) < 5e-6


def test_causality_and_window():
    torch.manual_seed(0)
    q, k, v = torch.randn(12, 4, 16), torch.randn(12, 2, 16), torch.randn(12, 2, 16)
    full = plain_impl.causal_attention(q, k, v, 0.25)
    # a position's output does not depend on later keys
    part = plain_impl.causal_attention(q[:7], k[:7], v[:7], 0.25)
    assert torch.allclose(full[:7], part, atol=1e-6)
    # a window as long as the sequence changes nothing; a window of 1 returns v itself
    assert torch.allclose(plain_impl.causal_attention(q, k, v, 0.25, window=12), full, atol=1e-6)
    one = plain_impl.causal_attention(q, k, v, 0.25, window=1)
    assert torch.allclose(one, v.repeat_interleave(2, dim=1), atol=1e-6)


def test_llama3_scaling_bands():
    inv = plain_impl.rope_inv_freq(32, 500000.0)
    out = plain_impl.llama3_inv_freq(inv, 8.0, 1.0, 4.0, 64)
    wavelen = 2 * torch.pi / inv
    assert torch.equal(out[wavelen < 16], inv[wavelen < 16])
    assert torch.allclose(out[wavelen > 64], inv[wavelen > 64] / 8.0)
    mid = (wavelen >= 16) & (wavelen <= 64)
    assert bool(((out[mid] <= inv[mid]) & (out[mid] >= inv[mid] / 8.0)).all())


def test_sampling_reference():
    torch.manual_seed(1)
    x = torch.randn(50)
    p = plain_impl.filtered_probs(x, 0.7)
    assert torch.allclose(p, torch.softmax(x / 0.7, -1), atol=1e-6)
    p = plain_impl.filtered_probs(x, 1.0, top_k=5)
    assert int((p > 0).sum()) == 5 and abs(float(p.sum()) - 1) < 1e-6
    p = plain_impl.filtered_probs(x, 1.0, top_p=0.5)
    s = torch.sort(torch.softmax(x, -1), descending=True).values
    n = int((torch.cumsum(s, 0) - s < 0.5).sum())
    assert int((p > 0).sum()) == n
    assert plain_impl.inverse_cdf_pick(torch.tensor([0.0, 0.25, 0.0, 0.75]), 0.2) == 1
    assert plain_impl.inverse_cdf_pick(torch.tensor([0.0, 0.25, 0.0, 0.75]), 0.25) == 3
    y = plain_impl.penalised(torch.tensor([1.0, -1.0, 2.0, 0.5]), [0, 1, 1], repetition=2.0, frequency=0.1,
                             presence=0.5, bias={3: 1.0})
    assert torch.allclose(y, torch.tensor([0.5 - 0.1 - 0.5, -2.0 - 0.2 - 0.5, 2.0, 1.5]))
