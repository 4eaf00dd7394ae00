"""bin/trace_run as a user runs it: a subprocess with an empty HOME, steps on standard input,
logits read back from the files it writes."""

import json
import os
import subprocess
import tempfile

import numpy as np
import pytest
import torch

import plain_impl
import tiny_models
from harness import model_dir
from test_engine_gpu import close, rounded

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(path, dtype, steps, max_tokens, tmp, vocab):
    out_dir = os.path.join(tmp, f"out_{dtype}_{len(steps)}")
    home = os.path.join(tmp, "home")
    os.makedirs(home, exist_ok=True)
    env = dict(os.environ, HOME=home)
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", out_dir,
                           "--max-tokens", str(max_tokens)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == [f"done {s['step']}" for s in steps]
    rows = {}
    for s in steps:
        f = os.path.join(out_dir, f"{s['step']}.f32")
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        assert os.path.exists(f) == (wanted > 0)
        if wanted:
            rows[s["step"]] = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(wanted, vocab).copy())
    return rows


class Trace:
    """Builds the steps of a replay and remembers which logits each step's file should hold."""

    def __init__(self, requests):
        self.requests, self.done = requests, {k: 0 for k in requests}
        self.steps, self.expect = [], []         # expect[i]: (request, position) of each wanted row of step i

    def step(self, portions, end=(), want=None):
        """``portions``: request -> how many of its next tokens; every place is wanted unless ``want`` gives, per
        request, the places among the portion's tokens."""
        entries, rows = [], []
        for k, n in portions.items():
            toks = self.requests[k][self.done[k]:self.done[k] + n]
            places = list(range(len(toks))) if want is None or k not in want else list(want[k])
            entries.append({"id": k, "tokens": toks, "want": places})
            rows += [(k, self.done[k] + w) for w in places]
            self.done[k] += len(toks)
        self.steps.append({"step": len(self.steps), "entries": entries, "end": list(end)})
        self.expect.append(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_qwen3", "tiny_llama", "odd_qwen3", "odd_llama"])
def test_replay_in_every_cutting(name, dtype):
    """One trace through the tool: a request whole; one with its last 32 tokens one by one; one in portions of
    changing size down to two tokens; then up to four live requests, portions of some beside decoded tokens of
    others, ends that free pages which later requests take.  The pool holds 320 tokens, so pages are used again
    from the second request on."""
    cfg = tiny_models.CONFIGS[name]
    v = cfg["vocab_size"]
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 71, tmp)
        reqs = {k: tiny_models.random_tokens(n, v, 120 + i) for i, (k, n) in enumerate(
            {"w": 150, "t": 140, "p": 131, "a": 100, "b": 70, "c": 64, "d": 90, "e": 40}.items())}
        t = Trace(reqs)
        t.step({"w": 150}, end=["w"])
        t.step({"t": 108})
        for i in range(32):
            t.step({"t": 1}, end=["t"] if i == 31 else [])
        for i, n in enumerate([8, 2, 30, 17, 2, 3, 40, 2, 5, 22]):
            t.step({"p": n}, end=["p"] if i == 9 else [])
        t.step({"a": 60})
        t.step({"a": 1, "b": 33})
        t.step({"a": 1, "b": 2, "c": 64}, want={"c": [63, 0]})
        t.step({"b": 35, "a": 1, "d": 5}, end=["c"])
        t.step({"a": 37, "d": 2}, end=["b"])
        t.step({"d": 83, "e": 3}, end=["a"])
        t.step({"e": 1}, end=["d"])
        t.step({"e": 36}, end=["e"])
        assert all(t.done[k] == len(ids) for k, ids in reqs.items())
        # live tokens, each request rounded up to 64: 192 at most while one request lives, and in the mixed part
        # 128 + 64 + 64 + 64 = 320 at its peak: five pages of 64
        rows = replay(path, dtype, t.steps, 320, tmp, v)
        plain = {k: plain_impl.all_logits(cfg, rounded(weights, dtype), ids) for k, ids in reqs.items()}
        for i, expect in enumerate(t.expect):
            want = torch.stack([plain[k][pos] for k, pos in expect])
            close(rows[i], want, dtype, f"step {i} ({', '.join(sorted({k for k, _ in expect}))})")


def test_replay_past_the_files_max_position():
    """A request of 300 tokens through a model whose config.json says max_position_embeddings 256: the pool
    (--max-tokens) bounds a request, not that number."""
    cfg = tiny_models.CONFIGS["tiny_qwen3"]
    v = cfg["vocab_size"]
    assert cfg["max_position_embeddings"] == 256
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 72, tmp)
        ids = tiny_models.random_tokens(300, v, 9)
        steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:268], "want": [267]}], "end": []}] + \
                [{"step": i, "entries": [{"id": "a", "tokens": ids[267 + i:268 + i], "want": [0]}], "end": []} for i in range(1, 33)]
        rows = replay(path, "float32", steps, 320, tmp, v)
        got = torch.cat([rows[i] for i in range(33)])
        close(got, plain_impl.all_logits(cfg, weights, ids)[267:], "float32", "positions 267 to 299")
