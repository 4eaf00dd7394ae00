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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_qwen3", "tiny_llama"])
def test_replay_mixed_trace(name, dtype):
    cfg = tiny_models.CONFIGS[name]
    v = cfg["vocab_size"]
    with tempfile.TemporaryDirectory() as tmp:
        path, weights = model_dir(cfg, 71, tmp)
        reqs = {k: tiny_models.random_tokens(n, v, 120 + i) for i, (k, n) in enumerate(
            {"a": 100, "b": 70, "c": 64, "d": 90, "e": 40}.items())}
        # up to four live; portions beside decoded tokens; ends free pages that later requests reuse
        plan = [({"a": 60}, []), ({"a": 1, "b": 33}, []), ({"a": 1, "b": 2, "c": 64}, []), ({"b": 35, "a": 1, "d": 5}, ["c"]),
                ({"a": 37, "d": 2}, ["b"]), ({"d": 83, "e": 3}, ["a"]), ({"e": 1}, ["d"]), ({"e": 36}, ["e"])]
        steps, done, where = [], {k: 0 for k in reqs}, {k: [] for k in reqs}
        for i, (step, end) in enumerate(plan):
            entries = []
            for k, n in step.items():
                toks = reqs[k][done[k]:done[k] + n]
                want = list(range(len(toks))) if k != "c" else [len(toks) - 1, 0]
                entries.append({"id": k, "tokens": toks, "want": want})
                where[k].append((i, done[k], want))
                done[k] += len(toks)
            steps.append({"step": i, "entries": entries, "end": end})
        # live tokens, each request rounded up to 64, peak at steps 3 to 5: 128 + 64 + 64 + 64 = 320, five pages of 64
        rows = replay(path, dtype, steps, 320, tmp, v)
        plain = {k: plain_impl.all_logits(cfg, rounded(weights, dtype), ids) for k, ids in reqs.items()}
        for i, s in enumerate(steps):
            at = 0
            for e in s["entries"]:
                k = e["id"]
                start = [w for w in where[k] if w[0] == i][0][1]
                for w in e["want"]:
                    close(rows[i][at:at + 1], plain[k][start + w:start + w + 1], dtype, f"step {i} request {k} place {w}")
                    at += 1


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
