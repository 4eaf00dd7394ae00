"""Decode step time over batch sizes at one context length, against the byte floor of each step.

    python -m lily_b200.bench.batch_sweep --context 4096 --batch 1 2 4 8 16 32 64 128
    python -m lily_b200.bench.batch_sweep --context 16384 --batch 1 8 32

Qwen3-8B sizes with seeded random weights (``bench.py``'s model; ``--layers`` for fewer, which the output names).
Every batch size prefills its requests to just short of the context and then runs decode steps of the step function
on tokens that stay on the device (the argmax kernel's result feeds the next step), through CUDA graphs as in
serving; CUDA events around 16 steps, the median of three rounds.  The floor of a step is every weight once plus the
keys and values of the live requests, over the measured copy bandwidth.  One JSON line per batch size.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 2, 4, 8, 16, 32, 64, 128])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in the output)")
    ap.add_argument("--steps", type=int, default=16)
    a = ap.parse_args()

    import torch

    import bench
    from lily_b200.config.server_args import ServerArgs
    from lily_b200.csrc import ops
    from lily_b200.engine.batch import FUTURE, StepEntry
    from lily_b200.engine.runner import ModelRunner

    cfg = dict(bench.QWEN3_8B, max_position_embeddings=max(a.context, bench.QWEN3_8B.get("max_position_embeddings", 0)))
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    layers = cfg["num_hidden_layers"]
    pk = bench.peaks()
    torch.cuda.set_device(0)
    most = max(a.batch)
    args = ServerArgs(dtype="bfloat16", device="cuda:0", context_length=a.context, page_size=64,
                      max_total_tokens=most * a.context + 4 * 64 * most, max_running_requests=most,
                      chunked_prefill_size=8192, max_prefill_tokens=16384, random_seed=0)
    runner = ModelRunner.from_random(cfg, seed=0, args=args)
    g = torch.Generator().manual_seed(1)
    ids = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
    layer_params, head_params = bench.gemm_params(cfg, layers)
    kv_bytes_tok = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * layers

    def timed(fn, reps):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps

    warm, rounds = 4, 3
    for b in a.batch:
        total = warm + rounds * a.steps
        start_len = a.context - total - 2
        slots = [runner.open_request() for _ in range(b)]
        for s in slots:                                      # prompts in portions of up to 8,192 tokens
            prompt, done = ids(start_len), 0
            while done < start_len:
                n = min(8192, start_len - done)
                runner.step([StepEntry(s, prompt[done:done + n], [])])
                done += n
        runner.store_future(ops.argmax(runner.step([StepEntry(s, [ids(1)[0]], [0]) for s in slots])))
        entries = [StepEntry(s, [FUTURE], [0]) for s in slots]
        one = lambda: runner.store_future(ops.argmax(runner.step(entries)))
        for _ in range(warm):
            one()
        ms = statistics.median(timed(one, a.steps) for _ in range(rounds))
        torch.cuda.synchronize()
        for s in slots:
            runner.close_request(s)
        mean_ctx = start_len + 1 + warm + (rounds * a.steps + 1) / 2
        floor_ms = (2 * (layer_params + head_params) + b * mean_ctx * kv_bytes_tok) / (pk["hbm_gbs"] * 1e9) * 1e3
        print(json.dumps({"context": a.context, "batch": b, "layers": layers, "ms_per_step": round(ms, 3),
                          "tokens_per_s": round(b / ms * 1e3, 1), "floor_ms": round(floor_ms, 3),
                          "hbm_frac": round(floor_ms / ms, 3), "peaks": pk["source"]}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
