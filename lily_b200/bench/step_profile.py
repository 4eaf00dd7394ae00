"""Where a decode step's time goes at the benchmark's sizes, from inside the running engine.

    python -m lily_b200.bench.step_profile --batch 1 8 [--context 4096] [--layers 36] [--steps 20] [--out DIR]

Builds the Qwen3-8B layer sizes with seeded random weights, runs ``--batch`` requests to just below
``--context`` positions through ``Engine`` (scheduler, overlap schedule, CUDA graphs: what serving
runs), and lets the engine's own step profiler (``lily_b200/engine/profiler.py``,
``LILY_B200_PROFILE_BS``) record ``--steps`` decode steps at each batch size.  Prints each table and,
with ``--out``, writes it to ``DIR/decode_step_bs<N>.txt``; a closing line relates the kernels'
summed device time to the bytes a step has to read (every weight once, the live requests' cache).
For figures to quote, give the batch sizes in rising order or one a process: a window that follows a larger
batch's in the same process has read every kernel 10 to 25 % slower than the same step timed with CUDA events
(batch 12 behind batch 16: 5.06 against 4.38 ms), which the steps themselves, timed without the profiler, are not.
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 8])
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()

    os.environ["LILY_B200_PROFILE_BS"] = ",".join(str(b) for b in a.batch)
    os.environ["LILY_B200_PROFILE_STEPS"] = str(a.steps)
    if a.out:
        os.environ["LILY_B200_PROFILE_OUT"] = a.out

    import torch

    from lily_b200.config.server_args import ServerArgs
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.engine.runner import ModelRunner
    from lily_b200.sampling.params import SamplingParams

    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": a.layers, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
           "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
           "max_position_embeddings": a.context, "hidden_act": "silu", "torch_dtype": "bfloat16"}
    most = max(a.batch)
    args = ServerArgs(dtype="bfloat16", device="cuda:0", context_length=a.context, page_size=64,
                      max_total_tokens=most * (a.context + 64), max_running_requests=most, random_seed=0)
    runner = ModelRunner.from_random(cfg, seed=0, args=args)
    eng = Engine(EngineConfig("<random>", dtype="bfloat16", device="cuda:0", context_length=a.context,
                              max_running_requests=most, server_args={"page_size": 64, "random_seed": 0}), runner=runner)
    g = torch.Generator().manual_seed(1)
    h, layers = cfg["hidden_size"], a.layers
    weights = 2 * (layers * (h * (32 + 16) * 128 + 32 * 128 * h + 3 * h * cfg["intermediate_size"]) + cfg["vocab_size"] * h)
    for batch in a.batch:
        # the first request decodes while the later ones are still being admitted, a portion of prompts a step:
        # it must still be there when the last one has joined and the window has passed
        new_tokens = a.steps + 12 + -(-batch * a.context // args.chunked_prefill_size)
        prompts = [torch.randint(0, cfg["vocab_size"], (a.context - new_tokens - 1,), generator=g).tolist() for _ in range(batch)]
        eng.generate(prompts, SamplingParams(max_new_tokens=new_tokens, ignore_eos=True))
        table = runner.profiler.tables.get(batch)
        if table is None:
            print(f"no window at batch {batch} (the requests did not decode side by side for {a.steps} steps)", file=sys.stderr)
            continue
        print(table)
        us = float(table.splitlines()[2].split()[0])
        step_bytes = weights + batch * (a.context - new_tokens / 2) * 2 * 8 * 128 * 2 * layers
        print(json.dumps({"batch": batch, "kernels_us_per_step": us, "bytes_per_step": int(step_bytes),
                          "GB/s_over_kernel_time": round(step_bytes / us / 1e3, 1)}))
        print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
