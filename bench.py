"""Measures the engine on one B200: decode tokens a second at batch 8 (and 1, 64) and prefill
tokens a second at 2,048 tokens, for the Qwen3-8B layer sizes with random weights in bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints one JSON line.  A step is one decode step of the whole batch.  ``value`` times K steps of
the engine's step function plus the sampler on the device (CUDA events, W untimed steps first);
``e2e`` times the same number of tokens through ``Engine.generate`` (scheduler, host token lists in,
host token lists out).  The method is the reference's own (bench/bench.py:104-172 there: random
ids, a batched prefill, warm-up and timed decode steps).  The weights (15 GB) are larger than the
126 MB L2, so nothing is flushed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
FULL_LAYERS = 36
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out, source = dict(FALLBACK_PEAKS), "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(raw)
            for k in out:
                if k in flat:
                    out[k] = flat[k]
                    source = "measured"
        except (OSError, ValueError):
            pass
    out["source"] = source
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(int(float(parts[0])))
                mx = max(mx, int(float(parts[1])))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def gemm_params(cfg, layers):
    h, nq, nkv, d, i = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                        cfg["intermediate_size"])
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i
    return per_layer * layers, cfg["vocab_size"] * h


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "CodeMan62/lily does not install offline here: its build backend (hatchling) is not in "
                          "the wheelhouse and its scheduler imports pyzmq, which is not installed"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2

    import torch

    from lily_b200.config.server_args import ServerArgs
    from lily_b200.csrc import ops
    from lily_b200.engine.batch import StepEntry
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.engine.runner import ModelRunner
    from lily_b200.sampling.params import SamplingParams

    warmup = max(3, a.warmup)
    steps = max(1, a.steps)
    cfg = dict(QWEN3_8B, num_hidden_layers=a.layers)
    pk = peaks()
    torch.cuda.set_device(0)
    max_batch = max(a.batch, 8 if a.skip_points else 64)
    args = ServerArgs(dtype="bfloat16", device="cuda:0", context_length=CONTEXT, page_size=64,
                      max_total_tokens=max_batch * CONTEXT + 4 * 64 * max_batch, max_running_requests=max_batch,
                      chunked_prefill_size=8192, max_prefill_tokens=16384, random_seed=0)
    t0 = time.time()
    runner = ModelRunner.from_random(cfg, seed=0, args=args)
    load_s = time.time() - t0
    vocab = cfg["vocab_size"]
    g = torch.Generator().manual_seed(1)

    def ids(n):
        return torch.randint(0, vocab, (n,), generator=g).tolist()

    def timed(fn, reps, warm):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps

    # ---- prefill: one request of 2,048 tokens ------------------------------------------
    prompt = ids(PREFILL_TOKENS)

    def prefill_once():
        slot = runner.open_request()
        runner.step([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        runner.close_request(slot)

    prefill_ms = timed(prefill_once, 5, 3)
    layer_params, head_params = gemm_params(cfg, a.layers)
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    attn_flops = 2 * 2 * nq * d * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2) * a.layers
    prefill_flops = 2 * PREFILL_TOKENS * layer_params + 2 * head_params + attn_flops
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode: batch B, contexts ending at 4,096 --------------------------------------
    def decode_point(batch, k, w):
        start_len = CONTEXT - (k + w) - 1
        slots = [runner.open_request() for _ in range(batch)]
        for s in slots:                                  # prompts go in whole, a few requests per step
            runner.step([StepEntry(s, ids(start_len), [])])
        tokens = [ids(1)[0] for _ in range(batch)]
        state = {"tokens": tokens}

        def one():
            logits = runner.step([StepEntry(s, [t], [0]) for s, t in zip(slots, state["tokens"])])
            state["tokens"] = ops.argmax(logits).tolist()
        l0 = ops.launches["count"]
        for _ in range(w):
            one()
        torch.cuda.synchronize()
        l1 = ops.launches["count"]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as clocks:
            e0.record()
            for _ in range(k):
                one()
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / k
        launches = ops.launches["count"] - l1
        mean_ctx = start_len + w + (k + 1) / 2
        for s in slots:
            runner.close_request(s)
        return ms, launches, mean_ctx, clocks.summary()

    ms, launches, mean_ctx, clocks = decode_point(a.batch, steps, warmup)
    value = a.batch / ms * 1e3
    kv_bytes_tok = 2 * cfg["num_key_value_heads"] * d * 2 * a.layers
    weight_bytes = 2 * (layer_params + head_params)
    step_bytes = weight_bytes + a.batch * mean_ctx * kv_bytes_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            pms, _, _, _ = decode_point(b, min(steps, 32), warmup)
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)

    # ---- end to end: the Python entry point, host tokens in and out ---------------------
    eng = Engine(EngineConfig("<random>", dtype="bfloat16", device="cuda:0", context_length=CONTEXT,
                              max_running_requests=max_batch,
                              server_args={"page_size": 64, "random_seed": 0, "chunked_prefill_size": 8192}), runner=runner)
    # requests admitted first decode a few tokens while the others' prompts go in: leave them room,
    # so that all of the batch is still decoding when the timed steps end
    slack = 2 * a.batch
    e2e_prompt = CONTEXT - (steps + warmup) - slack
    prompts = [ids(e2e_prompt) for _ in range(a.batch)]
    sched = eng.new_scheduler()
    for i, p in enumerate(prompts):
        sched.add_request(f"b{i}", p, SamplingParams(max_new_tokens=steps + warmup + slack, ignore_eos=True))
    guard = 0
    while (sched.waiting_queue or len(sched.running) < a.batch) and guard < 10000:   # prompts in; first tokens sampled
        sched.step()
        guard += 1
    for _ in range(warmup - 1):
        sched.step()
    torch.cuda.synchronize()
    t_start = time.perf_counter()
    done, stamps, graph_before = 0, [], runner.graph_steps
    while done < steps and sched.running:
        sched.step()
        done += 1
        stamps.append(time.perf_counter())
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t_start) * 1e3 / max(done, 1)
    gaps = sorted((b - a) * 1e3 for a, b in zip([t_start] + stamps[:-1], stamps))
    print(f"e2e: {done} steps, {runner.graph_steps - graph_before} through graphs, running {len(sched.running)}, "
          f"per-step ms min {gaps[0]:.2f} median {gaps[len(gaps) // 2]:.2f} max {gaps[-1]:.2f}", file=sys.stderr)
    sched.run_to_completion()
    meta_ints = 3 * a.batch + 4 * a.batch + 1 + a.batch + a.batch * (CONTEXT // 64)
    e2e = {"value": round(a.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * meta_ints,
           "d2h_bytes_per_step": 4 * a.batch}

    out = {
        "metric": "decode tokens/s, Qwen3-8B sizes bf16, batch %d, context 4096" % a.batch,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02), token ids uniform in [0, vocab)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B sizes", "layers": a.layers, "layers_of_model": FULL_LAYERS, "hidden": 4096,
                   "q_heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": vocab,
                   "global_batch": a.batch, "seq_len": CONTEXT, "context_start": int(CONTEXT - steps - 1),
                   "page_size": 64, "parallelism": "single GPU", "l2": "inputs larger than L2 (15 GB of weights)",
                   "peaks": pk["source"], "load_s": round(load_s, 1)},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
