"""Measures the engine on one B200: decode tokens a second at batch 8 (and 1, 64) and prefill
tokens a second at 2,048 tokens, for the Qwen3-8B layer sizes with random weights in bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints one JSON line.  A step is one decode step of the whole batch.  After W untimed steps, ``value``
times K steps of the engine's step function plus the argmax kernel on the device (CUDA events; the tokens
stay on the device from step to step) and
``e2e`` times K steps of the scheduler behind ``Engine`` on the host (token lists in, token lists out,
the overlap schedule as in serving), in alternating rounds (medians are reported) under one record of
the SM clocks, sampled through NVML every 10 ms and tagged by region; ``e2e.host_ms_per_step`` is what
the host itself spends on a step.  ``--impl reference`` measures the unmodified reference the same way
(``baseline/reference_arm.py``).  The method is the reference's own (bench/bench.py:104-172 there:
random ids, a batched prefill, warm-up and timed decode steps).  The weights (15 GB) are larger than
the 126 MB L2, so nothing is flushed between steps.
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
    """Samples SM clocks and throttle reasons while regions are timed: through NVML in a thread (a sample every
    10 ms, each tagged with the region the timing loop says it is in), else with nvidia-smi every 100 ms.
    Reading only; nothing of the GPU is set."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []            # (region, sm MHz, reasons bit mask)
        self.region = "idle"
        self.max_mhz = 0
        self._stop = threading.Event()
        self._thread = None
        self._proc = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            first = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].strip() or "0"
            self._handle = (pynvml.nvmlDeviceGetHandleByIndex(int(first)) if first.isdigit()
                            else pynvml.nvmlDeviceGetHandleByUUID(first.encode()))
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
            try:
                self._proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                               "--format=csv,noheader,nounits", "-lms", "100"],
                                              stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self._thread = threading.Thread(target=self._read_smi, daemon=True)
                self._thread.start()
            except OSError:
                self._proc = None
        return self

    def _poll_nvml(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                self.samples.append((self.region, mhz, mask))
            except Exception:
                pass
            self._stop.wait(0.01)

    def _read_smi(self):
        names = list(self.REASONS)
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz = int(float(parts[0]))
                self.max_mhz = max(self.max_mhz, int(float(parts[1])))
            except ValueError:
                continue
            mask = sum(self.REASONS[n] for n, v in zip(names, parts[2:6]) if v.lower().startswith("active"))
            self.samples.append((self.region, mhz, mask))

    def __exit__(self, *exc):
        self._stop.set()
        if self._proc is not None:
            time.sleep(0.15)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        elif self._thread is not None:
            self._thread.join(timeout=1)

    def summary(self, region=None):
        """Median SM MHz, the highest clock the device offers, the throttle reasons seen, and the number of samples,
        over the samples of one region (default: all that were taken inside any named region)."""
        rows = [s for s in self.samples if (s[0] == region if region else s[0] != "idle")]
        mhz = [s[1] for s in rows]
        seen = 0
        for s in rows:
            seen |= s[2]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": self.max_mhz or None,
                "reasons": sorted(n for n, bit in self.REASONS.items() if seen & bit), "samples": len(mhz)}


def gemm_params(cfg, layers):
    h, nq, nkv, d, i = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                        cfg["intermediate_size"])
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i
    return per_layer * layers, cfg["vocab_size"] * h


def rounds_for(steps: int, step_ms: float = 4.2) -> int:
    """Rounds of ``steps`` device-timed and ``steps`` host-timed steps in turn: enough for about a second of load
    (so that the clocks settle under the power cap and are sampled), within the room the context leaves."""
    want = -(-1000 // int(2 * steps * step_ms))
    return max(3, min(12, want, max(1, 600 // steps)))


def json_line(a, cfg, pk, *, impl, ms, e2e, launches, clocks, prefill_ms, mean_ctx, points, rounds, load_s, extra=None):
    layer_params, head_params = gemm_params(cfg, a.layers)
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    attn_flops = 2 * 2 * nq * d * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2) * a.layers
    prefill_flops = 2 * PREFILL_TOKENS * layer_params + 2 * head_params + attn_flops
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    kv_bytes_tok = 2 * cfg["num_key_value_heads"] * d * 2 * a.layers
    step_bytes = 2 * (layer_params + head_params) + a.batch * mean_ctx * kv_bytes_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": "decode tokens/s, Qwen3-8B sizes bf16, batch %d, context 4096" % a.batch,
        "value": round(a.batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": max(1, a.steps),
        "warmup": max(3, a.warmup), "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), token ids uniform in [0, vocab)", "impl": impl,
        "config": {"model": "Qwen3-8B sizes", "layers": a.layers, "layers_of_model": FULL_LAYERS, "hidden": 4096,
                   "q_heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": cfg["vocab_size"],
                   "global_batch": a.batch, "seq_len": CONTEXT, "context_mean": int(mean_ctx), "page_size": 64,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (15 GB of weights)",
                   "peaks": pk["source"], "load_s": round(load_s, 1), "rounds": rounds},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    out.update(extra or {})
    return out


def run_reference(a, cfg, pk) -> int:
    """The reference arm: the unmodified reference from ``baseline/_ref``; nothing of this package is imported."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
    except Exception as exc:
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"}))
        return 0
    rounds = rounds_for(max(1, a.steps))
    try:
        r = reference_arm.run(a, cfg, CONTEXT, PREFILL_TOKENS, ClockSampler, rounds)
    except Exception as exc:                      # the line names what the reference (or its set-up) raised on this box
        import traceback
        traceback.print_exc(file=sys.stderr)
        text = " ".join(f"{type(exc).__name__}: {exc}".split())
        print(json.dumps({"impl": "reference", "unavailable": text[:400]}))
        return 0
    e2e = {"value": round(a.batch / r["e2e_ms"] * 1e3, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]}
    line = json_line(a, cfg, pk, impl="reference", ms=r["ms"], e2e=e2e, launches=None, clocks=r["clocks"],
                     prefill_ms=r["prefill_ms"], mean_ctx=r["mean_ctx"], points=r["points"], rounds=rounds,
                     load_s=r["load_s"], extra={"cuda_graphs": r["cuda_graphs"]})
    del line["gpu_launches"]
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    a = ap.parse_args()

    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    cfg = dict(QWEN3_8B, num_hidden_layers=a.layers)
    pk = peaks()
    if a.impl == "reference":
        return run_reference(a, cfg, pk)

    import torch

    from lily_b200.config.server_args import ServerArgs
    from lily_b200.csrc import ops
    from lily_b200.engine.batch import StepEntry
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.engine.runner import ModelRunner
    from lily_b200.sampling.params import SamplingParams

    warmup = max(3, a.warmup)
    steps = max(1, a.steps)
    rounds = rounds_for(steps)
    torch.cuda.set_device(0)
    max_batch = max(2 * a.batch, 8 if a.skip_points else 64)
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

    def device_timed(fn, reps):
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

    for _ in range(3):
        prefill_once()
    prefill_ms = device_timed(prefill_once, 5)

    # ---- decode: batch B, contexts ending at 4,096 --------------------------------------
    class RawBatch:
        """``batch`` requests driven by hand through the step function and the argmax kernel.  The sampled tokens
        stay on the device (the step function's ``FUTURE`` entries: the embedding kernel looks each request's last
        token up where the argmax left it), so the steps queue behind one another without the host reading
        anything back: what is timed is the device's work for a step."""

        def __init__(self, batch, total_steps):
            from lily_b200.engine.batch import FUTURE
            self.start_len = CONTEXT - total_steps - 2
            self.slots = [runner.open_request() for _ in range(batch)]
            for s in self.slots:                             # prompts go in whole, one request a step
                runner.step([StepEntry(s, ids(self.start_len), [])])
            logits = runner.step([StepEntry(s, [ids(1)[0]], [0]) for s in self.slots])
            runner.store_future(ops.argmax(logits))
            self.entries = [StepEntry(s, [FUTURE], [0]) for s in self.slots]

        def one(self):
            runner.store_future(ops.argmax(runner.step(self.entries)))

        def close(self):
            torch.cuda.synchronize()
            for s in self.slots:
                runner.close_request(s)

    def decode_point(batch, k, w, rounds=3):
        """Median over ``rounds`` of k device-timed steps each, after w untimed ones."""
        raw = RawBatch(batch, w + rounds * k)
        for _ in range(w):
            raw.one()
        ms = statistics.median(device_timed(raw.one, k) for _ in range(rounds))
        raw.close()
        return ms

    # the headline: device-timed steps of the step function and host-timed steps of the entry point's scheduler,
    # in alternating rounds under one clock record
    total = warmup + rounds * steps
    raw = RawBatch(a.batch, total)
    eng = Engine(EngineConfig("<random>", dtype="bfloat16", device="cuda:0", context_length=CONTEXT,
                              max_running_requests=max_batch,
                              server_args={"page_size": 64, "random_seed": 0, "chunked_prefill_size": 8192}), runner=runner)
    # requests admitted first decode a few tokens while the others' prompts go in: leave them room,
    # so that all of the batch is still decoding when the timed steps end
    slack = 2 * a.batch
    sched = eng.new_scheduler()
    for i in range(a.batch):
        sched.add_request(f"b{i}", ids(CONTEXT - total - slack),
                          SamplingParams(max_new_tokens=total + slack, ignore_eos=True))
    guard = 0
    while (sched.waiting_queue or len(sched.running) < a.batch) and guard < 10000:   # prompts in; first tokens sampled
        sched.step()
        guard += 1
    for _ in range(warmup):
        raw.one()
    for _ in range(warmup - 1):
        sched.step()
    dev_ms, host_ms, launches, graph_before = [], [], 0, runner.graph_steps
    with ClockSampler() as clocks:
        for _ in range(rounds):
            clocks.region = "value"
            l0 = ops.launches["count"]
            dev_ms.append(device_timed(raw.one, steps))
            launches = ops.launches["count"] - l0
            clocks.region = "e2e"
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            for _ in range(steps):
                sched.step()
            torch.cuda.synchronize()
            host_ms.append((time.perf_counter() - t_start) * 1e3 / steps)
        clocks.region = "idle"
    ms, e2e_ms = statistics.median(dev_ms), statistics.median(host_ms)
    graph_steps = runner.graph_steps - graph_before
    mean_ctx = raw.start_len + 1 + warmup + (rounds * steps + 1) / 2
    # what the host itself spends on a step of the entry point: with the device idle before each call, a call
    # launches one step and reads the tokens of the step before, which are there already
    host_only = []
    for _ in range(8):
        if len(sched.running) < a.batch:
            break
        torch.cuda.synchronize()
        t = time.perf_counter()
        sched.step()
        host_only.append((time.perf_counter() - t) * 1e3)
    running = len(sched.running)
    sched.run_to_completion()
    raw.close()
    cv, ce = clocks.summary("value"), clocks.summary("e2e")
    print(f"rounds: value ms {[round(x, 3) for x in dev_ms]} at {cv['sm_mhz']} MHz; e2e ms {[round(x, 3) for x in host_ms]} "
          f"at {ce['sm_mhz']} MHz; {graph_steps} of {2 * rounds * steps} steps through graphs, {running} running at the "
          f"end; host alone {statistics.median(host_only) if host_only else float('nan'):.3f} ms a step", file=sys.stderr)
    meta_ints = 3 * a.batch + 4 * a.batch + 1 + a.batch + a.batch * (CONTEXT // 64)
    e2e = {"value": round(a.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * meta_ints,
           "d2h_bytes_per_step": 4 * a.batch, "ms_per_step": round(e2e_ms, 4),
           "host_ms_per_step": round(statistics.median(host_only), 4) if host_only else None,
           "sm_mhz": ce["sm_mhz"]}
    summary = clocks.summary()
    summary["sm_mhz_value"] = cv["sm_mhz"]
    summary["ms_x_mhz_value"] = round(ms * cv["sm_mhz"], 1) if cv["sm_mhz"] else None
    summary["ms_x_mhz_e2e"] = round(e2e_ms * ce["sm_mhz"], 1) if ce["sm_mhz"] else None

    points = {}
    if not a.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(b / decode_point(b, min(steps, 32), warmup) * 1e3, 1)

    print(json.dumps(json_line(a, cfg, pk, impl="ours", ms=ms, e2e=e2e, launches=launches, clocks=summary,
                               prefill_ms=prefill_ms, mean_ctx=mean_ctx, points=points, rounds=rounds, load_s=load_s)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
