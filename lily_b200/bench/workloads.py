"""The two serving-shaped workloads that go with the benchmark configurations beside the headline
one, run through ``Engine`` / ``Scheduler`` with seeded random weights on one B200:

``llama31_mixed``   Llama-3.1-8B sizes, context 8192: 32 requests with prompt lengths uniform in
                    [128, 6144], portions of 2,048 prompt tokens a step beside the decoding
                    requests, up to 512 new tokens each.
``qwen3_32b_long``  Qwen3-32B sizes (65 GB of weights), context 16384: 16 requests whose contexts
                    fill to 16,384 positions, 128 decoded tokens each (split-key decode attention
                    over long contexts; the KV pool beside the weights).

Each prints one JSON line: tokens in and out, wall-clock and device times, decode and prefill
throughput, what the scheduler did (steps, retractions, overlapped steps), and checks that every
request ended as asked, that no bounded wait of a tcgen05 kernel gave up, and that all pages came
back.  ``--layers`` runs fewer layers than the configuration has (reported) where time is short.

    python -m lily_b200.bench.workloads llama31_mixed
    python -m lily_b200.bench.workloads qwen3_32b_long --layers 16
"""

from __future__ import annotations

import argparse
import json
import sys
import time

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192, "hidden_act": "silu",
    "torch_dtype": "bfloat16",
}
QWEN3_32B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 64, "hidden_size": 5120,
    "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 25600,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 16384, "hidden_act": "silu", "torch_dtype": "bfloat16",
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=["llama31_mixed", "qwen3_32b_long"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (reported)")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--new-tokens", type=int, default=0)
    ap.add_argument("--disable-overlap-schedule", action="store_true")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    a = ap.parse_args()

    import torch

    from lily_b200.config.server_args import ServerArgs
    from lily_b200.csrc import ops
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.engine.runner import ModelRunner
    from lily_b200.sampling.params import SamplingParams

    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(2)
    if a.workload == "llama31_mixed":
        cfg, context = dict(LLAMA31_8B), 8192
        requests, new_tokens = a.requests or 32, a.new_tokens or 512
        lengths = torch.randint(128, 6145, (requests,), generator=g).tolist()
        chunk = 2048
    else:
        cfg, context = dict(QWEN3_32B), 16384
        requests, new_tokens = a.requests or 16, a.new_tokens or 128
        lengths = [context - new_tokens] * requests
        chunk = 8192
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    vocab = cfg["vocab_size"]
    pool_tokens = sum(-(-(n + new_tokens) // 64) * 64 for n in lengths) + 64 * requests
    args = ServerArgs(dtype="bfloat16", device="cuda:0", context_length=context, page_size=64, max_total_tokens=pool_tokens,
                      max_running_requests=requests, chunked_prefill_size=chunk, max_prefill_tokens=max(chunk, 16384),
                      random_seed=0, disable_overlap_schedule=a.disable_overlap_schedule)
    t0 = time.time()
    runner = ModelRunner.from_random(cfg, seed=0, args=args)
    load_s = time.time() - t0
    free_before = runner.free_tokens()
    eng = Engine(EngineConfig("<random>", dtype="bfloat16", device="cuda:0", context_length=context,
                              max_running_requests=requests,
                              server_args={"page_size": 64, "random_seed": 0, "chunked_prefill_size": chunk,
                                           "max_prefill_tokens": max(chunk, 16384),
                                           "disable_overlap_schedule": a.disable_overlap_schedule}), runner=runner)
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
    sched = eng.new_scheduler()
    for i, p in enumerate(prompts):
        sched.add_request(f"w{i}", p, SamplingParams(max_new_tokens=new_tokens, ignore_eos=True, temperature=a.temperature,
                                                     top_k=a.top_k, top_p=a.top_p, seed=i))
    runner.capture_decode_graphs(range(1, requests + 1))      # as a server would: no step of the run pays for a capture
    torch.cuda.synchronize()
    start = time.perf_counter()
    steps = decode_only_steps = 0
    decode_only_time = 0.0
    prefill_steps_time = 0.0
    while sched.has_work():
        t = time.perf_counter()
        if not sched.step():
            break
        dt = time.perf_counter() - t
        steps += 1
        if sched.last_batch.get("prefill_tokens", 0) == 0:
            decode_only_steps += 1
            decode_only_time += dt
        else:
            prefill_steps_time += dt
    torch.cuda.synchronize()
    wall = time.perf_counter() - start
    results = [sched.results[f"w{i}"] for i in range(requests)]
    produced = sum(len(r.output_ids) for r in results)
    problems = []
    for i, r in enumerate(results):
        if len(r.output_ids) != new_tokens or (r.finish_reason or {}).get("type") != "length":
            problems.append(f"request {i}: {len(r.output_ids)} tokens, {r.finish_reason}")
        if any(not (0 <= t < vocab) for t in r.output_ids):
            problems.append(f"request {i}: token outside the vocabulary")
    if ops.attention_tc_status() != 0 or ops.gemm_tc_status() != 0:
        problems.append("a bounded wait of a tcgen05 kernel gave up")
    if runner.free_tokens() != free_before or runner.cache.held_pages() != [0] * len(runner.cache.groups):
        problems.append("pages were not all given back")
    out = {
        "workload": a.workload, "sampling": {"temperature": a.temperature, "top_k": a.top_k, "top_p": a.top_p}, "layers": cfg["num_hidden_layers"], "layers_of_model": full_layers, "requests": requests,
        "prompt_tokens": sum(lengths), "new_tokens": produced, "wall_s": round(wall, 3),
        "tokens_per_s_out": round(produced / wall, 1), "tokens_per_s_in_and_out": round((sum(lengths) + produced) / wall, 1),
        "steps": steps, "decode_only_steps": decode_only_steps,
        "decode_only_ms_per_step": round(decode_only_time / max(decode_only_steps, 1) * 1e3, 3),
        "steps_with_prompt_portions": steps - decode_only_steps,
        "ms_per_step_with_portions": round(prefill_steps_time / max(steps - decode_only_steps, 1) * 1e3, 3),
        "prefill_tokens_computed": sched.prefill_tokens_computed, "retractions": sched.retractions,
        "overlapped_steps": sched.overlapped_steps, "graph_steps": runner.graph_steps,
        "weights_gb": round(runner.weight_bytes / 1e9, 2), "pool_tokens": pool_tokens, "load_s": round(load_s, 1),
        "problems": problems,
    }
    print(json.dumps(out))
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
