"""Is what the engine generated greedily really the model's greedy output?  In the manner of the reference's
bench/check_greedy.py:1-41: the prompt and the generated tokens go through the prefill path once more (teacher
forcing, logits at every position) and the positions are reported where the generated token is not that run's
argmax, with the gap between the top logit and the generated token's.  Decode and prefill take different kernels
and round differently, so a few tiny gaps are expected in bfloat16; a large gap means the two paths disagree.

    python -m lily_b200.bench.check_greedy --model-path DIR [--dtype bfloat16] [--prompts 8] [--prompt-len 200] [--new-tokens 64]

Prints one JSON line: tokens checked, how many were not the argmax, the largest gap.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Sequence


def check_greedy(engine, prompts: Sequence[Sequence[int]], outputs: Sequence[Sequence[int]]) -> Dict:
    """``outputs[i]`` was generated greedily from ``prompts[i]``.  Returns counts and the gaps (top logit minus the
    generated token's logit at the positions where they differ), from one teacher-forced prefill per request."""
    import torch

    total, gaps = 0, []
    for prompt, out in zip(prompts, outputs):
        if not out:
            continue
        logits = engine.all_prefill_logits(list(prompt) + list(out[:-1]))[len(prompt) - 1:]
        emitted = torch.tensor(list(out), device=logits.device)
        gap = logits.max(dim=-1).values - logits.gather(1, emitted[:, None]).squeeze(1)
        total += len(out)
        gaps += [float(g) for g in gap[gap > 0].tolist()]
    gaps.sort()
    return {"tokens": total, "not_argmax": len(gaps), "max_gap": round(max(gaps, default=0.0), 4),
            "largest_gaps": [round(g, 4) for g in gaps[-8:]]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-path", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=200)
    ap.add_argument("--new-tokens", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()

    import torch

    from lily_b200 import Engine, EngineConfig, SamplingParams

    need = a.prompts * (a.prompt_len + a.new_tokens + 64)
    eng = Engine(EngineConfig(a.model_path, dtype=a.dtype, max_total_tokens=max(need, 4096), max_running_requests=a.prompts))
    g = torch.Generator().manual_seed(a.seed)
    vocab = eng.runner.spec.vocab_size
    prompts: List[List[int]] = [torch.randint(0, vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
    outs = [o["output_ids"] for o in eng.generate(prompts, SamplingParams(max_new_tokens=a.new_tokens, ignore_eos=True))]
    print(json.dumps({"model": a.model_path, "dtype": a.dtype, **check_greedy(eng, prompts, outs)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
