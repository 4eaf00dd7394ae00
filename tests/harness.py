"""Shared helpers of the tests: model folders in temporary places, runners, replay schedules."""

from __future__ import annotations

import os
from typing import Dict, List, Sequence

import torch

import kernel_refs
import tiny_models
from lily_b200.config.server_args import ServerArgs
from lily_b200.engine.batch import StepEntry
from lily_b200.engine.runner import ModelRunner


def model_dir(cfg: dict, seed: int, tmp: str, dtype=torch.float32, jitter: float = 0.01):
    weights = tiny_models.make_weights(cfg, seed, norm_jitter=jitter, dtype=dtype)
    path = os.path.join(tmp, f"m{seed}")
    tiny_models.write_model_dir(path, cfg, weights)
    return path, weights


def make_runner(path: str, dtype: str = "float32", device: str = "cpu", max_tokens: int = 1024, page_size: int = 16,
                max_requests: int = 8, **kw) -> ModelRunner:
    args = ServerArgs(model_path=path, dtype=dtype, device=device, max_total_tokens=max_tokens, page_size=page_size,
                      max_running_requests=max_requests, **kw)
    return ModelRunner.from_model_dir(args, ops=kernel_refs if device == "cpu" else None)


def run_whole(runner: ModelRunner, ids: Sequence[int]) -> torch.Tensor:
    slot = runner.open_request()
    out = runner.step([StepEntry(slot, list(ids), list(range(len(ids))))])
    runner.close_request(slot)
    return out.float().cpu()


def run_portions(runner: ModelRunner, ids: Sequence[int], cuts: Sequence[int]) -> torch.Tensor:
    """The same request cut into portions of the given sizes (the last portion takes the rest)."""
    slot = runner.open_request()
    rows, done = [], 0
    sizes = list(cuts)
    while done < len(ids):
        n = min(sizes.pop(0) if sizes else len(ids) - done, len(ids) - done)
        rows.append(runner.step([StepEntry(slot, list(ids[done:done + n]), list(range(n)))]).float().cpu())
        done += n
    runner.close_request(slot)
    return torch.cat(rows)


def run_mixed(runner: ModelRunner, requests: Dict[str, List[int]], plan: List[Dict[str, int]],
              ends: Dict[int, List[str]] = None) -> Dict[str, torch.Tensor]:
    """``plan[s]`` maps a request name to how many of its next tokens step s brings; every token's
    logits are wanted.  ``ends[s]`` lists requests closed after step s (all others at the end)."""
    slots, done, rows = {}, {k: 0 for k in requests}, {k: [] for k in requests}
    for s, step in enumerate(plan):
        entries, names = [], []
        for name, n in step.items():
            if name not in slots:
                slots[name] = runner.open_request()
            toks = requests[name][done[name]:done[name] + n]
            if not toks:
                continue
            entries.append(StepEntry(slots[name], toks, list(range(len(toks)))))
            names.append(name)
            done[name] += len(toks)
        out = runner.step(entries).float().cpu()
        at = 0
        for name, e in zip(names, entries):
            rows[name].append(out[at:at + len(e.tokens)])
            at += len(e.tokens)
        for name in (ends or {}).get(s, []):
            runner.close_request(slots.pop(name))
    for name in list(slots):
        runner.close_request(slots.pop(name))
    return {k: torch.cat(v) for k, v in rows.items() if v}
