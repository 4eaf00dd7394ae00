"""From logits to the next token of each request.

Order as in lily/layers/sampler.py:34-133: penalties and bias on the logits, argmax when every
row is greedy, else temperature, top-k, top-p, min-p and a draw, all in CUDA kernels
(lily_b200/csrc/sampling.cu).  The draw's uniform number comes from ``uniform_for``: a counter
generator keyed by the request's seed and the index of the token being drawn, so a request's
tokens depend neither on the batch it is in nor on whether it was retracted and run again.
"""

from __future__ import annotations

from collections import Counter
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch

from lily_b200.sampling.params import SamplingParams

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of (seed, index)."""
    return (_splitmix64(_splitmix64(seed & _MASK) ^ (index & _MASK)) >> 40) / float(1 << 24)


@dataclass
class SampleRow:
    params: SamplingParams
    seed: int
    index: int                         # how many tokens the request has produced so far
    seen: Sequence[int] = ()           # prompt + produced tokens (for the penalties)


@dataclass
class Sampled:
    """What one call of the sampler left on the device, and how it reaches the host."""

    tokens: Optional[torch.Tensor]                 # int32 [rows] on the device
    logprobs: Optional[torch.Tensor] = None        # float32 [rows] on the device
    host_tokens: Optional[torch.Tensor] = None     # where an asynchronous copy puts them
    host_logprobs: Optional[torch.Tensor] = None
    copied: Any = None                             # event after the copies
    top: Any = None                                # (tokens, logprobs, counts, k per row) of ``top_logprobs`` rows

    def start_copy(self, pinned_tokens: torch.Tensor, pinned_logprobs: Optional[torch.Tensor] = None) -> None:
        """Starts the copy to pinned host memory behind the sampling kernels and records an event,
        so that the host can read the tokens later without waiting for work queued after them."""
        n = self.tokens.numel()
        self.host_tokens = pinned_tokens[:n]
        self.host_tokens.copy_(self.tokens, non_blocking=True)
        if self.logprobs is not None and pinned_logprobs is not None:
            self.host_logprobs = pinned_logprobs[:n]
            self.host_logprobs.copy_(self.logprobs, non_blocking=True)
        self.copied = torch.cuda.Event()
        self.copied.record()

    def read_top(self) -> Optional[List[Optional[List[Tuple[int, float]]]]]:
        """Per row None, or the ``top_logprobs`` most probable tokens as (token, log-probability), most
        probable first, ties by the lower token id (lily/layers/sampler.py:124-132)."""
        if self.top is None:
            return None
        tokens, logprobs, counts, ks = self.top
        tokens, logprobs, counts = tokens.tolist(), logprobs.tolist(), counts.tolist()
        out: List[Optional[List[Tuple[int, float]]]] = []
        for r, k in enumerate(ks):
            if k <= 0:
                out.append(None)
                continue
            pairs = sorted(zip(tokens[r][:counts[r]], logprobs[r][:counts[r]]), key=lambda tv: (-tv[1], tv[0]))
            out.append([(int(t), float(v)) for t, v in pairs[:k]])
        return out

    def read(self) -> Tuple[List[int], Optional[List[float]]]:
        if self.tokens is None:
            return [], None
        if self.copied is not None:
            self.copied.synchronize()
            return (self.host_tokens.tolist(),
                    self.host_logprobs.tolist() if self.host_logprobs is not None else
                    (self.logprobs.tolist() if self.logprobs is not None else None))
        return self.tokens.tolist(), (self.logprobs.tolist() if self.logprobs is not None else None)


class _Staging:
    """A few pinned int32 buffers used in turn for the per-step sampling parameters: one asynchronous
    copy a step (a copy from pageable memory would hold the host until the device gets to it, which
    is after the step it was queued behind).  A buffer is reused only after its copy has finished."""

    def __init__(self, count: int = 4):
        self.buffers: List[Optional[torch.Tensor]] = [None] * count
        self.events: List[Any] = [None] * count
        self.next = 0

    def upload(self, columns: Sequence[torch.Tensor], device) -> List[torch.Tensor]:
        """``columns``: equally long int32 / float32 host tensors.  Returns their copies on the device."""
        n = columns[0].numel()
        i = self.next
        self.next = (i + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.buffers[i] is None or self.buffers[i].numel() < len(columns) * n:
            self.buffers[i] = torch.empty(max(len(columns) * n, 1024), dtype=torch.int32, pin_memory=True)
        host = self.buffers[i][:len(columns) * n].view(len(columns), n)
        for row, col in zip(host, columns):
            row.copy_(col.view(torch.int32))
        dev = host.to(device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return [dev[j].view(col.dtype) for j, col in enumerate(columns)]


class Sampler:
    def __init__(self, ops: Any, device):
        self.ops, self.device = ops, device
        self._staging = _Staging() if torch.device(device).type == "cuda" else None

    def launch(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> Sampled:
        """``logits`` float32 [len(rows), vocab] on the device (modified in place by penalties).
        Queues the sampling kernels and returns the tokens (and, when any row asks for them, the
        chosen tokens' log-probabilities) as device tensors."""
        if len(rows) == 0:
            return Sampled(None)
        assert logits.shape[0] == len(rows), (logits.shape, len(rows))
        ops, dev = self.ops, self.device
        if any(not r.params.plain for r in rows):
            self._penalties(logits, rows)
        need_lp = any(r.params.logprobs for r in rows)
        top = None
        ks = [int(r.params.top_logprobs or 0) for r in rows]
        if any(ks):
            top = (*ops.top_logprobs(logits, torch.tensor(ks, dtype=torch.int32).to(dev)), ks)
        if all(r.params.greedy for r in rows) and not need_lp:
            return Sampled(ops.argmax(logits), top=top)
        columns = [torch.tensor([0.0 if r.params.greedy else r.params.temperature for r in rows], dtype=torch.float32),
                   torch.tensor([r.params.top_k for r in rows], dtype=torch.int32),
                   torch.tensor([r.params.top_p for r in rows], dtype=torch.float32),
                   torch.tensor([r.params.min_p for r in rows], dtype=torch.float32),
                   torch.tensor([uniform_for(r.seed, r.index) for r in rows], dtype=torch.float32)]
        if self._staging is not None:
            temperature, top_k, top_p, min_p, uniform = self._staging.upload(columns, dev)
        else:
            temperature, top_k, top_p, min_p, uniform = (c.to(dev) for c in columns)
        tokens, logprobs = ops.sample(logits, temperature, top_k, top_p, min_p, uniform, want_logprob=need_lp)
        return Sampled(tokens, logprobs, top=top)

    def __call__(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> Tuple[List[int], Optional[List[float]]]:
        """``launch`` and read the result at once."""
        return self.launch(logits, rows).read()

    def _penalties(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> None:
        e_row: List[int] = []
        e_tok: List[int] = []
        e_cnt: List[int] = []
        e_bias: List[float] = []
        for i, r in enumerate(rows):
            p = r.params
            if p.plain:
                continue
            counts = Counter(r.seen) if (p.repetition_penalty != 1.0 or p.frequency_penalty or p.presence_penalty) else {}
            bias = p.logit_bias or {}
            for tok in set(counts) | set(bias):
                e_row.append(i)
                e_tok.append(tok)
                e_cnt.append(counts.get(tok, 0))
                e_bias.append(bias.get(tok, 0.0))
        if not e_row:
            return
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.ops.apply_penalties(
            logits, torch.tensor(e_row, **i32), torch.tensor(e_tok, **i32), torch.tensor(e_cnt, **i32),
            torch.tensor(e_bias, **f32),
            torch.tensor([r.params.repetition_penalty for r in rows], **f32),
            torch.tensor([r.params.frequency_penalty for r in rows], **f32),
            torch.tensor([r.params.presence_penalty for r in rows], **f32))
