"""The batch of one step: what the step function and the mixers read.

A step brings, for each request in it, the next tokens of that request: a portion of its
prompt (any length, cut anywhere) or one decoded token.  Requests that bring exactly one token
come first (``num_decode`` of them) so that their attention can run through the split-key decode
kernel while the portions run through the prefill kernel; the reference orders a mixed batch the
same way (lily/scheduler/schedule_batch.py:300-323).

All integer metadata lives in one int32 buffer that is filled on the host and copied to the
device once per step.  Field meanings follow lily/model_executor/forward_batch_info.py:40-63:
``positions`` (position of each token in its sequence), ``seq_lens`` (positions cached after the
step), ``prefix_lens`` (positions cached before it), ``cu_seqlens`` (offsets of each request's
tokens in the flat token array); block tables replace ``req_to_token`` rows.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch


# As the only token of an entry: the token sampled for this request by the step before, which the
# host may not have seen yet.  It travels as -(slot + 1) and the embedding kernel looks it up in the
# runner's table of future tokens (lily/scheduler/scheduler.py:194-216,488-492 of the reference
# keeps such a table by request slot for its overlap schedule).
FUTURE = -1


@dataclass
class StepEntry:
    """One request's share of a step."""

    slot: int                      # the request's slot in the cache manager
    tokens: Sequence[int]          # its next tokens (or [FUTURE])
    want: Sequence[int] = ()       # places among these tokens whose logits are asked for

    @property
    def wire_tokens(self) -> List[int]:
        """The token ids as the device reads them."""
        if len(self.tokens) == 1 and int(self.tokens[0]) == FUTURE:
            return [-(int(self.slot) + 1)]
        return [int(t) for t in self.tokens]


class Workspace:
    """Float32 scratch that kernels may use within a step; grows on demand, never shrinks,
    so its address is stable once a step of the largest shape has run."""

    def __init__(self, device):
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}

    def floats(self, name: str, count: int) -> torch.Tensor:
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < count:
            if torch.device(self.device).type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace {name!r} must be sized before a graph is captured")
            buf = torch.empty((max(count, 1),), dtype=torch.float32, device=self.device)
            self._buffers[name] = buf
        return buf

    def counters(self, name: str, count: int) -> torch.Tensor:
        """int32 counters that are zero when first handed out; kernels that use them leave them zero."""
        buf = self._buffers.get("int:" + name)
        if buf is None or buf.numel() < count:
            if torch.device(self.device).type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace {name!r} must be sized before a graph is captured")
            buf = torch.zeros((max(count, 1),), dtype=torch.int32, device=self.device)
            self._buffers["int:" + name] = buf
        return buf


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    num_decode: int
    # device int32
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_req: torch.Tensor
    cu_seqlens: torch.Tensor
    prefix_lens: torch.Tensor
    seq_lens: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    block_tables: List[torch.Tensor]
    # host
    h_new_lens: List[int]
    h_prefix_lens: List[int]
    h_slots: List[int]
    max_seq_len: int                                 # the longest sequence after the step (a bound, in a captured batch)
    max_decode_len: int = 0                          # the same over the requests that bring one token
    decode_even: bool = False                        # those requests are about equally long (``rows_are_even``); a mixer
    even_asked: bool = False                         # may plan by it, and says here that its plan depended on it
    workspace: Optional[Workspace] = None
    future_tokens: Optional[torch.Tensor] = None     # int32 [request slots]: what negative token ids stand for
    plans: Dict[Any, Any] = field(default_factory=dict)

    @property
    def num_prefill_requests(self) -> int:
        return self.num_requests - self.num_decode

    @property
    def h_seq_lens(self) -> List[int]:
        return [p + n for p, n in zip(self.h_prefix_lens, self.h_new_lens)]

    @property
    def fresh(self) -> List[bool]:
        """Requests whose first token comes in this step."""
        return [p == 0 for p in self.h_prefix_lens]

    def plan(self, key: Any, make: Callable[["StepBatch"], Any]) -> Any:
        """What a part worked out for this step, made once and shared by every layer that asks with the same
        ``key``: a mixer plans its step here (how to cut its work, which kernel form to take, lists it needs on
        the device) from the batch's host fields, so that the step function knows nothing of any mixer."""
        if key not in self.plans:
            self.plans[key] = make(self)
        return self.plans[key]


def rows_are_even(lengths: Sequence[int]) -> bool:
    """Whether the longest of these rows is at most an eighth longer than their mean."""
    return len(lengths) > 0 and 8 * max(lengths) * len(lengths) <= 9 * sum(lengths)


def order_entries(entries: Sequence[StepEntry]) -> List[int]:
    """Indices of ``entries`` with the one-token requests first, else in the given order."""
    ones = [i for i, e in enumerate(entries) if len(e.tokens) == 1]
    rest = [i for i, e in enumerate(entries) if len(e.tokens) != 1]
    return ones + rest


def build_step_batch(entries: Sequence[StepEntry], prefix_lens: Sequence[int],
                     tables: Sequence[Sequence[Sequence[int]]], device, *,
                     workspace: Optional[Workspace] = None, pinned: Optional[torch.Tensor] = None,
                     table_widths: Optional[Sequence[int]] = None,
                     logit_rows: Optional[Sequence[int]] = None) -> StepBatch:
    """Packs a step.  ``entries`` are already ordered (one-token requests first);
    ``prefix_lens[i]`` positions of entry i are cached; ``tables[g][i]`` is the block table of
    entry i in cache group g (covering prefix + new tokens).  ``logit_rows`` (flat token indices)
    replaces the rows that the entries' ``want`` give, e.g. to fix their order."""
    b = len(entries)
    new_lens = [len(e.tokens) for e in entries]
    n = sum(new_lens)
    num_decode = 0
    while num_decode < b and new_lens[num_decode] == 1:
        num_decode += 1
    if any(ln == 1 for ln in new_lens[num_decode:]):
        raise ValueError("one-token requests must come first in a step")
    seq_lens = [p + ln for p, ln in zip(prefix_lens, new_lens)]
    widths = list(table_widths) if table_widths is not None else [
        max((len(t) for t in g), default=0) for g in tables]
    widths = [max(1, w) for w in widths]
    wanted: List[int] = []
    cu = [0]
    for e, ln in zip(entries, new_lens):
        for w in e.want:
            if not (0 <= w < ln):
                raise ValueError(f"wanted place {w} is outside the {ln} tokens of the entry")
            wanted.append(cu[-1] + w)
        cu.append(cu[-1] + ln)
    if logit_rows is not None:
        wanted = [int(r) for r in logit_rows]
        if any(not (0 <= r < n) for r in wanted):
            raise ValueError("a wanted row lies outside the step's tokens")

    # one int32 buffer: tokens | positions | token_req | cu | prefix | seq | slots | rows | tables...
    sizes = [n, n, n, b + 1, b, b, b, len(wanted)] + [b * w for w in widths]
    total = sum(sizes)
    host = pinned[:total] if pinned is not None and pinned.numel() >= total else torch.empty(total, dtype=torch.int32)
    flat: List[int] = []
    for e in entries:
        flat.extend(e.wire_tokens)
    for p, ln in zip(prefix_lens, new_lens):
        flat.extend(range(p, p + ln))
    for i, ln in enumerate(new_lens):
        flat.extend([i] * ln)
    flat.extend(cu)
    flat.extend(prefix_lens)
    flat.extend(seq_lens)
    flat.extend(e.slot for e in entries)
    flat.extend(wanted)
    for g, w in zip(tables, widths):
        for t in g:
            if len(t) > w:
                raise ValueError(f"block table of {len(t)} pages exceeds the width {w}")
            flat.extend(t)
            flat.extend([0] * (w - len(t)))
    if total:
        host.copy_(torch.tensor(flat, dtype=torch.int32))
    dev = host.to(device, non_blocking=True) if torch.device(device).type != "cpu" else host.clone()
    parts = torch.split(dev, sizes) if total else [dev] * len(sizes)
    max_seq = max(seq_lens, default=0)
    return StepBatch(
        num_tokens=n, num_requests=b, num_decode=num_decode,
        token_ids=parts[0], positions=parts[1], token_req=parts[2], cu_seqlens=parts[3], prefix_lens=parts[4],
        seq_lens=parts[5], slots=parts[6], logit_rows=parts[7],
        block_tables=[parts[8 + i].view(b, w) for i, w in enumerate(widths)],
        h_new_lens=new_lens, h_prefix_lens=list(prefix_lens), h_slots=[e.slot for e in entries],
        max_seq_len=max_seq, max_decode_len=max((seq_lens[i] for i in range(num_decode)), default=0),
        decode_even=rows_are_even([seq_lens[i] for i in range(num_decode)]), workspace=workspace)
