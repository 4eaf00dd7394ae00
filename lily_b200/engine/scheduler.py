"""Continuous batching above the step function.

Each ``step()``:

1. **decode**: every running request brings its last token.  If the pool cannot give the pages
   these tokens need, the youngest running requests are *retracted*: everything they hold is
   given back, their produced tokens are kept, and they go to the front of the waiting queue to
   be run again over prompt + produced tokens (lily/scheduler/scheduler.py:374-380,399-417).
2. **admit**: waiting requests are taken first come first served while request slots and a token
   budget remain.  The budget is ``min(max_prefill_tokens, chunked_prefill_size, what the free
   pages hold after one page is kept back for each running request)``; a request that needs more
   than what is left takes what is left and stays at the front of the queue for the next step with
   what it has cached (chunked prefill: scheduler.py:56-70,320-359,577-582).
3. one batch of decode tokens and prompt portions goes through ``ModelRunner.step``; logits are
   asked for at the decode tokens and at the last token of every portion that completes its prompt.
4. sampled tokens are appended; a request finishes on ``max_new_tokens`` (``{"type": "length"}``),
   on an eos or stop token unless ``ignore_eos`` (``{"type": "stop"}``), or when it fills the
   context; a finished request gives back its pages and slot (lily/scheduler/schedule_batch.py:
   88-97, scheduler.py:629-650).

With ``overlap`` the host does not wait for a step's tokens before it launches the next one
(lily/scheduler/scheduler.py:463-551 does the same): a running request whose last token is still
on the device brings ``FUTURE`` instead of a token id, the sampler's kernels leave each token in
the runner's table by request slot where the next step's embedding finds it, and the host reads
the tokens of step N (an asynchronous copy and an event) after it has queued step N + 1.  A request
that is known to end with the token in flight (``max_new_tokens``, the context limit) is left out
of the next step; one that turns out to have ended (a stop token) has the extra token dropped when
it arrives.  What it held is given back at once: the device runs the steps in order, so whoever
gets the pages next writes them after the step in flight has.  Steps that need the tokens on the
host first are not overlapped: sampling with penalties, and a step that has to retract.

When pages run out: decode retracts as above; a waiting request simply waits; a request that
could never fit (prompt beyond the context or beyond the whole pool) is refused when it is added
(``{"type": "abort"}``), and a lone running request that cannot grow even with the pool to itself
finishes with ``{"type": "length", "message": "KV cache exhausted"}``.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

from lily_b200.cache.pages import pages_for
from lily_b200.engine.batch import FUTURE, StepEntry
from lily_b200.sampling.params import SamplingParams
from lily_b200.sampling.sampler import Sampled, SampleRow, Sampler

logger = logging.getLogger(__name__)


@dataclass
class Req:
    rid: str
    origin_input_ids: List[int]
    sampling_params: SamplingParams
    eos_token_ids: List[int]
    seed: int = 0
    output_ids: List[int] = field(default_factory=list)
    output_logprobs: Optional[List[float]] = None
    output_top_logprobs: Optional[List[List[tuple]]] = None
    slot: Optional[int] = None
    seq_len: int = 0                    # positions cached
    extend_input_len: int = 0           # tokens this step brings
    is_chunked: bool = False
    finished_reason: Optional[dict] = None
    retractions: int = 0
    pending: int = 0                    # tokens sampled for it that the host has not read yet

    @property
    def fill_ids(self) -> List[int]:
        return self.origin_input_ids + self.output_ids

    @property
    def finished(self) -> bool:
        return self.finished_reason is not None

    def ends_with_pending(self, context_len: int) -> bool:
        """Whether the tokens in flight are known to be its last (length or context limit)."""
        n = len(self.output_ids) + self.pending
        return self.pending > 0 and (n >= self.sampling_params.max_new_tokens
                                     or len(self.origin_input_ids) + n >= context_len)

    def check_finished(self, context_len: int) -> Optional[dict]:
        """lily/scheduler/schedule_batch.py:88-97, plus the context limit."""
        if self.finished_reason is not None:
            return self.finished_reason
        p = self.sampling_params
        if len(self.output_ids) >= p.max_new_tokens:
            self.finished_reason = {"type": "length"}
        elif self.output_ids and not p.ignore_eos and (
                self.output_ids[-1] in set(self.eos_token_ids) | set(p.stop_token_ids)):
            self.finished_reason = {"type": "stop", "value": self.output_ids[-1]}
        elif len(self.origin_input_ids) + len(self.output_ids) >= context_len:
            self.finished_reason = {"type": "length", "message": "context length reached"}
        return self.finished_reason


@dataclass
class _Launched:
    """A step whose sampled tokens are still on the device."""

    sampled: List[Req]
    result: Sampled


@dataclass
class SchedulerOutput:
    rid: str
    output_ids: List[int]
    prompt_tokens: int
    completion_tokens: int
    finished: bool
    finish_reason: Optional[dict]
    logprobs: Optional[List[float]] = None
    top_logprobs: Optional[List[List[tuple]]] = None


class Scheduler:
    def __init__(self, runner: Any, *, max_prefill_tokens: int = 16384, chunked_prefill_size: int = 8192,
                 max_running_requests: Optional[int] = None, eos_token_ids: Sequence[int] = (),
                 random_seed: Optional[int] = None, sampler: Optional[Sampler] = None, overlap: bool = False):
        self.runner = runner
        self.max_prefill_tokens = max_prefill_tokens
        self.chunked_prefill_size = chunked_prefill_size
        self.max_running_requests = min(max_running_requests or runner.max_requests, runner.max_requests)
        self.eos_token_ids = list(eos_token_ids)
        self.sampler = sampler or Sampler(runner.model.ctx.ops, runner.device)
        self.base_seed = random_seed if random_seed is not None else int.from_bytes(os.urandom(8), "little")
        self.waiting_queue: List[Req] = []
        self.running: List[Req] = []
        self.results: Dict[str, SchedulerOutput] = {}
        self.on_token: Optional[Callable[[Req, int], None]] = None
        self._arrivals = 0
        self.prefill_tokens_computed = 0
        self.decode_steps = 0
        self.retractions = 0
        self.last_batch: Dict[str, int] = {}
        self.overlap = bool(overlap)
        self.overlapped_steps = 0
        self._inflight: Optional[_Launched] = None
        self._pinned: List[Any] = []
        self._pinned_turn = 0

    # ---- intake --------------------------------------------------------------------

    def add_request(self, rid: str, input_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None) -> Req:
        params = sampling_params or SamplingParams()
        seed = params.seed if params.seed is not None else (self.base_seed * 1000003 + self._arrivals)
        self._arrivals += 1
        req = Req(rid=rid, origin_input_ids=[int(t) for t in input_ids], sampling_params=params,
                  eos_token_ids=self.eos_token_ids, seed=seed)
        if params.logprobs:
            req.output_logprobs = []
        if params.top_logprobs:
            req.output_top_logprobs = []
        cache = self.runner.cache
        n = len(req.origin_input_ids)
        problem = None
        if n == 0:
            problem = "empty prompt"
        elif n >= self.runner.context_len:
            problem = f"prompt of {n} tokens leaves no room in the context of {self.runner.context_len}"
        elif pages_for(n + 1, cache.page_size) > cache.num_pages:
            problem = f"prompt of {n} tokens exceeds the whole KV pool ({cache.num_pages} pages of {cache.page_size})"
        elif any(not (0 <= t < self.runner.spec.vocab_size) for t in req.origin_input_ids):
            problem = "token id outside the vocabulary"
        if problem:
            req.finished_reason = {"type": "abort", "message": problem}
            self._publish(req)
            return req
        self.waiting_queue.append(req)
        return req

    def abort_request(self, rid: str) -> None:
        """lily/scheduler/scheduler.py:241-258: wherever the request is, what it holds goes back."""
        for queue in (self.waiting_queue, self.running):
            for req in list(queue):
                if req.rid == rid:
                    queue.remove(req)
                    self._release(req)
                    req.finished_reason = {"type": "abort", "message": "aborted"}
                    self._publish(req)

    def has_work(self) -> bool:
        return bool(self.waiting_queue or self.running or self._inflight is not None)

    # ---- bookkeeping ---------------------------------------------------------------

    def _release(self, req: Req) -> None:
        if req.slot is not None:
            self.runner.close_request(req.slot)
            req.slot = None
        req.seq_len = 0

    def _publish(self, req: Req) -> None:
        self.results[req.rid] = SchedulerOutput(
            rid=req.rid, output_ids=list(req.output_ids), prompt_tokens=len(req.origin_input_ids),
            completion_tokens=len(req.output_ids), finished=req.finished, finish_reason=req.finished_reason,
            logprobs=list(req.output_logprobs) if req.output_logprobs is not None else None,
            top_logprobs=list(req.output_top_logprobs) if req.output_top_logprobs is not None else None)

    def _retract(self, req: Req) -> None:
        self._release(req)
        req.is_chunked = False
        req.extend_input_len = 0
        req.retractions += 1
        self.retractions += 1
        self.waiting_queue.insert(0, req)
        logger.info("retract: %s goes back to the queue (%d running)", req.rid, len(self.running))

    # ---- decisions -----------------------------------------------------------------

    def _decode_pages(self, reqs: Sequence[Req]) -> int:
        cache = self.runner.cache
        return sum(cache.pages_needed(r.slot, r.seq_len + 1) for r in reqs)

    def _decode_candidates(self) -> List[Req]:
        """Running requests that take another step: all but those whose token in flight is their last."""
        ctx = self.runner.context_len
        return [r for r in self.running if not r.ends_with_pending(ctx)]

    def _plan_decode(self) -> List[Req]:
        """Running requests that decode this step, after taking pages back while the pool cannot give
        every one of them its next position: first from a request still filling its prompt, then by
        retracting the youngest running one.  (Nothing is in flight when it retracts:
        ``step`` reads the tokens first when the pages are short.)"""
        cache = self.runner.cache
        while self.running and self._decode_pages(self._decode_candidates()) > cache.free_pages():
            filling = next((r for r in reversed(self.waiting_queue) if r.slot is not None), None)
            if filling is not None:
                # a request that waits with part of its prompt cached gives that back first and keeps its place
                self._release(filling)
                filling.extend_input_len = 0
                filling.retractions += 1
                self.retractions += 1
                continue
            if len(self.running) == 1:
                req = self.running.pop()
                self._release(req)
                req.finished_reason = {"type": "length", "message": "KV cache exhausted"}
                self._publish(req)
                break
            self._retract(self.running.pop())
        return self._decode_candidates()

    def _plan_prefill(self, decoding: Sequence[Req]) -> List[Req]:
        cache = self.runner.cache
        page = cache.page_size
        # pages the decode tokens take now, and one kept back per running request for its next page
        free_pages = cache.free_pages() - self._decode_pages(decoding) - len(decoding)
        budget = min(self.max_prefill_tokens, self.chunked_prefill_size)
        # every request with a slot counts, also one whose last token is still in flight and one that waits
        # with part of its prompt cached
        slots = self.max_running_requests - len(self.running) - sum(r.slot is not None for r in self.waiting_queue)
        selected: List[Req] = []
        for req in list(self.waiting_queue):
            if budget <= 0 or (req.slot is None and slots <= 0):
                break
            needed = len(req.fill_ids) - req.seq_len
            held = pages_for(req.seq_len, page)
            # tokens the request could still cache: what is left of the last page it holds, and the free pages
            room = (held + max(free_pages, 0)) * page - req.seq_len
            take = min(needed, budget, room)
            if take <= 0:
                break
            req.extend_input_len = take
            req.is_chunked = take < needed
            selected.append(req)
            budget -= take
            slots -= req.slot is None
            free_pages -= pages_for(req.seq_len + take, page) - held
            if req.is_chunked:
                break                      # the rest of this prompt comes before any later request
        return selected

    # ---- one step ------------------------------------------------------------------

    def _next_needs_host_tokens(self) -> bool:
        """With a step in flight: whether the next one has to wait for its tokens (penalties read
        the history; a retraction re-queues prompt + produced tokens)."""
        candidates = self._decode_candidates()
        if any(not r.sampling_params.plain or r.sampling_params.top_logprobs for r in candidates):
            return True
        return self._decode_pages(candidates) > self.runner.cache.free_pages()

    def step(self) -> bool:
        """Runs one batch.  Returns False when there was nothing to run."""
        if self._inflight is not None and self._next_needs_host_tokens():
            self._collect(self._take_inflight())
        launched = self._launch()
        previous = self._take_inflight()
        if previous is not None:
            self._collect(previous)
        if launched is None:
            if previous is not None:
                return True
            if self.waiting_queue and not self.running:
                # nothing runs and the head of the queue cannot start: it never will
                req = self.waiting_queue.pop(0)
                self._release(req)
                req.finished_reason = {"type": "abort", "message": "request does not fit the KV pool"}
                self._publish(req)
                return True
            return False
        if self.overlap and launched.result.tokens is not None:
            if self.runner.device.type == "cuda":
                launched.result.start_copy(*self._pinned_pair())
            self._inflight = launched
            self.overlapped_steps += 1
        else:
            self._collect(launched)
        return True

    def _take_inflight(self) -> Optional[_Launched]:
        launched, self._inflight = self._inflight, None
        return launched

    def _pinned_pair(self):
        """Two pairs of pinned buffers used in turn: a pair is read by ``_collect`` before the launch
        after the next takes it again."""
        if not self._pinned:
            import torch
            n = self.runner.max_requests + 1
            self._pinned = [(torch.zeros(n, dtype=torch.int32, pin_memory=True),
                             torch.zeros(n, dtype=torch.float32, pin_memory=True)) for _ in range(2)]
        self._pinned_turn ^= 1
        return self._pinned[self._pinned_turn]

    def _launch(self) -> Optional[_Launched]:
        """Plans a batch, queues it and its sampling on the device, and moves the requests on as if
        every sampled token were an ordinary one; ``_collect`` corrects that when it reads them."""
        decoding = self._plan_decode()
        prefilling = self._plan_prefill(decoding)
        if not decoding and not prefilling:
            return None
        entries: List[StepEntry] = []
        for req in decoding:
            entries.append(StepEntry(req.slot, [FUTURE if req.pending else req.output_ids[-1]], [0]))
        for req in prefilling:
            if req.slot is None:
                req.slot = self.runner.open_request()
            ids = req.fill_ids[req.seq_len:req.seq_len + req.extend_input_len]
            entries.append(StepEntry(req.slot, ids, [] if req.is_chunked else [len(ids) - 1]))
            self.waiting_queue.remove(req)
        self.last_batch = {"decode": len(decoding), "prefill_requests": len(prefilling),
                           "prefill_tokens": sum(r.extend_input_len for r in prefilling)}
        logits = self.runner.step(entries)
        self.decode_steps += len(decoding)
        self.prefill_tokens_computed += self.last_batch["prefill_tokens"]

        sampled = [r for r in decoding] + [r for r in prefilling if not r.is_chunked]
        rows = [SampleRow(r.sampling_params, r.seed, len(r.output_ids) + r.pending,
                          r.fill_ids if not r.sampling_params.plain else ()) for r in sampled]
        result = self.sampler.launch(logits, rows)
        if self.overlap and result.tokens is not None:
            self.runner.store_future(result.tokens)

        for req in decoding:
            req.seq_len += 1
        requeue: List[Req] = []
        for req in prefilling:
            req.seq_len += req.extend_input_len
            if req.is_chunked:
                req.is_chunked = False
                requeue.append(req)
            else:
                self.running.append(req)
        for req in sampled:
            req.pending += 1
        self.waiting_queue[:0] = requeue
        return _Launched(sampled, result)

    def _collect(self, launched: _Launched) -> None:
        """Reads the tokens of a launched step and lets each request take its own."""
        tokens, logprobs = launched.result.read()
        tops = launched.result.read_top()
        for i, req in enumerate(launched.sampled):
            req.pending -= 1
            if req.finished:
                continue                   # it ended a step ago (or was aborted): this token is one too many
            req.output_ids.append(int(tokens[i]))
            if req.output_logprobs is not None and logprobs is not None:
                req.output_logprobs.append(float(logprobs[i]))
            if req.output_top_logprobs is not None and tops is not None and tops[i] is not None:
                req.output_top_logprobs.append(tops[i])
            if self.on_token is not None:
                self.on_token(req, int(tokens[i]))
            if req.check_finished(self.runner.context_len):
                self._release(req)
                self._publish(req)
                if req in self.running:
                    self.running.remove(req)

    def run_to_completion(self, max_steps: int = 1 << 30) -> None:
        steps = 0
        while self.has_work() and steps < max_steps:
            if not self.step():
                break
            steps += 1
