"""The Python entry point, in the manner of lily/engine.py:24-145.

``Engine(EngineConfig(model_path, ...))`` loads a model folder and offers the reference's helpers
(``prefill_logits``, ``all_prefill_logits``, ``generate_greedy``, ``kv_available``) and, beyond the
reference's one-sequence engine, ``generate`` for many prompts at once through the scheduler.
Token ids in, token ids out; ``generate_text`` works when the model folder holds a tokenizer.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from lily_b200.config.server_args import ServerArgs
from lily_b200.engine.batch import StepEntry
from lily_b200.engine.runner import ModelRunner
from lily_b200.engine.scheduler import Scheduler
from lily_b200.sampling.params import SamplingParams


@dataclass
class EngineConfig:
    model_path: str
    dtype: str = "auto"
    device: str = "cuda"
    context_length: Optional[int] = None
    max_running_requests: Optional[int] = None
    max_total_tokens: Optional[int] = None
    mem_fraction_static: Optional[float] = None
    # Any other ServerArgs field, e.g. {"page_size": 16, "chunked_prefill_size": 512}.
    server_args: Optional[dict] = None


class Engine:
    def __init__(self, config: EngineConfig, runner: Optional[ModelRunner] = None):
        self.config = config
        self.server_args = ServerArgs(model_path=config.model_path, dtype=config.dtype, device=config.device,
                                      context_length=config.context_length,
                                      max_running_requests=config.max_running_requests,
                                      max_total_tokens=config.max_total_tokens,
                                      mem_fraction_static=config.mem_fraction_static,
                                      **(config.server_args or {}))
        self.runner = runner or ModelRunner.from_model_dir(self.server_args)
        self.device = self.runner.device
        self.eos_token_ids = list(self.runner.spec.eos_token_ids)
        self._tokenizer = None
        self._requests = 0

    # ---- one sequence, by hand (lily/engine.py:91-131) ---------------------------------

    @torch.inference_mode()
    def prefill_logits(self, prompt_ids: Sequence[int]) -> torch.Tensor:
        slot = self.runner.open_request()
        try:
            return self.runner.step([StepEntry(slot, list(prompt_ids), [len(prompt_ids) - 1])])[0]
        finally:
            self.runner.close_request(slot)

    @torch.inference_mode()
    def all_prefill_logits(self, prompt_ids: Sequence[int]) -> torch.Tensor:
        """Logits for every prompt position, [len, vocab] float32."""
        slot = self.runner.open_request()
        try:
            return self.runner.step([StepEntry(slot, list(prompt_ids), list(range(len(prompt_ids))))])
        finally:
            self.runner.close_request(slot)

    @torch.inference_mode()
    def generate_greedy(self, prompt_ids: Sequence[int], max_new_tokens: int, ignore_eos: bool = True) -> List[int]:
        out = self.generate([list(prompt_ids)], SamplingParams(max_new_tokens=max_new_tokens, ignore_eos=ignore_eos))
        return out[0]["output_ids"]

    @torch.inference_mode()
    def capture_decode_graphs(self, batch_sizes: Optional[Sequence[int]] = None,
                              max_len: Optional[int] = None) -> List[int]:
        """Captures the CUDA graphs of decode steps with these numbers of requests now (default: every bucket up to
        ``max_running_requests``) rather than at the first step of each size, for sequences of up to ``max_len``
        positions (default: every length class up to the context length); returns the buckets captured."""
        return self.runner.capture_decode_graphs(batch_sizes, max_len)

    # ---- many sequences, through the scheduler ------------------------------------------

    def new_scheduler(self) -> Scheduler:
        a = self.server_args
        return Scheduler(self.runner, max_prefill_tokens=a.max_prefill_tokens,
                         chunked_prefill_size=a.chunked_prefill_size, max_running_requests=a.max_running_requests,
                         eos_token_ids=self.eos_token_ids, random_seed=a.random_seed,
                         overlap=not a.disable_overlap_schedule)

    @torch.inference_mode()
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[Dict[str, Any]]:
        """Runs the prompts (lists of token ids) to completion with continuous batching and
        returns, per prompt, ``{"output_ids", "finish_reason", "prompt_tokens", "logprobs", "top_logprobs"}``."""
        sched = self.new_scheduler()
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            plist = [sampling_params or SamplingParams()] * len(prompts)
        else:
            plist = list(sampling_params)
            if len(plist) != len(prompts):
                raise ValueError("one SamplingParams per prompt, or one for all")
        rids = []
        for ids, p in zip(prompts, plist):
            rid = f"r{self._requests}"
            self._requests += 1
            rids.append(rid)
            sched.add_request(rid, ids, p)
        sched.run_to_completion()
        self.last_scheduler = sched
        out = []
        for rid in rids:
            r = sched.results[rid]
            out.append({"output_ids": r.output_ids, "finish_reason": r.finish_reason, "prompt_tokens": r.prompt_tokens,
                        "logprobs": r.logprobs, "top_logprobs": r.top_logprobs})
        return out

    # ---- text, when a tokenizer is at hand (lily/engine.py:133-142) ---------------------

    def _tok(self):
        if self._tokenizer is None:
            from transformers import AutoTokenizer      # tokenisation only; no model code of any library is used
            self._tokenizer = AutoTokenizer.from_pretrained(self.config.model_path)
        return self._tokenizer

    def generate_text(self, prompt: str, max_new_tokens: int = 64, chat: bool = True) -> str:
        """Text in, text out, greedy, for a model folder that holds a tokenizer: the prompt goes through the
        tokenizer's chat template when it has one and ``chat`` is set (the helper of lily/engine.py:133-142)."""
        tok = self._tok()
        use_template = chat and bool(getattr(tok, "chat_template", None))
        if use_template:
            encoded = tok.apply_chat_template([{"role": "user", "content": prompt}], tokenize=True,
                                              add_generation_prompt=True)
            encoded = encoded["input_ids"] if hasattr(encoded, "keys") else encoded
        else:
            encoded = tok.encode(prompt)
        produced = self.generate([[int(t) for t in encoded]],
                                 SamplingParams(max_new_tokens=max_new_tokens, ignore_eos=False))[0]["output_ids"]
        return tok.decode(produced, skip_special_tokens=True)

    def kv_available(self) -> int:
        """Tokens the free pages of the pool can hold."""
        return self.runner.free_tokens()
