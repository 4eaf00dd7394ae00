"""Per-request sampling parameters: the fields, defaults and checks of
lily/sampling/sampling_params.py:9-52.  ``stop`` strings, ``stream`` and ``n`` belong to the text
front end and the server, which this engine does not have; they are accepted and checked so that a
caller's parameters carry over, and ``stop`` raises when set because nothing here could honour it."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Union


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logit_bias: Optional[Dict[int, float]] = None
    stop_token_ids: List[int] = field(default_factory=list)
    stop: Optional[Union[str, List[str]]] = None
    ignore_eos: bool = False
    seed: Optional[int] = None
    stream: bool = False
    n: int = 1
    logprobs: bool = False
    top_logprobs: Optional[int] = None

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be positive")
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not (0 < self.top_p <= 1):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError("top_k must be -1 or a positive integer")
        if not (0 <= self.min_p < 1):
            raise ValueError("min_p must be in [0, 1)")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.stop:
            raise ValueError("stop strings need a detokenizer; this engine is token in, token out "
                             "(use stop_token_ids)")
        if self.top_logprobs is not None and not (1 <= self.top_logprobs <= 64):
            raise ValueError("top_logprobs must be between 1 and 64")
        if self.n != 1:
            raise ValueError("n must be 1; submit the prompt n times with different seeds")
        if self.logit_bias is not None:
            self.logit_bias = {int(k): float(v) for k, v in self.logit_bias.items()}

    @property
    def greedy(self) -> bool:
        """No randomness: a single deterministic token is produced."""
        return self.temperature == 0 or self.top_k == 1

    @property
    def plain(self) -> bool:
        """Neither penalties nor bias touch the logits."""
        return (self.repetition_penalty == 1.0 and self.frequency_penalty == 0.0 and self.presence_penalty == 0.0
                and not self.logit_bias)
