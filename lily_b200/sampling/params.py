"""Per-request sampling parameters: the fields, defaults and checks of
lily/sampling/sampling_params.py:9-52.  ``stop`` strings, ``stream`` and ``n`` belong to the text
front end and the server, which this engine does not have; they are accepted and checked so that a
caller's parameters carry over, and ``stop`` raises when set because nothing here could honour it."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, Dict, List, Optional, Union


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

    # what each number may be: (field, lowest, lowest allowed itself?, highest, highest allowed itself?)
    _RANGES: ClassVar[tuple] = (("max_new_tokens", 1, True, None, True), ("temperature", 0.0, True, None, True),
               ("top_p", 0.0, False, 1.0, True), ("min_p", 0.0, True, 1.0, False),
               ("repetition_penalty", 0.0, False, None, True))

    def __post_init__(self) -> None:
        for name, low, low_ok, high, high_ok in self._RANGES:
            v = getattr(self, name)
            below = v < low or (v == low and not low_ok)
            above = high is not None and (v > high or (v == high and not high_ok))
            if below or above:
                span = f"{'[' if low_ok else '('}{low}, {'inf' if high is None else high}{']' if high_ok and high is not None else ')'}"
                raise ValueError(f"{name} = {v!r} lies outside {span}")
        if self.top_k != -1 and self.top_k < 1:
            raise ValueError(f"top_k = {self.top_k!r}: -1 keeps every token, a positive number the k most probable")
        if self.stop:
            raise ValueError("stop strings need a detokenizer; this engine is token in, token out "
                             "(use stop_token_ids)")
        if self.top_logprobs is not None and not (1 <= self.top_logprobs <= 64):
            raise ValueError("top_logprobs must be between 1 and 64")
        if self.n != 1:
            raise ValueError("n must be 1; submit the prompt n times with different seeds")
        if self.logit_bias:
            self.logit_bias = {int(token): float(bias) for token, bias in dict(self.logit_bias).items()}
        else:
            self.logit_bias = None

    @property
    def greedy(self) -> bool:
        """Whether the most probable token is taken (temperature 0, or only one token kept)."""
        return self.top_k == 1 or self.temperature == 0

    @property
    def plain(self) -> bool:
        """Neither penalties nor bias touch the logits."""
        return (self.repetition_penalty == 1.0 and self.frequency_penalty == 0.0 and self.presence_penalty == 0.0
                and not self.logit_bias)
