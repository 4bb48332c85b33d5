"""Per-request sampling options, with the reference's names, defaults and checks
(src/sparseengine/sampling_params.py:38-88)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DEFAULT_MAX_TOKENS = 8192
GREEDY_EPS = 1e-10     # temperatures at or below this are greedy (src/sparseengine/layers/sampler.py:75)


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = DEFAULT_MAX_TOKENS
    ignore_eos: bool = False
    eos_token_ids: object = None
    logprobs: Optional[int] = None
    benchmark_forced_token_ids: Optional[tuple] = None

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError("temperature must be non-negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be non-negative")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError("presence_penalty must be in [-2, 2]")
        if not self.repetition_penalty > 0.0:
            raise ValueError("repetition_penalty must be positive")
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if self.eos_token_ids is None:
            self.eos_token_ids = ()
        elif isinstance(self.eos_token_ids, int):
            self.eos_token_ids = (int(self.eos_token_ids),)
        else:
            self.eos_token_ids = tuple(dict.fromkeys(int(t) for t in self.eos_token_ids))
        if any(t < 0 for t in self.eos_token_ids):
            raise ValueError("eos_token_ids must contain non-negative token ids")
        if self.logprobs is not None and self.logprobs < 0:
            raise ValueError("logprobs must be non-negative")
        forced = self.benchmark_forced_token_ids
        if forced is not None:
            if not self.ignore_eos:
                raise ValueError("benchmark_forced_token_ids requires ignore_eos")
            if (not isinstance(forced, (list, tuple)) or len(forced) != self.max_tokens
                    or any(type(t) is not int or t < 0 for t in forced)):
                raise ValueError("benchmark_forced_token_ids must contain exactly max_tokens nonnegative integers")
            self.benchmark_forced_token_ids = tuple(forced)

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_EPS

    @property
    def has_penalties(self) -> bool:
        return self.presence_penalty != 0.0 or self.repetition_penalty != 1.0

    def validate_for_vocab(self, vocab_size: int) -> None:
        forced = self.benchmark_forced_token_ids
        if forced is not None and any(t >= vocab_size for t in forced):
            raise ValueError(f"benchmark_forced_token_ids contains a token outside the vocabulary ({vocab_size})")
