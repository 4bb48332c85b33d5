"""Per-request sampling options.  Field names, defaults and accepted ranges are the
reference's (src/sparseengine/sampling_params.py:38-88), so that a caller's keyword
arguments carry over; the checks are a table of rules evaluated in one pass, and every
rule that fails is reported at once."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DEFAULT_MAX_TOKENS = 8192
GREEDY_EPS = 1e-10     # temperatures at or below this are greedy (src/sparseengine/layers/sampler.py:75)


def _token_tuple(value) -> tuple:
    """None, one id or an iterable of ids -> a tuple without repeats, first occurrence kept."""
    if value is None:
        return ()
    if isinstance(value, int) and not isinstance(value, bool):
        return (value,)
    seen, out = set(), []
    for t in value:
        t = int(t)
        if t not in seen:
            seen.add(t)
            out.append(t)
    return tuple(out)


def _is_token(t) -> bool:
    return type(t) is int and t >= 0


# (what is checked, rule over the record, what to tell the caller)
_RULES = (
    ("temperature", lambda p: p.temperature >= 0.0, "needs temperature >= 0 (0 means greedy)"),
    ("top_p", lambda p: 0.0 < p.top_p <= 1.0, "needs 0 < top_p <= 1 (1 keeps every token)"),
    ("top_k", lambda p: p.top_k >= 0, "needs top_k >= 0 (0 keeps every token)"),
    ("presence_penalty", lambda p: -2.0 <= p.presence_penalty <= 2.0, "needs -2 <= presence_penalty <= 2"),
    ("repetition_penalty", lambda p: p.repetition_penalty > 0.0, "needs repetition_penalty > 0 (1 means none)"),
    ("max_tokens", lambda p: p.max_tokens >= 1, "needs max_tokens >= 1"),
    ("eos_token_ids", lambda p: all(t >= 0 for t in p.eos_token_ids), "holds a negative token id"),
    ("logprobs", lambda p: p.logprobs is None or p.logprobs >= 0, "needs logprobs >= 0 or None"),
    ("benchmark_forced_token_ids",
     lambda p: p.benchmark_forced_token_ids is None or p.ignore_eos,
     "only works with ignore_eos=True (a forced end-of-sequence token would end the run early)"),
    ("benchmark_forced_token_ids",
     lambda p: p.benchmark_forced_token_ids is None or (
         isinstance(p.benchmark_forced_token_ids, (list, tuple))
         and len(p.benchmark_forced_token_ids) == p.max_tokens
         and all(_is_token(t) for t in p.benchmark_forced_token_ids)),
     "has to be a list of max_tokens token ids (plain ints >= 0), one per generated token"),
)


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
        self.eos_token_ids = _token_tuple(self.eos_token_ids)
        broken = [f"{name} {message}" for name, rule, message in _RULES if not rule(self)]
        if broken:
            raise ValueError("SamplingParams: " + "; ".join(broken))
        if self.benchmark_forced_token_ids is not None:
            self.benchmark_forced_token_ids = tuple(self.benchmark_forced_token_ids)

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_EPS

    @property
    def has_penalties(self) -> bool:
        return self.presence_penalty != 0.0 or self.repetition_penalty != 1.0

    def validate_for_vocab(self, vocab_size: int) -> None:
        """Forced tokens have to exist in the model's vocabulary (known only to the engine)."""
        outside = [t for t in (self.benchmark_forced_token_ids or ()) if t >= vocab_size]
        if outside:
            raise ValueError(f"SamplingParams: benchmark_forced_token_ids names token {outside[0]}, "
                             f"the vocabulary has {vocab_size}")
