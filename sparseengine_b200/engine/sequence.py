"""A request's state between steps (cf. src/sparseengine/engine/sequence.py:87-483)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from ..sampling.params import SamplingParams


class Status(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


@dataclass
class Sequence:
    seq_id: int
    prompt_ids: list
    params: SamplingParams
    output_ids: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    top_logprobs: list = field(default_factory=list)     # per produced token: {token id: log-probability} or None
    num_computed: int = 0          # tokens whose keys/values are in the cache
    status: Status = Status.WAITING
    preemptions: int = 0
    finish_reason: str = ""

    @property
    def tokens(self) -> list:
        return self.prompt_ids + self.output_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def remaining(self) -> int:
        """Tokens that still have to go through the model before the next sample."""
        return self.num_tokens - self.num_computed

    @property
    def in_decode(self) -> bool:
        return self.remaining == 1 and self.num_computed > 0 and len(self.output_ids) > 0

    def slice(self, start: int, n: int) -> list:
        """Tokens ``start .. start+n`` of prompt + output without building the whole list."""
        lp = len(self.prompt_ids)
        if start >= lp:
            return self.output_ids[start - lp:start - lp + n]
        if start + n <= lp:
            return self.prompt_ids[start:start + n]
        return self.prompt_ids[start:] + self.output_ids[:start + n - lp]
