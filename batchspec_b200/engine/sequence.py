"""A request as the scheduler sees it (the reference's record:
batchspec/backends/continuous/sequence.py:8-33, with the token buffer on the host
and per-request limits and sampling settings added)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional


class Status(Enum):
    PENDING = "pending"      # waiting for admission (or preempted and waiting again)
    PREFILL = "prefill"      # live; more than one known token not yet in the cache
    DECODE = "decode"        # live; exactly the last known token is not yet in the cache
    COMPLETE = "complete"
    FAILED = "failed"        # could never run (too long for the model or the cache)


@dataclass
class Sequence:
    seq_id: int
    prompt_ids: List[int]
    max_new_tokens: int
    temperature: Optional[float] = None      # None: the engine's setting
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    status: Status = Status.PENDING
    output_ids: List[int] = field(default_factory=list)
    num_computed: int = 0                     # tokens of prompt+output already in the cache
    finish_reason: Optional[str] = None       # "eos" | "length" | "context" | error text
    num_preemptions: int = 0
    admitted_at: int = -1                     # admission counter, for the preemption order

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_ids)

    @property
    def num_generated_tokens(self) -> int:
        return len(self.output_ids)

    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    def known_token(self, i: int) -> int:
        n = len(self.prompt_ids)
        return self.prompt_ids[i] if i < n else self.output_ids[i - n]

    def known_tokens(self, start: int, stop: int) -> List[int]:
        n = len(self.prompt_ids)
        if stop <= n:
            return list(self.prompt_ids[start:stop])
        if start >= n:
            return list(self.output_ids[start - n:stop - n])
        return list(self.prompt_ids[start:]) + list(self.output_ids[:stop - n])

    def get_id(self) -> int:
        return self.seq_id
