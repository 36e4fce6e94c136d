"""Request state shared by the scheduler and the engine (src/infer/engine/sequence.py:11-105)."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from ..cache.manager import CacheHandle
from ..sampling.params import SamplingParams


PLACEHOLDER = -1        # stands in a request's output list for a token that is chosen but not read yet


class Status(Enum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2      # pages released; resumes by recomputing prompt + generated tokens
    FINISHED = 3


@dataclass(eq=False)          # identity semantics: two requests with equal fields are still two requests
class Sequence:
    id: str
    prompt_ids: list[int]
    params: SamplingParams
    cache: CacheHandle
    output_ids: list[int] = field(default_factory=list)
    status: Status = Status.WAITING
    arrival_time: float = 0.0
    first_token_time: float | None = None
    finish_time: float | None = None
    finish_reason: str | None = None          # stop | length | abort
    num_computed_tokens: int = 0              # tokens whose keys and values are in the cache
    admit_order: int = -1                     # grows on every (re)admission; the newest is preempted first
    num_preemptions: int = 0
    sample_seed: int = 0                      # key of the request's random stream
    num_draws: int = 0                        # random draws taken so far
    finishing: bool = False                   # ends with a step already launched: not scheduled again

    def __repr__(self) -> str:
        return (f"Sequence({self.id!r}, {self.status.name}, prompt={len(self.prompt_ids)}, "
                f"out={len(self.output_ids)}, computed={self.num_computed_tokens})")

    @property
    def length(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_ids + self.output_ids

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_ids)

    @property
    def last_token(self) -> int:
        return self.output_ids[-1] if self.output_ids else self.prompt_ids[-1]

    @property
    def num_new_tokens(self) -> int:
        """Tokens the next forward pass has to run for this request: the whole uncached tail."""
        return self.length - self.num_computed_tokens

    @property
    def awaits_token(self) -> bool:
        """Its last token is still on the device (a decode step in flight): the ids are not all known."""
        return bool(self.output_ids) and self.output_ids[-1] == PLACEHOLDER

    @property
    def is_finished(self) -> bool:
        return self.status == Status.FINISHED


@dataclass
class RequestOutput:
    """One engine step's result for one request."""

    request_id: str
    new_token_ids: list[int]
    finished: bool
    finish_reason: str | None
    num_prompt_tokens: int
    num_output_tokens: int
    arrival_time: float = 0.0
    first_token_time: float | None = None
    finish_time: float | None = None
    num_preemptions: int = 0
    error: str | None = None
