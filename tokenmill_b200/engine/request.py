"""One generation request as the engine keeps it, and what a step reports about it.

The fields a user of the reference knows are here under the same meaning (prompt ids, output ids, sampling
parameters, finish reason, counts of tokens and preemptions: src/infer/engine/sequence.py:11-105); what is
this engine's own is the rest: the cache handle (page tables per cache group and a state slot), the count of
tokens whose keys and values are already in the cache, the per-request random stream, and the place kept in
the output list for a token that a launched step has chosen but the host has not read yet.
"""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field

from ..cache.manager import CacheHandle
from ..sampling.params import SamplingParams

TOKEN_IN_FLIGHT = -1      # stands in ``output_ids`` for a token that is on the device and not yet on the host


class Phase(enum.Enum):
    QUEUED = "queued"       # waits for admission; holds nothing
    RUNNING = "running"     # holds pages (and a state slot); takes part in steps
    EVICTED = "evicted"     # gave its pages back under pressure; queued again, everything is recomputed
    DONE = "done"


@dataclass
class RequestTimes:
    """Monotonic clock readings (seconds); None until the event has happened."""

    arrival: float = 0.0
    first_token: float | None = None
    finish: float | None = None


@dataclass(eq=False)        # a request is itself, whatever its fields hold
class Request:
    id: str
    prompt_ids: list[int]
    params: SamplingParams
    cache: CacheHandle
    output_ids: list[int] = field(default_factory=list)
    phase: Phase = Phase.QUEUED
    finish_reason: str | None = None          # "stop", "length" or "abort" once done
    cached_tokens: int = 0                    # leading tokens whose keys and values the cache holds
    seat: int = -1                            # stamp of the latest admission: the highest seat is evicted first
    evictions: int = 0
    sample_seed: int = 0                      # key of the request's random stream (sampling/sampler.py)
    draws: int = 0                            # uniforms taken from that stream so far
    closing: bool = False                     # the step in flight brings its last token: plan it no further
    times: RequestTimes = field(default_factory=lambda: RequestTimes(arrival=time.monotonic()))

    def __repr__(self) -> str:
        return (f"Request({self.id!r}, {self.phase.value}, {self.n_prompt} + {self.n_output} tokens, "
                f"{self.cached_tokens} cached)")

    @property
    def n_prompt(self) -> int:
        return len(self.prompt_ids)

    @property
    def n_output(self) -> int:
        return len(self.output_ids)

    @property
    def n_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def tokens(self) -> list[int]:
        """Prompt and outputs in one list (what an evicted request recomputes)."""
        return self.prompt_ids + self.output_ids

    @property
    def backlog(self) -> int:
        """Tokens the cache does not hold yet: the next steps have to run these."""
        return self.n_tokens - self.cached_tokens

    @property
    def awaits_token(self) -> bool:
        """The newest output is still on the device, so the ids are not all known on the host."""
        return bool(self.output_ids) and self.output_ids[-1] == TOKEN_IN_FLIGHT

    @property
    def done(self) -> bool:
        return self.phase is Phase.DONE


@dataclass(frozen=True)
class RequestOutput:
    """What one engine step has to say about one request: the tokens it added, and where the request
    stands. ``error`` is set when the request ended without being served."""

    request_id: str
    new_token_ids: list[int]
    finished: bool
    finish_reason: str | None = None
    error: str | None = None
    num_prompt_tokens: int = 0
    num_output_tokens: int = 0
    num_preemptions: int = 0
    times: RequestTimes | None = None
