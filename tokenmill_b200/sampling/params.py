"""Sampling parameters of one request, with the reference's names, defaults and meaning
(src/infer/engine/sequence.py:19-31): greedy when ``temperature <= 1e-5`` or ``top_k == 1``.
``stop`` strings belong to the reference's text API and are not part of this token-id engine.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = -1
    seed: int | None = None
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must lie in (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 1e-5 or self.top_k == 1
