"""Choosing the next token of every request that finished its portion of the step.

Greedy rows take the arg-max kernel; the others take the sampling kernel (temperature, top-k,
top-p, one inverse-CDF draw). As in the reference (src/infer/sampling.py:1-5,28-54) a request's
random stream is its own: it is keyed by the request's seed (``SamplingParams.seed``, or a number
drawn from the engine's seeded generator when the request gives none) and by how many tokens the
request has drawn so far, so its tokens do not depend on which other requests share the batch.
The stream itself is this engine's (a counter-based generator on the host), not torch's.
"""

from __future__ import annotations

import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, draw: int) -> float:
    """The draw-th uniform number in [0, 1) of the stream keyed by ``seed``; 24 random bits, so the
    value is exact in float32."""
    return (_mix(_mix(seed & _MASK) ^ ((draw * 0xD1B54A32D192ED03) & _MASK)) >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: list, seeds: list[int], draws: list[int]) -> list[int]:
        """logits [n, V] float32 on the device; one entry of params / seeds / draws per row."""
        n = logits.shape[0]
        if n == 0:
            return []
        greedy = ops.argmax(logits)
        random_rows = [i for i, p in enumerate(params) if not p.greedy]
        if not random_rows:
            return greedy.tolist()
        host = torch.empty((4, len(random_rows)), dtype=torch.float32, pin_memory=True)
        for j, i in enumerate(random_rows):
            p = params[i]
            host[0, j] = p.temperature
            host[1, j] = p.top_p
            host[2, j] = uniform_for(seeds[i], draws[i])
            host[3, j] = float(i)
        ints = torch.tensor([[params[i].top_k for i in random_rows], random_rows], dtype=torch.int32,
                            pin_memory=True)
        dev = host.to(self.device, non_blocking=True)
        dev_i = ints.to(self.device, non_blocking=True)
        drawn = ops.sample(logits, dev[0], dev_i[0], dev[1], dev[2], rows=dev_i[1])
        tokens = greedy.tolist()
        for j, tok in zip(random_rows, drawn.tolist()):
            tokens[j] = tok
        return tokens
