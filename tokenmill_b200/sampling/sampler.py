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


class PendingSample:
    """Tokens a launch has chosen but the host has not read yet: ``dev`` (int32, one entry per logits row)
    can feed the next step on the device; ``Sampler.collect`` waits for the copy and returns the list."""

    __slots__ = ("dev", "host", "event", "n")

    def __init__(self, dev: torch.Tensor, host: torch.Tensor, event: torch.cuda.Event, n: int):
        self.dev, self.host, self.event, self.n = dev, host, event, n


class Sampler:
    RING = 4              # launches whose tokens may be outstanding at once
    MAX_ROWS = 4096

    def __init__(self, device: torch.device):
        self.device = device
        self._ring: list[tuple[torch.Tensor, torch.Tensor, torch.cuda.Event]] = []
        self._at = 0

    def _slot(self, n: int):
        if n > self.MAX_ROWS:        # wider than the ring's buffers: a one-off pair
            return (torch.empty(n, dtype=torch.int32, device=self.device),
                    torch.empty(n, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
        if not self._ring:
            self._ring = [(torch.zeros(self.MAX_ROWS, dtype=torch.int32, device=self.device),
                           torch.zeros(self.MAX_ROWS, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                          for _ in range(self.RING)]
        slot = self._ring[self._at]
        self._at = (self._at + 1) % self.RING
        slot[2].synchronize()          # the copy that last wrote this pinned buffer is done (and was read)
        return slot

    def launch(self, logits: torch.Tensor, params: list, seeds: list[int], draws: list[int]) -> PendingSample:
        """Choose a token for every row of logits [n, V] (float32, on the device) without waiting for the
        result: greedy rows by the arg-max kernel, the others by the sampling kernel, which writes its
        draws into the same device array; then one asynchronous copy to pinned host memory."""
        n = logits.shape[0]
        dev, host, event = self._slot(n)
        if n:
            ops.argmax(logits, out=dev[:n])
            random_rows = [i for i, p in enumerate(params) if not p.greedy]
            if random_rows:
                m = len(random_rows)
                hp = torch.empty((4, m), dtype=torch.float32, pin_memory=True)
                for j, i in enumerate(random_rows):
                    p = params[i]
                    hp[0, j] = p.temperature
                    hp[1, j] = p.top_p
                    hp[2, j] = uniform_for(seeds[i], draws[i])
                ints = torch.tensor([[params[i].top_k for i in random_rows], random_rows], dtype=torch.int32,
                                    pin_memory=True)
                dp = hp.to(self.device, non_blocking=True)
                di = ints.to(self.device, non_blocking=True)
                ops.sample(logits, dp[0], di[0], dp[1], dp[2], rows=di[1], out=dev, scatter=True)
            host[:n].copy_(dev[:n], non_blocking=True)
        event.record()
        return PendingSample(dev, host, event, n)

    def launch_filled(self, n: int, fill) -> PendingSample:
        """As ``launch`` for a step whose tokens a kernel writes itself: ``fill(dev)`` is called with the int32
        device array to write its n tokens into (the output matrix's arg-max epilogue does)."""
        dev, host, event = self._slot(n)
        fill(dev)
        host[:n].copy_(dev[:n], non_blocking=True)
        event.record()
        return PendingSample(dev, host, event, n)

    def collect(self, pending: PendingSample) -> list[int]:
        pending.event.synchronize()
        return pending.host[:pending.n].tolist()

    def sample(self, logits: torch.Tensor, params: list, seeds: list[int], draws: list[int]) -> list[int]:
        """logits [n, V] float32 on the device; one entry of params / seeds / draws per row."""
        if logits.shape[0] == 0:
            return []
        return self.collect(self.launch(logits, params, seeds, draws))
