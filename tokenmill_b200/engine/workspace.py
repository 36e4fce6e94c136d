"""Named scratch buffers that outlive a step: partial results of split attention, arrival counters,
whatever a part's kernels need beyond their inputs and outputs.

A part asks ``step.workspace.get(name, numel, dtype)`` while it runs. A buffer grows to the largest size
ever asked for under its name and never shrinks; buffers of different names grow independently, so layers
of different shapes may share a name (they get the largest) or use names of their own. Buffers asked for
with ``zeroed=True`` are zero when handed out for the first time; the kernels that use them as counters
leave them zero.

Captured CUDA graphs hold raw addresses. ``freeze()`` (called by the runner after a capture) marks every
buffer that exists as fixed: it keeps its address and size for good. A later request that needs more under
a frozen name (a mixed step of many tokens between graph replays, or a graph for a larger batch) gets
another buffer of that name, which may grow until it is frozen in turn; the graphs keep pointing at the
buffers they captured. Inside a capture nothing may be allocated: a request that the warm-up runs before
the capture did not already make raises.
"""

from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._gens: dict[str, list[torch.Tensor]] = {}     # per name: buffers by generation, all but the last frozen
        self._frozen: dict[str, int] = {}                  # per name: how many generations are frozen

    def get(self, name: str, numel: int, dtype: torch.dtype, *, zeroed: bool = False) -> torch.Tensor:
        numel = max(int(numel), 1)
        gens = self._gens.setdefault(name, [])
        for t in gens:
            if t.dtype != dtype:
                raise TypeError(f"workspace buffer {name!r} is {t.dtype}, asked for as {dtype}")
            if t.numel() >= numel:
                return t
        if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"workspace buffer {name!r} ({numel} elements) was not made before the capture")
        make = torch.zeros if zeroed else torch.empty
        t = make(numel, dtype=dtype, device=self.device)
        if len(gens) > self._frozen.get(name, 0):
            gens[-1] = t               # the last generation is nobody's captured address: let it grow
        else:
            gens.append(t)
        return t

    def freeze(self) -> None:
        """Every buffer that exists now keeps its address for good (a graph has captured it)."""
        for name, gens in self._gens.items():
            self._frozen[name] = len(gens)

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for gens in self._gens.values() for t in gens)
