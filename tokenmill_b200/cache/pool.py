"""The device memory the cache manager's page numbers refer to.

One tensor per group, ``[entries, 2 (K and V), pages, page_size, kv_heads, head_dim]`` in the run's
dtype (the reference keeps one such tensor for all layers, src/infer/kv/paged_cache.py:25-34), and
one tensor per stateful run-order entry, ``[slots, *shape]``. A ``sink`` page may be appended to each
group, and a sink slot to the state tensors: padded rows of a captured decode graph write there, and the
manager never hands them out (src/infer/engine/cuda_graphs.py:56-58).
"""

from __future__ import annotations

import torch

from ..parts.base import LayerCache
from ..parts.model import CacheLayout

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CachePools:
    def __init__(self, layout: CacheLayout, num_pages: list[int], page_size: int, dtype: torch.dtype,
                 device: torch.device, num_state_slots: int = 0, sink_page: bool = False,
                 run_order_cache_of: list[int | None] | None = None):
        self.layout, self.page_size, self.dtype, self.device = layout, page_size, dtype, device
        self.num_pages = list(num_pages)
        extra = 1 if sink_page else 0
        self.sink = [n if sink_page else -1 for n in num_pages]       # page index of the sink per group
        self.kv = [torch.zeros((len(g.entries), 2, n + extra, page_size, g.need.kv_heads, g.need.head_dim),
                               dtype=dtype, device=device)
                   for g, n in zip(layout.groups, num_pages)]
        self.state_sink = num_state_slots if sink_page else -1        # index of the sink state slot
        self.state = {pos: torch.zeros((max(num_state_slots, 1) + extra, *need.shape), dtype=_STATE_DTYPES[need.dtype],
                                       device=device)
                      for pos, need in layout.entry_state.items()}
        self._cache_of = run_order_cache_of or []

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.state.values())

    def layer_caches(self, n_entries: int) -> list[LayerCache]:
        """One LayerCache per run-order entry."""
        out = []
        for pos in range(n_entries):
            lc = LayerCache()
            if pos in self.layout.entry_group:
                g, idx = self.layout.entry_group[pos]
                lc.k, lc.v, lc.group = self.kv[g][idx, 0], self.kv[g][idx, 1], g
                lc.writes = not (pos < len(self._cache_of) and self._cache_of[pos] is not None)
            lc.state = self.state.get(pos)
            out.append(lc)
        return out

    def zero_state(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()
