"""Interfaces every part implements, and the two objects a part sees at run time.

A part is built from ``PartSpec.params`` only (sizes and constants), declares the checkpoint tensors
it needs relative to its layer's prefix, receives them through ``bind``, and then runs on flat
``[T, ...]`` batches. It is given a ``StepInputs`` (which token belongs to which request, where it
sits) and, for mixers, a ``LayerCache`` (this run-order entry's pages and per-request state). No
part knows which model it is in, or which layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, NamedTuple, Protocol

import torch

from .spec import PagedKVNeed, StateNeed, WeightSpec


@dataclass
class LayerCache:
    """What one run-order entry may touch in the cache.

    k, v: [pages, page_size, kv_heads, head_dim] views of the entry's group pool (None for a mixer
    without paged needs). group: index of the block-table / slot-map set in StepInputs. writes:
    False when the entry reads another entry's cache. state: [slots, *shape] per-request state."""

    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    group: int = 0
    writes: bool = True
    state: torch.Tensor | None = None


class PrefillUnits(NamedTuple):
    """Work units of the tensor-core prompt attention for one group size (engine/batch.py packed_units):
    one 8-int record per unit (a tile of tile_rows rows of one request times one chunk of chunk_keys keys),
    heaviest first; n_slots partial-result slots (of tile_rows rows) are needed, for n_tiles row tiles."""

    records: torch.Tensor
    n_units: int
    n_tiles: int
    n_slots: int
    chunk_keys: int
    tile_rows: int = 64


@dataclass
class StepInputs:
    """One step's batch, already on the device (int32 everywhere).

    Tokens of all requests lie side by side: request s owns flat rows cu_q[s] .. cu_q[s+1]-1, at
    absolute positions kv_before[s] + 0, 1, ... ; kv_before[s] tokens of it are already in the cache.
    A decoded token is a request with one row. The host-side lists mirror the device tensors for
    parts that plan on the host; they are None when a captured graph replays the step."""

    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T]
    seq_of_token: torch.Tensor         # [T]
    cu_q: torch.Tensor                 # [S + 1]
    kv_before: torch.Tensor            # [S]
    state_slots: torch.Tensor          # [S]
    block_tables: list[torch.Tensor]   # per cache group: [S, W]
    slot_maps: list[torch.Tensor]      # per cache group: [T]
    want_rows: torch.Tensor            # [n_want] flat rows whose logits are asked for
    n_want: int
    max_q_len: int
    max_kv_len: int
    q_lens: list[int] | None = None
    kv_befores: list[int] | None = None
    tiles: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = field(default_factory=dict)
    prefill: dict[int, PrefillUnits] = field(default_factory=dict)     # by group size
    scratch: Any = None                # engine-owned scratch provider (attention partials)
    logits_out: torch.Tensor | None = None   # where a step program writes the logits ([n_want, vocab] float32)
    split_keys: int = 0                # > 0: short-query attention cuts keys at multiples of this
    max_splits: int = 0                # number of such cuts the step may need

    def attention_tiles(self, group_size: int) -> tuple[torch.Tensor, torch.Tensor, int]:
        """(tile_seq, tile_row0, n_tiles) for tiles of 32 (token, head-in-group) rows."""
        return self.tiles[group_size]


class Part(Protocol):
    def weight_specs(self) -> list[WeightSpec]:
        """Checkpoint tensors, named relative to the part's prefix."""
        ...

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the loaded tensors (same relative names), already on the device."""
        ...


class Mixer(Part, Protocol):
    def cache_need(self) -> PagedKVNeed | None: ...
    def state_need(self) -> StateNeed | None: ...
    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        """x [T, H] normed input -> branch output [T, H]."""
        ...


class FeedForward(Part, Protocol):
    def forward(self, x: torch.Tensor, step: StepInputs) -> torch.Tensor: ...


class Norm(Part, Protocol):
    def forward(self, resid: torch.Tensor, out: torch.Tensor, *, branch: torch.Tensor | None = None,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """Fused (embedding gather | residual add) + norm over the 32-bit residual stream."""
        ...


class PositionEncoding(Protocol):
    def tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]: ...
