"""Interfaces every part implements, and the objects a part sees at run time.

A part is built from ``PartSpec.params`` only (sizes and constants), declares the checkpoint tensors
it needs relative to its layer's prefix, receives them through ``bind``, and then runs on flat
``[T, ...]`` batches. It is given a ``StepInputs`` (which token belongs to which request, where it
sits) and, for mixers, a ``LayerCache`` (this run-order entry's pages and per-request state). No
part knows which model it is in, or which layer.

What the engine knows about a part it learns by asking, never by looking at the part's attributes:

* ``cache_need()`` / ``state_need()``: pages and fixed-size per-request state (mixers);
* ``step_metadata(shape)``: integer arrays and host-side numbers the part wants prepared for every step
  (work lists for its kernels, scan boundaries, ...). The engine packs the arrays into the step's one
  host-to-device copy and hands them back as ``step.meta[part.metadata_key()]``; parts that return the
  same key share one set;
* ``max_positions()`` / ``limit_positions(n)``: how far the part's position tables reach, and the chance
  to size them for the engine's own limit before the weights are bound;
* ``activation_bytes(n_tokens)``: working memory a step of that many tokens needs inside the part (the
  cache budget leaves room for it).

All of these are optional; ``part_*`` helpers below supply the defaults.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Hashable, NamedTuple, Protocol

import numpy as np
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
    """Work units of the tensor-core prompt attention for one group size (parts/attention_plan.py
    packed_units): one 8-int record per unit (a tile of tile_rows rows of one request times one chunk of
    chunk_keys keys), heaviest first; n_slots partial-result slots (of tile_rows rows) are needed, for
    n_tiles row tiles."""

    records: torch.Tensor
    n_units: int
    n_tiles: int
    n_slots: int
    chunk_keys: int
    tile_rows: int = 64


@dataclass
class StepShape:
    """What a part's ``step_metadata`` is told about the step at hand (host side, numpy).

    Request s brings q_lens[s] tokens that continue it at position starts[s]. ``max_kv_len`` is the
    longest context the metadata has to serve: the step's own, or, when ``for_graph`` is set, the
    engine's limit, because the arrays and numbers are then captured once in a CUDA graph that later
    replays steps of the same q_lens with other starts."""

    q_lens: np.ndarray
    starts: np.ndarray
    page_size: int
    max_kv_len: int
    for_graph: bool = False


@dataclass
class StepMetadata:
    """A part's answer: ``arrays`` are int32 numpy arrays (any shape; they reach the device inside the
    step's packed buffer), ``host`` holds numbers that stay on the host (launch sizes and the like).
    ``constant_in_graph``: a captured decode graph fills the arrays once instead of at every replay
    (they do not depend on ``starts``)."""

    arrays: dict[str, np.ndarray] = field(default_factory=dict)
    host: dict[str, Any] = field(default_factory=dict)
    constant_in_graph: bool = False


@dataclass
class PartMeta:
    """A part's step metadata as the part sees it at run time: the arrays as device tensors."""

    arrays: dict[str, torch.Tensor]
    host: dict[str, Any]


class Workspace(Protocol):
    """Named scratch buffers the engine keeps between steps (engine/workspace.py)."""

    def get(self, name: str, numel: int, dtype: torch.dtype, *, zeroed: bool = False) -> torch.Tensor: ...


@dataclass
class StepInputs:
    """One step's batch, already on the device (int32 everywhere).

    Tokens of all requests lie side by side: request s owns flat rows cu_q[s] .. cu_q[s+1]-1, at
    absolute positions kv_before[s] + 0, 1, ... ; kv_before[s] tokens of it are already in the cache.
    A decoded token is a request with one row. The host-side lists mirror the device tensors for
    parts that plan on the host; they are None when a captured graph replays the step.
    ``meta`` holds what the parts asked for through ``step_metadata``, by their ``metadata_key()``;
    ``workspace`` lends named scratch buffers that survive the step."""

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
    meta: dict[Hashable, PartMeta] = field(default_factory=dict)
    workspace: Any = None              # engine-owned provider of named scratch buffers (Workspace)
    logits_out: torch.Tensor | None = None   # where a step program writes the logits ([n_want, vocab] float32)


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
    """Either of two forms. ``tables(device)`` returns (cos, sin), each [positions, head_dim / 2] float32,
    for the rotate-half kernels (fused into the projection's epilogue), or None. An encoding without
    tables has ``apply(q, k, positions)``: q [T, heads, head_dim] and k [T, kv_heads, head_dim] in the
    run's dtype, bias already added, changed in place by whatever kernel the part brings, before k is
    written to the cache. ``max_positions`` (attribute) and ``limit_positions(n)`` are optional."""

    def tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor] | None: ...


# --- defaults for what a part may leave out ---------------------------------------------------------------

def part_max_positions(part) -> int | None:
    """Positions the part can serve (None: no limit of its own)."""
    fn = getattr(part, "max_positions", None)
    if callable(fn):
        return fn()
    return fn if isinstance(fn, int) else None


def part_limit_positions(part, n: int) -> None:
    fn = getattr(part, "limit_positions", None)
    if callable(fn):
        fn(int(n))


def part_activation_bytes(part, n_tokens: int, hidden_size: int) -> int:
    """Working memory of one step inside the part; a part that does not say is taken to need four
    rows of the hidden size in 32-bit per token."""
    fn = getattr(part, "activation_bytes", None)
    if callable(fn):
        return int(fn(int(n_tokens)))
    return 16 * hidden_size * int(n_tokens)


def part_metadata_key(part) -> Hashable | None:
    """The key under which the part's step metadata is kept, or None when it asks for none."""
    if not callable(getattr(part, "step_metadata", None)):
        return None
    fn = getattr(part, "metadata_key", None)
    return fn() if callable(fn) else ("part", id(part))
