"""Data that describes a model: which parts each layer is made of, and in which order layers run.

Nothing here computes. An architecture's builder turns its typed configuration into a ``ModelSpec``;
``parts.model.DecoderModel`` turns the spec into parts through the registry. Every size and constant
a part needs travels in ``PartSpec.params``, so a part never looks at a model configuration.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class WeightSpec:
    """One tensor of the checkpoint, by its safetensors name.

    dtype: "compute" - held in the run's dtype (bfloat16 or float32);
           "float32" - held in 32-bit whatever the run's dtype (norm weights, biases: small vectors
                       whose arithmetic is 32-bit in the kernels);
           "int32"   - an integer table.
    init:  how the random-weights writer fills it: ("normal", std) or ("ones_plus_normal", std).
    """

    name: str
    shape: tuple[int, ...]
    dtype: str = "compute"
    init: tuple[str, float] = ("normal", 0.02)


@dataclass(frozen=True)
class PagedKVNeed:
    """A mixer that keeps per-token keys and values. window=None: all keys stay; window=w: a query at
    position p reads keys p-w+1..p only, and pages wholly behind every future window are given back."""

    kv_heads: int
    head_dim: int
    window: int | None = None

    def group_key(self) -> tuple:
        return ("paged_kv", self.kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a fixed-size state per request (zeroed when the request is admitted)."""

    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind a norm, put together by a block kind.
    ``prefix`` is the checkpoint-name prefix of the layer's tensors ("model.layers.3")."""

    prefix: str
    block: str                      # arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    mixer_name: str = "self_attn"                       # checkpoint sub-prefix of each part's tensors
    feed_forward_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    feed_forward_norm_name: str = "post_attention_layernorm"


@dataclass(frozen=True)
class RunEntry:
    """One stop in the order layers run. ``layer`` indexes ``ModelSpec.layers`` and may appear in
    several entries (the same weights run twice; each run keeps a cache of its own). ``cache_of``
    names an EARLIER entry (by its place in the run order) whose cache this entry reads instead of
    keeping one."""

    layer: int
    cache_of: int | None = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding_name: str
    layers: list[LayerSpec]
    run_order: list[RunEntry]
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_name: str | None          # None: the output matrix is the embedding (tied)
    max_positions: int
    eos_token_ids: list[int] = field(default_factory=list)
    ignored_name_patterns: tuple[str, ...] = ()   # checkpoint names that may be present and are not loaded

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.run_order):
            if not (0 <= e.layer < n):
                raise ValueError(f"run_order[{i}] names layer {e.layer}, the model has {n}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"run_order[{i}].cache_of={e.cache_of} must name an earlier entry")
                if self.run_order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run_order[{i}].cache_of={e.cache_of} names an entry that has no cache "
                                     f"of its own")
