"""A decoder built from a ``ModelSpec``: embedding, the layers in their run order, final norm,
output matrix. Every part comes from the registry by the kind its spec names, layer by layer, so
one model may mix different mixers and feed-forwards, run a layer twice, or let a layer read
another's cache.

Run (src/infer/model/qwen2.py:43-52): ``x = E[ids]``; each run-order entry's block; final norm on
the wanted rows only (src/infer/engine/model_runner.py:94-96); ``logits = h . W_out^T`` with
``W_out`` the embedding itself when the spec has no lm_head (tied, qwen2.py:39-41). Logits are 32-bit.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops
from ..registry import get_part
from .base import (LayerCache, StepInputs, part_activation_bytes, part_limit_positions, part_max_positions)
from .block import Pending
from .spec import LayerSpec, ModelSpec, PagedKVNeed, PartSpec, StateNeed, WeightSpec


@dataclass
class CacheGroup:
    """Run-order entries whose mixers keep the same kind of pages; they share block tables."""

    need: PagedKVNeed
    entries: list[int]          # run-order positions that own a cache in this group


@dataclass
class CacheLayout:
    groups: list[CacheGroup]
    entry_group: dict[int, tuple[int, int]]   # run-order position -> (group, index within group)
    entry_state: dict[int, StateNeed]         # run-order position -> per-request state need

    def bytes_per_token(self, elt_bytes: int) -> int:
        return sum(2 * len(g.entries) * g.need.kv_heads * g.need.head_dim * elt_bytes for g in self.groups)

    @property
    def windows(self) -> list[int | None]:
        return [g.need.window for g in self.groups]


def _build(role: str, spec: PartSpec, dtype: torch.dtype, device: torch.device):
    return get_part(role, spec.kind)(dtype=dtype, device=device, **spec.params)


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, device
        self.blocks = []
        self._named: list[tuple[str, object]] = []     # (checkpoint prefix, part)
        for layer in spec.layers:
            mixer = _build("mixer", layer.mixer, dtype, device)
            ffn = _build("feed_forward", layer.feed_forward, dtype, device)
            n1 = _build("norm", layer.mixer_norm, dtype, device)
            n2 = _build("norm", layer.feed_forward_norm, dtype, device)
            self.blocks.append(get_part("block", layer.block)(mixer, ffn, n1, n2))
            self._named += [(f"{layer.prefix}.{layer.mixer_name}", mixer),
                            (f"{layer.prefix}.{layer.feed_forward_name}", ffn),
                            (f"{layer.prefix}.{layer.mixer_norm_name}", n1),
                            (f"{layer.prefix}.{layer.feed_forward_norm_name}", n2)]
        self.final_norm = _build("norm", spec.final_norm, dtype, device)
        self._named.append((spec.final_norm_prefix, self.final_norm))
        self.embedding: torch.Tensor | None = None
        self.output_weight: torch.Tensor | None = None

    # --- weights --------------------------------------------------------------------------------

    def weight_specs(self) -> list[WeightSpec]:
        """Every checkpoint tensor, by full name, in a fixed order (the random-weights writer
        draws them in this order)."""
        s = self.spec
        out = [WeightSpec(s.embedding_name, (s.vocab_size, s.hidden_size))]
        for prefix, part in self._named:
            out += [WeightSpec(f"{prefix}.{w.name}", w.shape, w.dtype, w.init) for w in part.weight_specs()]
        if s.lm_head_name is not None:
            out.append(WeightSpec(s.lm_head_name, (s.vocab_size, s.hidden_size)))
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_name]
        self.output_weight = self.embedding if s.lm_head_name is None else tensors[s.lm_head_name]
        for prefix, part in self._named:
            part.bind({w.name: tensors[f"{prefix}.{w.name}"] for w in part.weight_specs()})

    # --- what the engine asks the parts -----------------------------------------------------------

    def parts(self) -> list:
        """Every part of the model, layer by layer (mixer, feed-forward, the two norms), then the final norm."""
        out = []
        for blk in self.blocks:
            out += [blk.mixer, blk.feed_forward, blk.mixer_norm, blk.feed_forward_norm]
        return out + [self.final_norm]

    def max_positions(self) -> int:
        """The longest sequence the model can serve: the architecture's own limit, or less where a part's
        position tables are shorter."""
        limits = [self.spec.max_positions] + [n for n in (part_max_positions(p) for p in self.parts()) if n is not None]
        return min(limits)

    def limit_positions(self, n: int) -> None:
        """Tell the parts, before the weights are bound, that no position >= n will be asked for, so that
        position tables are sized for the engine's own limit (src/infer/model/qwen2.py:34)."""
        for p in self.parts():
            part_limit_positions(p, n)

    def activation_bytes(self, n_tokens: int) -> int:
        """Working memory of a step of n_tokens: the 32-bit residual stream, a normed copy, and the largest
        layer's own need (layers run one after another and reuse the memory)."""
        H = self.spec.hidden_size
        per_layer = max((part_activation_bytes(b.mixer, n_tokens, H) + part_activation_bytes(b.feed_forward, n_tokens, H)
                         for b in self.blocks), default=0)
        return n_tokens * H * 8 + per_layer

    # --- cache needs ----------------------------------------------------------------------------

    def cache_layout(self) -> CacheLayout:
        groups: list[CacheGroup] = []
        by_key: dict[tuple, int] = {}
        entry_group: dict[int, tuple[int, int]] = {}
        entry_state: dict[int, StateNeed] = {}
        for pos, entry in enumerate(self.spec.run_order):
            mixer = self.blocks[entry.layer].mixer
            need = mixer.cache_need()
            if entry.cache_of is not None:
                owner = self.blocks[self.spec.run_order[entry.cache_of].layer].mixer.cache_need()
                if need is None or owner is None or need.group_key() != owner.group_key():
                    raise ValueError(f"run_order[{pos}] reads the cache of entry {entry.cache_of}, whose pages "
                                     f"have a different shape")
                entry_group[pos] = entry_group[entry.cache_of]
            elif need is not None:
                g = by_key.setdefault(need.group_key(), len(groups))
                if g == len(groups):
                    groups.append(CacheGroup(need, []))
                entry_group[pos] = (g, len(groups[g].entries))
                groups[g].entries.append(pos)
            st = mixer.state_need()
            if st is not None:
                entry_state[pos] = st
        return CacheLayout(groups, entry_group, entry_state)

    # --- run ------------------------------------------------------------------------------------

    def program(self, caches: list[LayerCache], capacity: int):
        """The whole forward pass as a step program for steps of up to ``capacity`` tokens
        (kernels/program.py), or None when the model is not bfloat16 or one of its parts cannot write its
        launches down (it has no ``emit``). The program's last launch writes the logits to the address in the
        step parameter "logits" ([n_want, vocab] float32, which the caller allocates)."""
        from ..kernels.program import OP_GEMM_BF16, ProgramBuilder
        s = self.spec
        parts = [p for blk in self.blocks for p in (blk, blk.mixer, blk.feed_forward, blk.mixer_norm, blk.feed_forward_norm)]
        if self.dtype != torch.bfloat16 or not all(hasattr(p, "emit") for p in parts + [self.final_norm]):
            return None
        b = ProgramBuilder(self.device, self.dtype)
        try:
            resid = b.buffer("residual", s.hidden_size * 4)
            pending = {"ids": b.param("token_ids", lambda st: st.token_ids.data_ptr()), "table": self.embedding}
            for pos, entry in enumerate(s.run_order):
                pending = self.blocks[entry.layer].emit(b, resid, pending, caches[pos])
            n_want = b.param("n_want", lambda st: st.n_want)
            hidden = self.final_norm.emit(b, resid, n_rows=n_want, out_tag="wanted_rows",
                                          rows=b.param("want_rows", lambda st: st.want_rows.data_ptr()), cond=n_want,
                                          **pending)
            b.emit(OP_GEMM_BF16, [hidden, self.output_weight, b.param("logits", lambda st: st.logits_out.data_ptr()),
                                  n_want, s.vocab_size, s.hidden_size, 1], cond=n_want)
        except NotImplementedError:
            return None
        return b.finish(capacity)

    def forward(self, step: StepInputs, caches: list[LayerCache]) -> torch.Tensor:
        """Run the step's tokens; returns logits [n_want, vocab] float32."""
        s = self.spec
        resid = torch.empty((step.n_tokens, s.hidden_size), dtype=torch.float32, device=self.device)
        pending = Pending(ids=step.token_ids, table=self.embedding)
        for pos, entry in enumerate(s.run_order):
            pending = self.blocks[entry.layer].forward(resid, pending, step, caches[pos])
        if step.n_want == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=self.device)
        hidden = self.final_norm.forward(resid, rows=step.want_rows, **pending.kwargs())
        return ops.linear(hidden, self.output_weight, out_dtype=torch.float32)
