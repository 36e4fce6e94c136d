"""Pre-norm block: ``x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x))``
(src/infer/model/qwen2.py:13-23).

The residual stream ``x`` is 32-bit. A branch output is not added where it is produced: it is
handed on as ``Pending`` and the next norm adds it while it reads the row anyway (one pass over the
stream instead of two). The embedding gather enters the same way, as the first pending item.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..registry import register_block
from .base import LayerCache, StepInputs


@dataclass
class Pending:
    """What still has to be added to the residual stream: a branch output, a stack of 32-bit partial
    products, or (at the very start) the embedding rows of the token ids."""

    branch: torch.Tensor | None = None
    partials: torch.Tensor | None = None
    ids: torch.Tensor | None = None
    table: torch.Tensor | None = None

    @classmethod
    def of(cls, y: torch.Tensor) -> "Pending":
        """A part's output: [T, H] in the activation dtype, or [n, T, H] float32 partial products of a
        matrix product whose K range was cut (the norm that follows adds them up in index order), or None
        when the part has added its output into the stream itself."""
        if y is None:
            return cls()
        return cls(partials=y) if y.dim() == 3 else cls(branch=y)

    def kwargs(self) -> dict:
        return {"branch": self.branch, "partials": self.partials, "ids": self.ids, "table": self.table}


class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, resid: torch.Tensor, pending: Pending, step: StepInputs, cache: LayerCache) -> Pending:
        # A part that says ``adds_to_residual`` is offered the stream: it may add its output there itself (its
        # last product's epilogue) and return None; the norm that follows then has nothing left to add.
        normed = self.mixer_norm.forward(resid, **pending.kwargs())
        offer = {"residual": resid} if getattr(self.mixer, "adds_to_residual", False) else {}
        mixed = Pending.of(self.mixer.forward(normed, step, cache, **offer))
        normed = self.feed_forward_norm.forward(resid, **mixed.kwargs())
        offer = {"residual": resid} if getattr(self.feed_forward, "adds_to_residual", False) else {}
        return Pending.of(self.feed_forward.forward(normed, step, **offer))


    def emit(self, b, resid, pending: dict, cache: LayerCache) -> dict:
        """The block's launches written into a step program (kernels/program.py). ``pending`` holds what the
        first norm still has to add to the stream (``branch``: a workspace buffer, or ``ids`` and ``table``);
        returns the same for the norm that follows the block."""
        T = b.tokens()
        normed = self.mixer_norm.emit(b, resid, n_rows=T, **pending)
        mixed = self.mixer.emit(b, normed, cache)
        normed = self.feed_forward_norm.emit(b, resid, n_rows=T, branch=mixed)
        return {"branch": self.feed_forward.emit(b, normed)}


register_block("pre_norm", PreNormBlock)
