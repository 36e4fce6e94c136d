"""RMSNorm over the 32-bit residual stream, fused with whatever feeds the stream.

Formula (src/infer/model/layers.py:35-44): ``x32 * rsqrt(mean(x32^2) + eps)`` in 32-bit, cast to the
activation dtype, then multiplied by the weight. The weight is held in float32 (a 16-bit checkpoint
value converts exactly; the product is rounded once to the activation dtype, which equals the
reference's 16-bit multiply).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import register_norm
from .spec import WeightSpec


class RMSNorm:
    def __init__(self, *, hidden_size: int, eps: float, dtype: torch.dtype, device: torch.device):
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.dtype = dtype
        self.device = device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("weight", (self.hidden_size,), dtype="float32", init=("ones_plus_normal", 0.02))]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, resid: torch.Tensor, out: torch.Tensor | None = None, *,
                branch: torch.Tensor | None = None, partials: torch.Tensor | None = None,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        n = rows.numel() if rows is not None else resid.shape[0]
        if out is None:
            out = torch.empty((n, self.hidden_size), dtype=self.dtype, device=resid.device)
        return ops.add_rmsnorm(resid, self.weight, self.eps, out, branch=branch, partials=partials, ids=ids,
                               table=table, rows=rows)


    def emit(self, b, resid, *, n_rows, out_tag: str = "normed", branch=None, ids=None, table=None, rows=None,
             cond=None):
        """The same launch, written into a step program (kernels/program.py): ``resid`` and ``branch`` are
        workspace buffers, ``ids`` / ``rows`` / ``n_rows`` step parameters. Returns the output buffer."""
        from ..kernels.program import OP_ADD_RMSNORM, Float
        out = b.buffer(out_tag, self.hidden_size * (torch.finfo(self.dtype).bits // 8))
        b.emit(OP_ADD_RMSNORM, [ops.dtype_code(self.dtype), resid, branch, ids, table, rows, self.weight, Float(self.eps), out,
                                n_rows, self.hidden_size], cond=cond)
        return out


register_norm("rmsnorm", RMSNorm)
