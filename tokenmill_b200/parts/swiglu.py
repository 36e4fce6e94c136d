"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no biases.

The gate and up matrices are stored fused, rows [gate; up], from the checkpoint's gate_proj and
up_proj tensors (src/infer/model/layers.py:153-164, src/infer/model/loader.py:46,114-116).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import register_feed_forward
from .base import StepInputs
from .spec import WeightSpec


class SwiGLUFeedForward:
    def __init__(self, *, hidden_size: int, intermediate_size: int, dtype: torch.dtype, device: torch.device):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec("gate_proj.weight", (I, H)), WeightSpec("up_proj.weight", (I, H)),
                WeightSpec("down_proj.weight", (H, I))]

    def activation_bytes(self, n_tokens: int) -> int:
        """The [T, 2 I] product, the [T, I] activation and the branch output of one step."""
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * (3 * self.intermediate_size + self.hidden_size) * elt

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    adds_to_residual = True      # forward(..., residual=stream) may add its output into the stream and return None

    def forward(self, x: torch.Tensor, step: StepInputs | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor | None:
        T = x.shape[0]
        act = torch.empty((T, self.intermediate_size), dtype=self.dtype, device=x.device)
        if ops.skinny_ok(x, self.w_gate_up) and ops.skinny_ok(act, self.w_down, allow_split=True):
            # decode step: two weight-streaming kernels; the activation is the first one's epilogue, and
            # the second may hand its K-range partials to the norm that follows
            ops.skinny_gate_up_swiglu(x, self.w_gate_up, act)
            return ops.skinny_linear(act, self.w_down, k_splits=ops.skinny_k_splits(T, self.intermediate_size))
        if self.intermediate_size % 8 == 0 and ops.tc_ok(x, self.w_gate_up):
            # prompt step on tcgen05 (when switched on): the activation is the product's epilogue
            ops.tc_gate_up_swiglu(x, self.w_gate_up, act)
            return ops.tc_linear(act, self.w_down) if ops.tc_ok(act, self.w_down) else ops.linear(act, self.w_down)
        if ops.tc_swiglu_decode_ok(x, self.w_gate_up):
            # a few dozen tokens: one tcgen05 tile of 32 gate and 32 up rows for every multiprocessor
            ops.tc_gate_up_swiglu(x, self.w_gate_up, act)
        else:
            gu = ops.linear(x, self.w_gate_up)
            ops.swiglu(gu, act)
        if ops.tc_add_ok(act, self.w_down, residual):
            # a few dozen tokens: the down projection cut along K over the whole chip, added into the stream
            ops.tc_linear_add(act, self.w_down, residual)
            return None
        return ops.linear(act, self.w_down)


    def emit(self, b, x):
        """The prompt-step launches (library product, activation, library product) written into a step program
        (kernels/program.py); ``x`` is a workspace buffer. Returns the output buffer."""
        from ..kernels.program import OP_GEMM_BF16, OP_SWIGLU
        if self.dtype != torch.bfloat16:
            raise NotImplementedError("step programs are built for the bfloat16 path")
        H, I, T = self.hidden_size, self.intermediate_size, b.tokens()
        gu = b.buffer("gate_up", 2 * I * 2)
        act = b.buffer("act", I * 2)
        out = b.buffer("feed_forward_out", H * 2)
        b.emit(OP_GEMM_BF16, [x, self.w_gate_up, gu, T, 2 * I, H, 0])
        b.emit(OP_SWIGLU, [ops.dtype_code(self.dtype), gu, act, T, I])
        b.emit(OP_GEMM_BF16, [act, self.w_down, out, T, H, I, 0])
        return out


register_feed_forward("swiglu", SwiGLUFeedForward)
