"""Rotate-half rotary position encoding: the 32-bit angle tables.

``inv_freq_i = 1 / theta^(2i / D)`` computed as ``1.0 / (theta ** (arange(0, D, 2).float() / D))``,
``angle = position.float() * inv_freq`` and 32-bit cos / sin, exactly as the reference builds its
tables (src/infer/model/layers.py:47-52). The reference's table repeats each half ([P, D]); only the
distinct half [P, D/2] is kept here. The rotation itself runs inside the mixer's fused kernel.
"""

from __future__ import annotations

import torch

from ..registry import register_position_encoding

_TABLES: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


class RotaryEmbedding:
    def __init__(self, *, head_dim: int, theta: float, max_positions: int):
        if head_dim % 2:
            raise ValueError(f"rotary position encoding needs an even head_dim, got {head_dim}")
        self.head_dim = head_dim
        self.theta = float(theta)
        self.max_positions = int(max_positions)

    def limit_positions(self, n: int) -> None:
        """No position >= n will be asked for: the tables are built that short
        (src/infer/model/qwen2.py:34: min(max_positions, max_position_embeddings))."""
        self.max_positions = max(1, min(self.max_positions, int(n)))

    def tables(self, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
        """(cos, sin), each [max_positions, head_dim / 2] float32 on ``device``; shared between layers."""
        key = (self.head_dim, self.theta, self.max_positions, str(device))
        if key not in _TABLES:
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.int64).float()
                                             / self.head_dim))
            freqs = torch.outer(torch.arange(self.max_positions).float(), inv_freq)
            _TABLES[key] = (freqs.cos().to(device).contiguous(), freqs.sin().to(device).contiguous())
        return _TABLES[key]


register_position_encoding("rope", RotaryEmbedding)
