"""Position encodings.  The rotary table is built as the reference builds it
(ullm/layers/rotary_embedding.py:58-75): inv_freq_i = 1 / theta^(2i/dim) and
angle[p, i] = p * inv_freq_i in float32 on the host, cos and sin of it in
float32.  The mixer's kernel reads row `position` of the tables and rotates in
32-bit registers.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope")
class RotaryPositions(PositionEncoding):
    def __init__(self, rotary_dim: int, theta: float, max_positions: int):
        super().__init__()
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim={rotary_dim} must be a positive even number")
        if max_positions <= 0:
            raise ValueError("max_positions must be positive")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_positions = max_positions
        self._tables: dict[str, torch.Tensor] = {}

    def build_tables(self, device) -> None:
        inv_freq = 1.0 / (
            self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim)
        )
        t = torch.arange(self.max_positions, dtype=torch.float32)
        freqs = torch.einsum("i,j->ij", t, inv_freq)
        self._tables = {
            "cos": freqs.cos().contiguous().to(device),
            "sin": freqs.sin().contiguous().to(device),
        }

    def tables(self):
        return self._tables


@register_position_encoding("none")
class NoPositions(PositionEncoding):
    def __init__(self, rotary_dim: int = 0, theta: float = 0.0, max_positions: int = 0):
        super().__init__()
        self.rotary_dim = 0
        self.max_positions = max_positions

    def build_tables(self, device) -> None:
        pass
