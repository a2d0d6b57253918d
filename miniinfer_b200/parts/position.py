"""Rotary position encoding as a part: it owns theta, the rotated width and the angle table.

The table is made exactly as the reference makes it, in float32 on the host
(miniinfer/layers/position_encoding.py:29-45): ``inv = 1 / theta^(2j/dim)``, ``angle = pos * inv``,
a row holds ``cos`` of all angles and then ``sin``.  The rotation itself happens inside the mixer's
fused QKV kernel, in float32 (the reference rotates in the model's dtype, position_encoding.py:105-106).
"""

from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
  def __init__(self, name: str, rotary_dim: int, theta: float, max_position_embeddings: int):
    super().__init__(name)
    if rotary_dim <= 0 or rotary_dim % 2:
      raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
    self.rotary_dim = rotary_dim
    self.theta = float(theta)
    self.max_position_embeddings = max_position_embeddings
    self._table: Optional[torch.Tensor] = None

  def build_table(self, positions: int) -> torch.Tensor:
    inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float) / self.rotary_dim))
    t = torch.arange(positions, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous()

  def prepare(self, device, max_positions: int) -> None:
    n = min(max_positions, self.max_position_embeddings)
    self._table = self.build_table(n).to(device)

  def rotary_table(self) -> Optional[torch.Tensor]:
    if self._table is None:
      raise RuntimeError("RotaryEncoding.prepare was not called")
    return self._table

  def max_positions(self) -> Optional[int]:
    return self.max_position_embeddings
