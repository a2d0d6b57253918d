"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up in one matrix
(miniinfer/models/fused_qwen3.py:111-138; order gate, up: miniinfer/loader/weight.py:87-93).
"""

from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, Piece, whole


class SwiGLUFeedForward(FeedForward):
  def __init__(self, name: str, hidden_size: int, intermediate_size: int):
    super().__init__(name)
    self.hidden_size = hidden_size
    self.intermediate_size = intermediate_size

  def param_specs(self) -> Dict[str, ParamSpec]:
    H, I = self.hidden_size, self.intermediate_size
    return {
      "gate_up": ParamSpec((2 * I, H), "matrix", [
        [Piece(f"{self.name}.gate_proj.weight", 0, (I, H)), Piece(f"{self.name}.up_proj.weight", I, (I, H))],
        whole(f"{self.name}.gate_up_proj.weight", (2 * I, H)),
      ]),
      "down": ParamSpec((H, I), "matrix", [whole(f"{self.name}.down_proj.weight", (H, I))]),
    }

  def validate(self, dtype: torch.dtype) -> None:
    if dtype == torch.bfloat16:
      for what, k in (("hidden_size", self.hidden_size), ("intermediate_size", self.intermediate_size)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")

  def takes_residual(self, norm, ctx) -> bool:
    return norm.as_rms() is not None and ops.fuses_few_rows(ctx.num_tokens, ctx.dtype)

  def forward_on_residual(self, resid: torch.Tensor, norm, ctx) -> None:
    """Two kernels: norm + gate-and-up product + SwiGLU, then the down product + residual add."""
    weight, eps = norm.as_rms()
    act = ctx.ws.buffer("ffn_act", (resid.shape[0], self.intermediate_size), ctx.dtype)
    ops.linear_swiglu_normed(act, resid, weight, eps, self.gate_up)
    ops.linear_add(resid, act, self.down)

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    T = x.shape[0]
    act = ctx.ws.buffer("ffn_act", (T, self.intermediate_size), ctx.dtype)
    ops.linear_swiglu(act, x, self.gate_up, ctx.ws)
    out = ctx.ws.buffer("ffn_out", (T, self.hidden_size), ctx.dtype)
    ops.linear(out, act, self.down)
    return out
