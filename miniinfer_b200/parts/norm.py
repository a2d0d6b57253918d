"""RMSNorm with the residual add in front of it (one kernel).

Formula of the reference: ``w * x * rsqrt(mean(x^2) + eps)`` in float32
(miniinfer/layers/layernorm.py:27-32), fused with the residual add as in its Triton kernel
(kernels/triton/rms_norm.py:66-108).  The residual stream here is float32.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import Norm, ParamSpec, whole


class RMSNorm(Norm):
  def __init__(self, name: str, dim: int, eps: float):
    super().__init__(name)
    self.dim = dim
    self.eps = float(eps)

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {"weight": ParamSpec((self.dim,), "vector", [whole(f"{self.name}.weight", (self.dim,))], init="ones_noise")}

  def as_rms(self):
    return self.weight, self.eps

  def add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx) -> torch.Tensor:
    out = ctx.ws.buffer("normed", (resid.shape[0], self.dim), ctx.dtype)
    ops.add_rmsnorm(out, resid, delta, self.weight, self.eps, None, True)
    return out

  def norm_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, ctx) -> torch.Tensor:
    out = ctx.ws.buffer("normed_rows", (rows.shape[0], self.dim), ctx.dtype)
    ops.add_rmsnorm(out, resid, delta, self.weight, self.eps, rows, False)
    return out
