"""Token embedding and LM head.

Embedding: a row lookup (miniinfer/layers/embedding.py:23-27), written as float32 because it starts
the residual stream.  LM head: ``x @ W^T`` (embedding.py:29-32) with float32 logits; it uses the
embedding's table when the configuration ties them.  The reference decides tying by whether the
file has ``lm_head.weight`` (embedding.py:41-48); here ``tie_word_embeddings`` decides and the file
is checked against it.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import Embedding, Head, ParamSpec, whole


class TokenEmbedding(Embedding):
  def __init__(self, name: str, vocab_size: int, hidden_size: int):
    super().__init__(name)
    self.vocab_size = vocab_size
    self.hidden_size = hidden_size

  def param_specs(self) -> Dict[str, ParamSpec]:
    shape = (self.vocab_size, self.hidden_size)
    return {"weight": ParamSpec(shape, "table", [whole(f"{self.name}.weight", shape)])}

  def forward(self, ids: torch.Tensor, ctx) -> torch.Tensor:
    out = ctx.ws.buffer("resid", (ids.shape[0], self.hidden_size), torch.float32)
    ops.embedding(out, self.weight, ids)
    return out


class LMHead(Head):
  def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: Optional[TokenEmbedding] = None):
    super().__init__(name)
    self.vocab_size = vocab_size
    self.hidden_size = hidden_size
    self.tied_to = tied_to

  def param_specs(self) -> Dict[str, ParamSpec]:
    if self.tied_to is not None:
      return {}
    shape = (self.vocab_size, self.hidden_size)
    return {"weight": ParamSpec(shape, "matrix", [whole(f"{self.name}.weight", shape)])}

  def validate(self, dtype: torch.dtype) -> None:
    if dtype == torch.bfloat16 and self.hidden_size % 8:
      raise ValueError(f"{self.name}: hidden_size={self.hidden_size} must be a multiple of 8 in bfloat16 "
                       f"(rows are read 16 bytes at a time)")

  def table(self) -> torch.Tensor:
    return self.tied_to.weight if self.tied_to is not None else self.weight

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    out = ctx.ws.buffer("logits", (x.shape[0], self.vocab_size), torch.float32)
    ops.linear(out, x, self.table())
    return out
