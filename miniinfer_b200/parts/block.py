"""The arrangement of the parts of a layer.

``PreNormBlock`` is the reference's wiring (miniinfer/models/fused_qwen3.py:175-196): the residual
is carried beside the hidden state; each norm first adds the previous part's output into the
residual and then normalises it.  The block returns its feed-forward output as the pending
addition for whoever comes next (the next block's first norm, or the final norm).
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Block, FeedForward, Mixer, Norm, Part


class PreNormBlock(Block):
  def __init__(self, name: str, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
    super().__init__(name)
    self.mixer_norm = mixer_norm
    self.mixer = mixer
    self.ffn_norm = ffn_norm
    self.ffn = ffn

  def sub_parts(self) -> List[Part]:
    return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

  def mixer_part(self) -> Optional[Mixer]:
    return self.mixer

  def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache) -> Optional[torch.Tensor]:
    # A part may offer to work on the residual stream itself - its norm in its first kernel, the add of its
    # output in its last (for a step of few rows: fewer launches).  Then nothing is pending behind it.
    if pending is None and self.mixer.takes_residual(self.mixer_norm, ctx):
      self.mixer.forward_on_residual(resid, self.mixer_norm, ctx, cache)
      a = None
    else:
      x = self.mixer_norm.add_norm(resid, pending, ctx)
      a = self.mixer.forward(x, ctx, cache)
    if a is None and self.ffn.takes_residual(self.ffn_norm, ctx):
      self.ffn.forward_on_residual(resid, self.ffn_norm, ctx)
      return None
    x = self.ffn_norm.add_norm(resid, a, ctx)
    return self.ffn.forward(x, ctx)
