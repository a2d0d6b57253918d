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
    x = self.mixer_norm.add_norm(resid, pending, ctx)
    a = self.mixer.forward(x, ctx, cache)
    x = self.ffn_norm.add_norm(resid, a, ctx)
    return self.ffn.forward(x, ctx)
