"""Per-request sampling options; names, defaults and checks as in the reference
(miniinfer/utils/sampling_params.py:5-23), plus a seed."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
  temperature: float = 1.0      # 0: greedy
  max_tokens: int = 1
  ignore_eos: bool = False
  top_k: int = 0                # 0: off
  top_p: float = 1.0            # 1: off
  seed: Optional[int] = None    # None: derived from the engine's seed and the request's number

  def __post_init__(self):
    if self.temperature < 0:
      raise ValueError("temperature must be >= 0")
    if self.max_tokens <= 0:
      raise ValueError("max_tokens must be > 0")
    if self.top_k is None:
      self.top_k = 0
    if self.top_k < 0:
      raise ValueError("top_k must be >= 0")
    if not (0.0 < float(self.top_p) <= 1.0):
      raise ValueError("top_p must be in (0, 1]")
