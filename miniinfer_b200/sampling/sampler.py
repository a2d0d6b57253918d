"""Turns rows of logits into tokens with the fused sampling kernel.

Rule for one row (see ``csrc/sampling.cu``): ``temperature == 0`` is the arg-max with the lowest
index among equals (miniinfer/layers/sample.py:111-112).  Otherwise ``z = logits / temperature``;
the ``top_k`` largest are kept, then the smallest set of most likely tokens whose probability
reaches ``top_p`` (top-k first, then top-p, as sample.py:115-122); the token is
``argmax(z_i - log(-log u_i))`` over the kept entries, which is a draw from their softmax.
``u_i`` comes from a counter-based generator keyed by (seed, number of the output token, i):

    mix(x): x ^= x >> 30; x *= 0xBF58476D1CE4E5B9; x ^= x >> 27; x *= 0x94D049BB133111EB; x ^= x >> 31
    key  = mix(seed ^ mix(counter + 0x9E3779B97F4A7C15))
    u_i  = ((mix(key ^ (i * 0xD1342543DE82EF95)) >> 41) + 0.5) / 2^23        (64-bit wrap-around; exact in float32, inside (0, 1))

so a request's tokens do not depend on what else is in the batch or on how its prompt was cut
(the reference draws from the global generator, sample.py:115-128).
"""

from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


def derive_seed(engine_seed: int, request_number: int) -> int:
  return (int(engine_seed) * 1000003 + int(request_number) * 7919 + 12345) & ((1 << 62) - 1)


class Sampler:
  """Packs the per-row options into int32 words (for the step's single host-to-device copy) and
  launches the kernel."""

  # a row of options that samples harmlessly (temperature 0: the arg-max, nothing filtered): what the padding
  # rows of a captured decode step get; options not named here are padded with zero words
  PAD_ROWS: Dict[str, np.ndarray] = {"top_p": np.array([1.0], dtype=np.float32).view(np.int32)}

  @staticmethod
  def pack(params: Sequence[SamplingParams], seeds: Sequence[int], counters: Sequence[int]) -> Dict[str, np.ndarray]:
    R = len(params)
    return {
      "temperature": np.array([p.temperature for p in params], dtype=np.float32).view(np.int32),
      "top_k": np.array([p.top_k for p in params], dtype=np.int32),
      "top_p": np.array([p.top_p for p in params], dtype=np.float32).view(np.int32),
      "seed": np.array(list(seeds), dtype=np.int64).view(np.int32).reshape(2 * R),
      "counter": np.array(list(counters), dtype=np.int64).view(np.int32).reshape(2 * R),
    }

  @staticmethod
  def sample(logits: torch.Tensor, extra: Dict[str, torch.Tensor], out: torch.Tensor, workspace=None) -> torch.Tensor:
    """``extra``: the device views of what ``pack`` made; ``out``: int32 [rows]; ``workspace`` lends
    the kernel's scratch (needed when the call is captured in a CUDA graph)."""
    ops.sample(out, logits, extra["temperature"].view(torch.float32), extra["top_k"],
               extra["top_p"].view(torch.float32), extra["seed"].view(torch.int64), extra["counter"].view(torch.int64),
               workspace)
    return out
