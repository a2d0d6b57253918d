"""What every part of a layer is: a named holder of parameters with a forward method.

A part knows its own sizes and constants (they are constructor arguments) and the names under
which its tensors may appear in a weights file.  It does not know which model it is in, which
layer it is, or what the other parts of its block are.

Interfaces (see the concrete parts for examples):

``Norm``           ``add_norm(resid, delta, ctx) -> x``: adds ``delta`` (or nothing) into the float32
                   residual rows in place and returns the normalised rows in the compute dtype;
                   ``norm_rows(resid, delta, rows, ctx) -> x``: the same for selected rows, without
                   changing the residual.
``Mixer``          ``cache_spec() -> CacheSpec | None`` and ``forward(x, ctx, cache) -> delta``: mixes
                   information across the tokens of a request, using and updating ``cache``.
``FeedForward``    ``forward(x, ctx) -> delta``: acts on each token alone.
``PositionEncoding`` gives mixers what they need to encode positions (``rotary_table()``), and may
                   act on the hidden state after the embedding (``apply_to_hidden``).
``Block``          ``forward(resid, pending, ctx, cache) -> pending``: the arrangement of the above.

Two more things any part may state: ``validate(dtype)`` refuses, when the engine is built, the sizes
its kernels cannot take; ``step_work()`` declares int32 work lists (``StepWork``) that its kernels
need for every step - the step function makes them on the host, uploads them with the rest of the
step's description and hands them to the part in ``ctx.work``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.specs import CacheSpec


@dataclass(frozen=True)
class Piece:
  """A tensor of the weights file that fills rows ``row_start .. row_start + shape[0]`` of a parameter."""

  file_name: str
  row_start: int
  shape: Tuple[int, ...]


@dataclass
class ParamSpec:
  """A parameter: its shape, its role (``matrix``/``table``: kept in the compute dtype; ``vector``:
  kept in float32; ``int``: kept as int32) and the alternative sets of file tensors that fill it."""

  shape: Tuple[int, ...]
  role: str
  sources: List[List[Piece]]
  init: str = "normal"            # random-weights mode: "normal" (std given by the model) or "ones_noise"

  def __post_init__(self):
    if self.role not in ("matrix", "table", "vector", "int"):
      raise ValueError(f"unknown parameter role {self.role!r}")


def whole(file_name: str, shape: Sequence[int]) -> List[Piece]:
  return [Piece(file_name, 0, tuple(shape))]


class HostStep:
  """The numbers of a step as the host knows them, for the makers of work lists: for every item its
  number of new tokens ``q_len`` and its length before the step ``start`` (int32 arrays)."""

  def __init__(self, q_len: np.ndarray, start: np.ndarray, max_model_len: int):
    self.q_len = q_len
    self.start = start
    self.max_model_len = max_model_len

  @property
  def num_items(self) -> int:
    return len(self.q_len)

  def decode_items(self) -> np.ndarray:
    """Indices of the items that bring exactly one token."""
    return np.flatnonzero(self.q_len == 1).astype(np.int32)

  def longest_decode_context(self) -> int:
    """The largest length, this step's token included, among the items that bring one token (0: none)."""
    one = self.q_len == 1
    return int((self.start[one] + 1).max()) if one.any() else 0

  def context_class(self, length: int, step: int) -> int:
    """``length`` rounded up to a multiple of ``step``, no more than the longest request allowed."""
    return min(self.max_model_len, -(-length // step) * step) if length else 0


class StepWork:
  """An int32 work list that a part's kernels need for each step.

  ``name`` identifies the list: parts that declare a list of the same name share it (it is made once
  per step).  ``build(step)`` returns the array.  ``key(step)`` returns what the part's launches
  depend on beyond the array's contents on the device - its length as a rule, and any bound that
  sizes a grid; steps with equal keys may be replayed from one recorded CUDA graph, and the key is
  handed to the part as ``ctx.work_key[name]``.  ``per_step``: set it if, for steps of single tokens
  only, the array depends on more than the number of items (it is then made anew for every step)."""

  name = ""
  per_step = False

  def build(self, step: HostStep) -> np.ndarray:
    raise NotImplementedError

  def key(self, step: HostStep) -> tuple:
    return (len(self.build(step)),)


class Part:
  """Base of all parts.  ``name`` is the prefix of the part's tensors in a weights file.

  ``reads_step_on_host``: set it to True in a part whose forward method reads the step's description
  on the host (``ctx.host``: lengths, slots, ...) or decides anything else in Python from the
  step's contents.  Decode steps of a model with such a part are not replayed from CUDA graphs,
  since a graph replays the kernels of the step it was recorded from."""

  reads_step_on_host = False

  def __init__(self, name: str):
    self.name = name
    self.params: Dict[str, torch.Tensor] = {}

  def param_specs(self) -> Dict[str, ParamSpec]:
    return {}

  def bind(self, params: Dict[str, torch.Tensor]) -> None:
    """Receives the loaded parameters (device tensors) by local name."""
    self.params = params
    for k, v in params.items():
      setattr(self, k, v)

  def sub_parts(self) -> List["Part"]:
    return []

  def validate(self, dtype: torch.dtype) -> None:
    """Raises ``ValueError`` if the part's kernels cannot take its sizes in this compute dtype.  Called
    once when the engine is built, so that a configuration is refused before any step runs."""

  def step_work(self) -> List["StepWork"]:
    """The work lists this part needs for every step (default: none)."""
    return []


class Norm(Part):
  def as_rms(self) -> Optional[Tuple[torch.Tensor, float]]:
    """(weight, eps) if this norm is a plain RMSNorm, ``weight * x * rsqrt(mean(x^2) + eps)``, which a part
    that follows it may then compute itself (``takes_residual``); None otherwise."""
    return None

  def add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx) -> torch.Tensor:
    raise NotImplementedError

  def norm_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor, ctx) -> torch.Tensor:
    raise NotImplementedError


class PositionEncoding(Part):
  def rotary_table(self) -> Optional[torch.Tensor]:
    """[positions, rotary_dim] float32, cos in the first half of a row and sin in the second; or None."""
    return None

  def max_positions(self) -> Optional[int]:
    return None

  def apply_to_hidden(self, resid: torch.Tensor, ctx) -> None:
    """Acts on the float32 hidden state right after the embedding; default: nothing."""

  def prepare(self, device, max_positions: int) -> None:
    """Builds device tables for positions below ``max_positions``."""


class Mixer(Part):
  def cache_spec(self) -> Optional[CacheSpec]:
    return None

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    raise NotImplementedError

  def takes_residual(self, norm: "Norm", ctx) -> bool:
    """Whether, for this step, the mixer would rather work on the residual stream itself: apply ``norm``
    in its first kernel and add its output into the residual in its last (``forward_on_residual``).  An
    option a part may offer where it saves launches; the default is the plain ``forward``."""
    return False

  def forward_on_residual(self, resid: torch.Tensor, norm: "Norm", ctx, cache) -> None:
    """resid += mixer(norm(resid)), in place."""
    raise NotImplementedError


class FeedForward(Part):
  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    raise NotImplementedError

  def takes_residual(self, norm: "Norm", ctx) -> bool:
    return False

  def forward_on_residual(self, resid: torch.Tensor, norm: "Norm", ctx) -> None:
    """resid += feed_forward(norm(resid)), in place."""
    raise NotImplementedError


class Embedding(Part):
  """The start of a model's frame: token ids to the float32 residual stream ``[tokens, hidden]`` (a buffer of
  ``ctx.ws``).  Any number of tables or none: the step function only calls ``forward``."""

  def forward(self, ids: torch.Tensor, ctx) -> torch.Tensor:
    raise NotImplementedError


class Head(Part):
  """The end of a model's frame: the rows the final norm wrote (``[wanted rows, hidden]``) to float32 logits
  ``[wanted rows, vocabulary]``."""

  def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
    raise NotImplementedError


class Block(Part):
  def mixer_part(self) -> Optional[Mixer]:
    return None

  def forward(self, resid: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache) -> Optional[torch.Tensor]:
    raise NotImplementedError
