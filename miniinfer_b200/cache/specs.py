"""What a layer asks of the cache manager.

The reference has one uniform store for all layers (``MHAKVCacheStorage``,
miniinfer/kvcache/memory_pool.py:18-64).  Here every layer states its need as data; layers with the
same need form a group that has pages (or state slots) of its own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union


@dataclass(frozen=True)
class PagedKVSpec:
  """Keys and values of every position (``window is None``) or of the last ``window`` positions."""

  num_kv_heads: int
  head_dim: int
  window: Optional[int] = None

  def __post_init__(self):
    if self.num_kv_heads <= 0 or self.head_dim <= 0:
      raise ValueError("num_kv_heads and head_dim must be positive")
    if self.window is not None and self.window <= 0:
      raise ValueError("window must be positive or None")


@dataclass(frozen=True)
class FixedStateSpec:
  """A tensor of fixed shape for each live request, zero when the request is admitted."""

  shape: Tuple[int, ...]
  dtype: str = "float32"

  def __post_init__(self):
    if any(int(s) <= 0 for s in self.shape):
      raise ValueError("state shape must be positive")


CacheSpec = Union[PagedKVSpec, FixedStateSpec]
