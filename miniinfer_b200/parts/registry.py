"""Tables from a kind's name to the class that builds it, one for each sort of part.

A model builder picks the parts of each layer by name from here, layer by layer, so a model may mix
kinds.  New kinds are added with the ``register_*`` decorators; nothing else in the package has to
change (the cache manager serves whatever ``cache_spec`` a mixer declares).
"""

from __future__ import annotations

from typing import Callable, Dict

MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], sort: str):
  def outer(kind: str):
    def deco(cls):
      if kind in table:
        raise ValueError(f"{sort} kind {kind!r} is already registered")
      table[kind] = cls
      return cls
    return deco
  return outer


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")


def make(table: Dict[str, Callable], kind: str, *args, **kwargs):
  try:
    cls = table[kind]
  except KeyError:
    raise KeyError(f"kind {kind!r} is not registered; known: {', '.join(sorted(table))}") from None
  return cls(*args, **kwargs)
