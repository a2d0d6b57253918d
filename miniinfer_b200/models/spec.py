"""A model as data: its parts and the order in which its layers run.

The frame around the layers is three parts by role - an ``Embedding``, a ``Norm``, a ``Head`` - and the step
function knows no more of them than the role's one method: an embedding made of several tables, or a head that
does more than a product, is a part like any other.

``run_list`` is the order of execution.  An entry names a block (a block may be named more than
once: its weights then run again, with a cache of their own) and, optionally, an earlier entry
whose cache it reads instead of keeping one (its mixer then writes nothing).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..cache.specs import CacheSpec
from ..config.model_config import ModelConfig
from ..parts.base import Block, Embedding, Head, Norm, Part, PositionEncoding


@dataclass(frozen=True)
class LayerRun:
  block: int                       # index into ModelSpec.blocks
  cache_of: Optional[int] = None   # index of an earlier run-list entry whose cache this entry reads


@dataclass
class ModelSpec:
  config: ModelConfig
  embedding: Embedding             # token ids -> float32 residual rows
  blocks: List[Block]
  final_norm: Norm                 # residual rows (+ what the last block left pending) -> the wanted rows, normed
  lm_head: Head                    # those rows -> float32 logits
  position_encodings: List[PositionEncoding] = field(default_factory=list)
  run_list: Optional[List[LayerRun]] = None
  # file tensors that may be present without being loaded, each equal to another file tensor
  aliases: Dict[str, str] = field(default_factory=dict)
  init_std: float = 0.02

  def __post_init__(self):
    if self.run_list is None:
      self.run_list = [LayerRun(i) for i in range(len(self.blocks))]
    for i, run in enumerate(self.run_list):
      if not (0 <= run.block < len(self.blocks)):
        raise ValueError(f"run list entry {i} names block {run.block}, which does not exist")
      if run.cache_of is not None:
        if not (0 <= run.cache_of < i):
          raise ValueError(f"run list entry {i} reads the cache of entry {run.cache_of}, which is not earlier")
        if self.run_list[run.cache_of].cache_of is not None:
          raise ValueError(f"run list entry {i} reads the cache of entry {run.cache_of}, which has none of its own")
        a = self.blocks[run.block].mixer_part()
        b = self.blocks[self.run_list[run.cache_of].block].mixer_part()
        if a is None or b is None or a.cache_spec() != b.cache_spec():
          raise ValueError(f"run list entry {i} and entry {run.cache_of} differ in what they keep in the cache")

  def all_parts(self) -> List[Part]:
    out: List[Part] = [self.embedding]
    out.extend(self.position_encodings)

    def walk(p: Part):
      out.append(p)
      for s in p.sub_parts():
        walk(s)

    for b in self.blocks:
      walk(b)
    out.append(self.final_norm)
    out.append(self.lm_head)
    return out

  def cache_layer_specs(self) -> List[Optional[CacheSpec]]:
    """The cache need of every run-list entry (None: it keeps nothing of its own)."""
    specs: List[Optional[CacheSpec]] = []
    for run in self.run_list:
      mixer = self.blocks[run.block].mixer_part()
      specs.append(None if (run.cache_of is not None or mixer is None) else mixer.cache_spec())
    return specs
