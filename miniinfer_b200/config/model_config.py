"""Typed model configurations, read from the architecture's own ``config.json`` keys.

The reference keeps every JSON key as an untyped attribute (miniinfer/config/model/base.py:29-31)
and gives defaults in the constructor (miniinfer/config/model/qwen3.py:16-35).  Here every key the
architecture defines is a typed field; keys that change the computation but are not implemented
raise an error that names the key instead of being ignored.
"""

from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
  """A configuration that cannot be run, with the key that is at fault."""


@dataclass
class ModelConfig:
  """What every architecture's configuration gives to the engine."""

  architectures: List[str] = field(default_factory=list)
  model_type: str = ""
  vocab_size: int = 0
  max_position_embeddings: int = 0
  bos_token_id: Optional[int] = None
  eos_token_id: Any = None          # int, list of ints or None
  torch_dtype: Optional[str] = None
  extra: Dict[str, Any] = field(default_factory=dict)

  @classmethod
  def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
    names = {f.name for f in dataclasses.fields(cls)}
    known = {k: v for k, v in d.items() if k in names and k != "extra"}
    cfg = cls(**known)
    cfg.extra = {k: v for k, v in d.items() if k not in names}
    # "dtype" is the newer spelling of "torch_dtype" in config.json files.
    if cfg.torch_dtype is None and "dtype" in cfg.extra:
      cfg.torch_dtype = cfg.extra.pop("dtype")
    cfg.validate()
    return cfg

  @classmethod
  def from_json(cls, path: str) -> "ModelConfig":
    if os.path.isdir(path):
      path = os.path.join(path, "config.json")
    with open(path, encoding="utf-8") as f:
      return cls.from_dict(json.load(f))

  def to_dict(self) -> Dict[str, Any]:
    d = dataclasses.asdict(self)
    extra = d.pop("extra")
    d.update(extra)
    return {k: v for k, v in d.items() if v is not None}

  def eos_ids(self) -> List[int]:
    if self.eos_token_id is None:
      return []
    if isinstance(self.eos_token_id, (list, tuple)):
      return [int(x) for x in self.eos_token_id]
    return [int(self.eos_token_id)]

  def validate(self) -> None:  # pragma: no cover - overridden
    pass


@dataclass
class Qwen3Config(ModelConfig):
  """Qwen3 dense decoder (defaults: miniinfer/config/model/qwen3.py:16-35)."""

  model_type: str = "qwen3"
  vocab_size: int = 151936
  hidden_size: int = 1024
  intermediate_size: int = 3072
  num_hidden_layers: int = 28
  num_attention_heads: int = 16
  num_key_value_heads: Optional[int] = 8
  head_dim: Optional[int] = 128
  hidden_act: str = "silu"
  max_position_embeddings: int = 40960
  initializer_range: float = 0.02
  rms_norm_eps: float = 1e-6
  rope_theta: float = 1000000.0
  rope_scaling: Optional[Dict[str, Any]] = None
  attention_bias: bool = False
  attention_dropout: float = 0.0
  tie_word_embeddings: bool = True
  use_cache: bool = True
  use_sliding_window: bool = False
  sliding_window: Optional[int] = None
  max_window_layers: Optional[int] = None
  layer_types: Optional[List[str]] = None

  def validate(self) -> None:
    if self.num_key_value_heads is None:            # qwen3.py:46-48
      self.num_key_value_heads = self.num_attention_heads
    if self.head_dim is None:                        # qwen3.py:75-79
      if self.hidden_size % self.num_attention_heads:
        raise ConfigError("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
      self.head_dim = self.hidden_size // self.num_attention_heads
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
      v = getattr(self, key)
      if not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {v!r}")
    if self.num_attention_heads % self.num_key_value_heads:
      raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads "
                        f"({self.num_attention_heads} vs {self.num_key_value_heads})")
    if self.head_dim % 2:
      raise ConfigError(f"head_dim must be even for the rotary encoding, got {self.head_dim}")
    if self.hidden_act != "silu":                    # fused_qwen3.py:122-123
      raise ConfigError(f"hidden_act={self.hidden_act!r} is not supported (only 'silu')")
    if self.rope_scaling not in (None, {}):
      kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
      if kind not in (None, "default"):
        raise ConfigError(f"rope_scaling={self.rope_scaling!r} is not supported")
    if self.attention_bias:
      raise ConfigError("attention_bias=true is not supported (the architecture has no QKV bias)")
    if not (self.rms_norm_eps > 0):
      raise ConfigError("rms_norm_eps must be positive")
    if self.use_sliding_window:
      if not self.sliding_window or self.sliding_window <= 0:
        raise ConfigError("use_sliding_window=true needs a positive sliding_window")
    if self.layer_types is not None:
      if len(self.layer_types) != self.num_hidden_layers:
        raise ConfigError("layer_types must have num_hidden_layers entries")
      for t in self.layer_types:
        if t not in ("full_attention", "sliding_attention"):
          raise ConfigError(f"layer_types entry {t!r} is not known")

  def window_of_layer(self, layer: int) -> Optional[int]:
    """The attention window of a layer, or None for all keys.  The reference carries these keys
    without reading them; their meaning here: ``layer_types`` decides if given, else the layers
    from ``max_window_layers`` on are windowed when ``use_sliding_window`` is set."""
    if not self.use_sliding_window or not self.sliding_window:
      return None
    if self.layer_types is not None:
      return int(self.sliding_window) if self.layer_types[layer] == "sliding_attention" else None
    first = self.max_window_layers if self.max_window_layers is not None else 0
    return int(self.sliding_window) if layer >= first else None
