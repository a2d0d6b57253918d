"""One registry from an architecture's name to its configuration class and model builder.

The reference picks the model with an if/elif chain on ``model_type`` and ``architectures``
(miniinfer/engine/model_runner.py:61-76) and ends with ``model = None`` for anything else.  Here the
name in ``config.json``'s ``architectures[0]`` is looked up in a table, and an unknown name is an
error that lists the known ones.
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, Tuple, Type

from .model_config import ConfigError, ModelConfig

# name -> (config class, builder(config) -> ModelSpec)
_MODELS: Dict[str, Tuple[Type[ModelConfig], Callable]] = {}


def register_model(name: str, config_cls: Type[ModelConfig]):
  """Decorator for a function ``build(config) -> ModelSpec``."""

  def deco(builder: Callable):
    if name in _MODELS:
      raise ValueError(f"architecture {name!r} is already registered")
    _MODELS[name] = (config_cls, builder)
    return builder

  return deco


def unregister_model(name: str) -> None:
  _MODELS.pop(name, None)


def known_architectures():
  _ensure_builtin()
  return sorted(_MODELS)


def _ensure_builtin() -> None:
  # importing the package of models fills the table
  from .. import models  # noqa: F401


def lookup(name: str) -> Tuple[Type[ModelConfig], Callable]:
  _ensure_builtin()
  try:
    return _MODELS[name]
  except KeyError:
    raise ConfigError(f"architecture {name!r} is not registered; known: {', '.join(sorted(_MODELS))}") from None


def architecture_of(config_dict: dict) -> str:
  archs = config_dict.get("architectures")
  if not archs:
    raise ConfigError("config.json has no 'architectures' entry")
  return archs[0]


def load_model_config(model_dir: str) -> ModelConfig:
  """Reads ``config.json`` with the configuration class its architecture registered."""
  path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
  if not os.path.exists(path):
    raise FileNotFoundError(f"no config.json at {path}")
  with open(path, encoding="utf-8") as f:
    d = json.load(f)
  config_cls, _ = lookup(architecture_of(d))
  return config_cls.from_dict(d)


def build_model_spec(config: ModelConfig):
  _, builder = lookup(architecture_of({"architectures": config.architectures}))
  return builder(config)
