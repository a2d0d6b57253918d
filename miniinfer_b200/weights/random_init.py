"""Random weights: a model folder (``config.json`` + ``model.safetensors``) from a configuration
and a seed, and the same initialisation made directly on the device for sizes where a file would
only cost time.

Matrices and the embedding table are drawn from N(0, initializer_range) and norm weights from
1 + N(0, 0.1), in float32 from one seeded CPU generator, tensor after tensor in the order the
model's parts declare them, and then cast to the stored dtype.  The reference has no such mode (its
tests build random models with another library, tests/unittests/test_weight_loader.py:23-36).
"""

from __future__ import annotations

import json
import os
from typing import Dict, Union

import torch

from ..config.model_config import ModelConfig
from ..config.registry import architecture_of, build_model_spec, lookup
from ..models.spec import ModelSpec
from .loader import role_dtype

NORM_NOISE = 0.1


def _draw(shape, init: str, std: float, gen: torch.Generator, device="cpu") -> torch.Tensor:
  t = torch.randn(tuple(shape), generator=gen, dtype=torch.float32, device=device)
  if init == "ones_noise":
    return 1.0 + NORM_NOISE * t
  return std * t


def random_state_dict(spec: ModelSpec, seed: int, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
  """File tensors (under the names of each parameter's first alternative, the split ones)."""
  gen = torch.Generator(device="cpu")
  gen.manual_seed(int(seed))
  out: Dict[str, torch.Tensor] = {}
  for part in spec.all_parts():
    for ps in part.param_specs().values():
      for piece in ps.sources[0]:
        t = _draw(piece.shape, ps.init, spec.init_std, gen)
        out[piece.file_name] = t.to(dtype if ps.role in ("matrix", "table") else torch.float32).contiguous() \
          if ps.role != "int" else t.to(torch.int32)
  return out


def write_random_model(config: Union[ModelConfig, dict], out_dir: str, seed: int = 0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
  """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``."""
  from safetensors.torch import save_file

  if isinstance(config, dict):
    config_cls, _ = lookup(architecture_of(config))
    config = config_cls.from_dict(config)
  spec = build_model_spec(config)
  os.makedirs(out_dir, exist_ok=True)
  d = config.to_dict()
  d["torch_dtype"] = str(dtype).replace("torch.", "")
  with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
    json.dump(d, f, indent=2)
  save_file(random_state_dict(spec, seed, dtype), os.path.join(out_dir, "model.safetensors"))
  return out_dir


def init_random_on_device(spec: ModelSpec, compute_dtype: torch.dtype, device, seed: int = 0) -> None:
  """Fills and binds every parameter with the same distributions, drawn on the device (the values
  differ from those of ``write_random_model``: another generator).  For benchmarks of large shapes."""
  gen = torch.Generator(device=device)
  gen.manual_seed(int(seed))
  for part in spec.all_parts():
    params = {}
    for local, ps in part.param_specs().items():
      dt = role_dtype(ps.role, compute_dtype)
      if ps.role == "int":
        params[local] = torch.zeros(ps.shape, dtype=dt, device=device)
        continue
      p = torch.empty(ps.shape, dtype=dt, device=device)
      rows = max(1, (1 << 26) // max(1, int(torch.tensor(ps.shape[1:]).prod()) if len(ps.shape) > 1 else 1))
      if len(ps.shape) == 1:
        p.copy_(_draw(ps.shape, ps.init, spec.init_std, gen, device))
      else:
        for r0 in range(0, ps.shape[0], rows):
          r1 = min(ps.shape[0], r0 + rows)
          p[r0:r1].copy_(_draw((r1 - r0,) + tuple(ps.shape[1:]), ps.init, spec.init_std, gen, device))
      params[local] = p
    part.bind(params)
