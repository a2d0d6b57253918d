"""Reads a model's parameters from ``*.safetensors`` by tensor name.

Against the reference (miniinfer/loader/weight.py:65-209): tensors go straight into the fused
parameters they belong to (q/k/v rows of the QKV matrix, gate/up halves), without a merged
dictionary on the host; names may lack the ``model.`` prefix (miniinfer/models/fused_qwen3.py:225-226);
and every problem with the file - tensors that are missing, tensors nobody asked for, wrong
shapes - is collected and raised as ONE error, where the reference raises a bare ``KeyError`` for a
missing tensor and ignores extra ones.

Kept dtypes: matrices and tables in the engine's compute dtype; vectors (norm weights) in float32,
so a vector stored in 32-bit stays so; integer tensors as int32.  A matrix stored in float32 is
rounded to bfloat16 when the engine computes in bfloat16, because the tensor-core products take
bfloat16 operands.
"""

from __future__ import annotations

import glob
import os
from typing import Dict, List, Tuple

import torch

from ..models.spec import ModelSpec
from ..parts.base import ParamSpec, Piece


class WeightLoadError(RuntimeError):
  def __init__(self, model_dir: str, missing: List[str], unexpected: List[str], wrong_shape: List[str],
               other: List[str] = ()):  # type: ignore[assignment]
    self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
    lines = [f"cannot load the weights in {model_dir}:"]
    if self.missing:
      lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
    if self.unexpected:
      lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
    if self.wrong_shape:
      lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
    for o in self.other:
      lines.append("  " + o)
    super().__init__("\n".join(lines))


def role_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
  if role in ("matrix", "table"):
    return compute_dtype
  if role == "vector":
    return torch.float32
  return torch.int32


def _index_files(model_dir: str) -> Dict[str, Tuple[str, Tuple[int, ...]]]:
  from safetensors import safe_open

  files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
  if not files:
    raise FileNotFoundError(f"no *.safetensors file in {model_dir}")
  index: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
  for path in files:
    with safe_open(path, framework="pt", device="cpu") as f:
      for key in f.keys():
        index[key] = (path, tuple(f.get_slice(key).get_shape()))
  return index


def load_weights(spec: ModelSpec, model_dir: str, compute_dtype: torch.dtype, device) -> None:
  """Fills and binds the parameters of every part of ``spec``."""
  from safetensors import safe_open

  index = _index_files(model_dir)
  # the file may name its tensors without the "model." prefix
  strip = ("model.embed_tokens.weight" not in index) and ("embed_tokens.weight" in index)

  def fname(n: str) -> str:
    return n[len("model."):] if strip and n.startswith("model.") else n

  missing: List[str] = []
  wrong: List[str] = []
  used: set = set()
  plan: List[Tuple[object, str, ParamSpec, List[Piece]]] = []
  for part in spec.all_parts():
    for local, ps in part.param_specs().items():
      chosen = None
      for alt in ps.sources:
        if all(fname(p.file_name) in index for p in alt):
          chosen = alt
          break
      if chosen is None:
        # report against the alternative of which most is there
        chosen = max(ps.sources, key=lambda alt: sum(fname(p.file_name) in index for p in alt))
      for p in chosen:
        n = fname(p.file_name)
        if n not in index:
          missing.append(n)
          continue
        used.add(n)
        if index[n][1] != tuple(p.shape):
          wrong.append(f"{n}: file has {list(index[n][1])}, the model needs {list(p.shape)}")
      plan.append((part, local, ps, chosen))

  other: List[str] = []
  alias_checks: List[Tuple[str, str]] = []
  for alias, target in spec.aliases.items():
    a, t = fname(alias), fname(target)
    if a in index:
      used.add(a)
      if t in index:
        if index[a][1] != index[t][1]:
          wrong.append(f"{a}: file has {list(index[a][1])}, but it must equal {t} {list(index[t][1])}")
        else:
          alias_checks.append((a, t))
  unexpected = sorted(n for n in index if n not in used)
  if missing or unexpected or wrong:
    raise WeightLoadError(model_dir, sorted(set(missing)), unexpected, wrong)

  handles: Dict[str, object] = {}

  def tensor(name: str) -> torch.Tensor:
    path = index[name][0]
    if path not in handles:
      handles[path] = safe_open(path, framework="pt", device="cpu")
    return handles[path].get_tensor(name)

  for a, t in alias_checks:
    if not torch.equal(tensor(a), tensor(t)):
      other.append(f"{a} is present and differs from {t}, but the configuration ties them")
  if other:
    raise WeightLoadError(model_dir, [], [], [], other)

  by_part: Dict[int, Dict[str, torch.Tensor]] = {}
  parts_by_id: Dict[int, object] = {}
  for part, local, ps, pieces in plan:
    dt = role_dtype(ps.role, compute_dtype)
    param = torch.empty(ps.shape, dtype=dt, device=device)
    for p in pieces:
      src = tensor(fname(p.file_name))
      if ps.role == "int" and src.is_floating_point():
        other.append(f"{p.file_name}: an integer table is stored as {src.dtype}")
        continue
      if ps.role != "int" and not src.is_floating_point():
        other.append(f"{p.file_name}: stored as {src.dtype}, a floating-point tensor is needed")
        continue
      dst = param if len(pieces) == 1 and p.row_start == 0 and tuple(p.shape) == tuple(ps.shape) \
        else param[p.row_start:p.row_start + p.shape[0]]
      dst.copy_(src)
    by_part.setdefault(id(part), {})[local] = param
    parts_by_id[id(part)] = part
  if other:
    raise WeightLoadError(model_dir, [], [], [], other)
  for part in spec.all_parts():
    part.bind(by_part.get(id(part), {}))
