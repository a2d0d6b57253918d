"""Engine options as one typed dataclass.

Field names follow the reference's ``EngineConfig`` (miniinfer/config/engine/config.py:8-60) where
it has them: ``model_path``, ``dtype``, ``gpu_memory_utilization``, ``page_size``, ``max_num_seqs``,
``max_context_len``, ``chunked_prefill_size``, ``enable_chunked_prefill``, ``enforce_eager``,
``num_pages`` and ``max_num_batched_tokens`` (named in its docstring, config.py:13-17).
``max_model_len`` is accepted as another name of ``max_context_len`` because the reference's own
scripts pass it (examples/minimal_engine.py:81, benchmark/bench_miniinfer.py:43).  Unlike the
reference (miniinfer/engine/llm_engine.py:102-104) an unknown option is an error, not dropped.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

_DTYPES = {
  "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
  "float32": torch.float32, "fp32": torch.float32, "float": torch.float32, torch.float32: torch.float32,
}


def parse_dtype(dtype: Any) -> torch.dtype:
  try:
    return _DTYPES[dtype]
  except (KeyError, TypeError):
    raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


@dataclass
class EngineConfig:
  model_path: str
  dtype: Any = torch.bfloat16
  device: str = "cuda:0"
  load_format: str = "safetensors"         # "random": config.json only, weights drawn on the device from `seed`
  # cache
  page_size: int = 64
  num_pages: Optional[int] = None          # pages of every cache group; None: from free memory
  gpu_memory_utilization: float = 0.9
  # scheduling
  max_num_seqs: int = 256
  max_context_len: int = 4096
  max_num_batched_tokens: int = 2048       # token budget of one step
  chunked_prefill_size: Optional[int] = None   # largest portion of one prompt in a step; None: the budget
  enable_chunked_prefill: bool = True
  # execution
  enforce_eager: bool = False              # True: no CUDA graphs for decode steps
  enable_overlap: bool = True              # a decode step is launched before the tokens of the step before it are read back
  seed: int = 0

  def __post_init__(self):
    self.dtype = parse_dtype(self.dtype)
    if self.load_format not in ("safetensors", "random"):
      raise ValueError("load_format must be 'safetensors' or 'random'")
    if self.page_size <= 0:
      raise ValueError("page_size must be positive")
    if self.num_pages is not None and self.num_pages < 1:
      raise ValueError("num_pages must be at least 1")
    if not (0.0 < self.gpu_memory_utilization <= 1.0):
      raise ValueError("gpu_memory_utilization must be in (0, 1]")
    if self.max_num_seqs <= 0 or self.max_context_len <= 0 or self.max_num_batched_tokens <= 0:
      raise ValueError("max_num_seqs, max_context_len and max_num_batched_tokens must be positive")
    if self.chunked_prefill_size is None:
      self.chunked_prefill_size = self.max_num_batched_tokens
    if not self.enable_chunked_prefill:
      # a prompt must then fit one step whole
      self.chunked_prefill_size = self.max_num_batched_tokens

  @property
  def max_model_len(self) -> int:
    return self.max_context_len

  @classmethod
  def from_kwargs(cls, model_path: str, **kwargs: Any) -> "EngineConfig":
    if "max_model_len" in kwargs:
      if "max_context_len" in kwargs:
        raise TypeError("give max_model_len or max_context_len, not both")
      kwargs["max_context_len"] = kwargs.pop("max_model_len")
    names = {f.name for f in dataclasses.fields(cls)}
    unknown = sorted(k for k in kwargs if k not in names)
    if unknown:
      raise TypeError(f"unknown engine option(s): {', '.join(unknown)}; known: {', '.join(sorted(names))}")
    return cls(model_path=model_path, **kwargs)

  def to_dict(self) -> Dict[str, Any]:
    d = dataclasses.asdict(self)
    d["dtype"] = str(self.dtype).replace("torch.", "")
    return d
