"""What a step hands to the parts: the batch's device-side description and a workspace.

The reference's counterpart is ``ForwardBatch`` (miniinfer/scheduler/scheduler_batch.py:235-442).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch


class Workspace:
  """Named activation buffers that keep their address from step to step, so that a captured step
  can be replayed.  A buffer grows when a larger one is asked for (never while capturing)."""

  def __init__(self, device):
    self.device = device
    self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
    self._views: Dict[tuple, torch.Tensor] = {}     # (name, dtype, shape) -> view of the buffer as it is now
    self.frozen = False

  def buffer(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
    vkey = (name, dtype, tuple(shape))
    view = self._views.get(vkey)
    if view is not None:
      return view
    n = 1
    for s in shape:
      n *= int(s)
    key = (name, dtype)
    buf = self._bufs.get(key)
    if buf is None or buf.numel() < n:
      if self.frozen:
        raise RuntimeError(f"workspace buffer {name!r} would have to grow to {n} elements while frozen")
      buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
      self._bufs[key] = buf
      for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
        del self._views[k]                          # views of the buffer this one replaces
    if len(self._views) > 1024:
      self._views.clear()
    view = buf[:n].view(*shape)
    self._views[vkey] = view
    return view

  def zeros(self, name: str, n: int, dtype: torch.dtype) -> torch.Tensor:
    """A buffer that starts at zero and is left to its users afterwards (counters that kernels reset
    themselves, status words)."""
    key = (name, dtype)
    buf = self._bufs.get(key)
    if buf is None or buf.numel() < n:
      if self.frozen:
        raise RuntimeError(f"workspace buffer {name!r} would have to grow to {n} elements while frozen")
      buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
      self._bufs[key] = buf
    return buf[:n]

  def bytes(self) -> int:
    return sum(b.numel() * b.element_size() for b in self._bufs.values())


class StepContext:
  """Everything about the running step that a part may read.

  ``positions[t]``, ``token_item[t]``: per token; ``q_start/q_len/ctx_len/seq_slot[b]``: per item;
  ``slot_mapping[g][t]`` and ``block_tables[g]``: per group of paged layers; ``state_slots`` is
  ``seq_slot`` (the row of a request in every per-request state tensor); ``host`` keeps the same
  numbers as Python lists for parts that loop on the host (such a part sets ``reads_step_on_host``).
  ``work[name]`` is the device view of a work list that a part declared (``Part.step_work``) and
  ``work_key[name]`` its key, the host-side numbers the part's launches may depend on; ``shared`` is
  a scratch dictionary for what the layers of one step want to make once and share; ``captured``
  says that the step is being recorded into a CUDA graph (or run to prepare that)."""

  def __init__(self, dtype: torch.dtype, device, ws: Workspace):
    self.dtype = dtype
    self.device = device
    self.ws = ws
    self.num_tokens = 0
    self.num_items = 0
    self.ids: Optional[torch.Tensor] = None
    self.positions: Optional[torch.Tensor] = None
    self.token_item: Optional[torch.Tensor] = None
    self.q_start: Optional[torch.Tensor] = None
    self.q_len: Optional[torch.Tensor] = None
    self.ctx_len: Optional[torch.Tensor] = None
    self.seq_slot: Optional[torch.Tensor] = None
    self.logit_rows: Optional[torch.Tensor] = None
    self.slot_mapping: List[torch.Tensor] = []
    self.block_tables: List[torch.Tensor] = []
    self.host: Dict[str, list] = {}
    self.extra: Dict[str, torch.Tensor] = {}
    self.work: Dict[str, torch.Tensor] = {}
    self.work_key: Dict[str, tuple] = {}
    self.shared: Dict[str, object] = {}
    self.captured = False

  @property
  def state_slots(self) -> torch.Tensor:
    return self.seq_slot
