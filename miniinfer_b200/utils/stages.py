"""Named stage ranges around the phases of an engine step, for profiler traces.

``with stage("schedule"):`` marks a range ``stage::schedule`` that ``torch.profiler`` (and any tool
that reads its ranges) shows beside the kernels.  Ranges cost a few microseconds each, so they are
off unless switched on: ``enable_stages(True)``, the command line's ``--profile``, or
``MINIINFER_B200_PROFILE_STAGES=1``.  The reference marks its engine's methods the same way
(miniinfer/utils/profiler_utils.py:17-79, ranges named ``stage::<component>.<method>``).
"""

from __future__ import annotations

import os
from contextlib import contextmanager

_enabled = os.environ.get("MINIINFER_B200_PROFILE_STAGES", "0").strip().lower() in ("1", "true", "on", "yes")


def enable_stages(on: bool = True) -> None:
  global _enabled
  _enabled = bool(on)


def stages_enabled() -> bool:
  return _enabled


@contextmanager
def stage(name: str):
  """A range ``stage::<name>`` around the block, if stage ranges are on; otherwise nothing."""
  if not _enabled:
    yield
    return
  from torch.profiler import record_function
  with record_function(f"stage::{name}"):
    yield


@contextmanager
def profile_to(path: str):
  """Runs the block under ``torch.profiler`` with stage ranges on and writes two tables to ``path``: the
  stage ranges with their host time, and the kernels with their device time."""
  import torch
  from torch.profiler import ProfilerActivity, profile
  was = _enabled
  enable_stages(True)
  activities = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
  try:
    with profile(activities=activities) as prof:
      yield
      if torch.cuda.is_available():
        torch.cuda.synchronize()
  finally:
    enable_stages(was)
  rows = prof.key_averages()
  stages = sorted((r for r in rows if r.key.startswith("stage::")), key=lambda r: -r.cpu_time_total)
  kernels = sorted((r for r in rows if (getattr(r, "device_time_total", 0) or 0) > 0 and not r.key.startswith("stage::")),
                   key=lambda r: -r.device_time_total)
  with open(path, "w", encoding="utf-8") as f:
    f.write("stage ranges (host time)\n")
    for r in stages:
      f.write(f"{r.cpu_time_total / 1e3:10.3f} ms  {r.count:7d} x  {r.cpu_time_total / max(r.count, 1):9.1f} us each  {r.key}\n")
    f.write("\nkernels (device time)\n")
    for r in kernels[:40]:
      f.write(f"{r.device_time_total / 1e3:10.3f} ms  {r.count:7d} x  {r.device_time_total / max(r.count, 1):9.1f} us each  {r.key[:120]}\n")
