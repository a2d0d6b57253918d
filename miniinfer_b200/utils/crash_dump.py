"""What the engine knew when a step failed, as one structured log record.

A traceback alone rarely says why a step raised: one also wants the scheduler's queues, the cache's
occupancy and the batch that was being run.  ``dump_step_failure`` collects them.  Every field is
read defensively - the dump must never raise and hide the error it reports - and tensors are
summarised (shape, dtype, device, a few statistics), not printed.  The reference has the same tool
(miniinfer/utils/crash_logger.py:1-239).
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from .logging import get_logger

logger = get_logger("crash")


def tensor_summary(t: Any) -> str:
  """Shape, dtype, device and a few statistics of a tensor; ``repr`` of anything else."""
  try:
    import torch
    if isinstance(t, torch.Tensor):
      s = f"shape={tuple(t.shape)} dtype={t.dtype} device={t.device}"
      if t.numel() > 0 and t.is_floating_point():
        f = t.detach().float()
        s += f" min={f.min().item():.4g} max={f.max().item():.4g} mean={f.mean().item():.4g} finite={bool(torch.isfinite(f).all())}"
      elif t.numel() > 0 and not t.is_complex():
        s += f" min={t.min().item()} max={t.max().item()}"
      return s
  except Exception as e:  # noqa: BLE001 - a failed summary is itself reported, not raised
    return f"<summary failed: {e!r}>"
  return repr(t)


def describe_step_failure(exc: BaseException, scheduler: Any = None, cache: Any = None, runner: Any = None,
                          items: Optional[List[Any]] = None, stage: str = "step") -> Dict[str, Any]:
  """The record as a dictionary (what ``dump_step_failure`` logs)."""
  rec: Dict[str, Any] = {"stage": stage, "error": f"{type(exc).__name__}: {exc}"}

  def guarded(name, fn):
    try:
      rec[name] = fn()
    except Exception as e:  # noqa: BLE001
      rec[name] = f"<unavailable: {e!r}>"

  if scheduler is not None:
    guarded("waiting", lambda: len(scheduler.waiting))
    guarded("running", lambda: [{"id": r.req_id, "prompt": len(r.prompt_ids), "outputs": len(r.output_ids),
                                 "computed": r.num_computed, "status": r.status} for r in scheduler.running])
    guarded("preemptions", lambda: scheduler.num_preemptions)
  if cache is not None:
    guarded("cache", lambda: cache.get_stats())
  if items is not None:
    guarded("batch", lambda: [{"id": it.req_id, "tokens": len(it.tokens), "want": len(it.want),
                               "length_before": cache.length_of(it.req_id) if cache is not None and cache.has_request(it.req_id) else None}
                              for it in items])
  if runner is not None:
    guarded("graphs", lambda: runner.num_graphs())
    guarded("last_launches", lambda: runner.last_launches)
    guarded("workspace_bytes", lambda: runner.ws.bytes())
    guarded("kernel_libraries", lambda: __import__("miniinfer_b200.kernels.ops", fromlist=["x"]).loaded_libraries())
  return rec


def dump_step_failure(exc: BaseException, scheduler: Any = None, cache: Any = None, runner: Any = None,
                      items: Optional[List[Any]] = None, stage: str = "step") -> Dict[str, Any]:
  """Logs the record at ERROR level, one line per field, and returns it.  Never raises."""
  try:
    rec = describe_step_failure(exc, scheduler, cache, runner, items, stage)
    logger.error("==== a step failed: %s ====", rec.get("error"))
    for k, v in rec.items():
      if k != "error":
        logger.error("  %s: %s", k, v)
    return rec
  except Exception as e:  # noqa: BLE001
    try:
      logger.error("crash dump failed: %r", e)
    except Exception:  # noqa: BLE001
      pass
    return {"error": repr(exc)}
