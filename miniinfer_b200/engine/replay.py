"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and schedules nothing.  It drives the package's own model, step function, cache
manager and kernels - the ones generation uses - with the steps it reads, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

A request is admitted when it first appears and released when a step lists it under ``end``.  For a
step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted places, in
the order of the entries and of ``want``, as little-endian float32 ``[wanted, vocab]``.  After every
step a line ``done <step>`` is printed and flushed.

The closest things in the reference are two debugging scripts that compare cached decoding with a
whole-prompt pass (tests/debug/test_kv_cache_consistency.py, test_multi_batch_kv_consistency.py).
"""

from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np
import torch

from ..cache.manager import KVCacheManager
from ..config import build_model_spec, load_model_config, parse_dtype
from ..weights import load_weights
from .runner import ModelRunner, StepItem

TRACE_PAGE_SIZE = 64
MAX_LIVE_REQUESTS = 8


class TraceRunner:
  def __init__(self, model_dir: str, dtype, max_tokens: int, device: str = "cuda:0",
               page_size: int = TRACE_PAGE_SIZE, num_pages: Optional[int] = None):
    self.dtype = parse_dtype(dtype)
    self.device = torch.device(device)
    if self.device.type == "cuda":
      torch.cuda.set_device(self.device)
      torch.backends.cuda.matmul.allow_tf32 = False
      torch.backends.cudnn.allow_tf32 = False
    self.model_config = load_model_config(model_dir)
    self.spec = build_model_spec(self.model_config)
    load_weights(self.spec, model_dir, self.dtype, self.device)
    if page_size < 1:
      raise ValueError(f"page size must be positive, got {page_size}")
    if num_pages is None:
      num_pages = max(1, -(-int(max_tokens) // page_size))
    max_len = min(self.model_config.max_position_embeddings, num_pages * page_size)
    self.cache = KVCacheManager(self.spec.cache_layer_specs(), page_size, num_pages, MAX_LIVE_REQUESTS, max_len,
                                self.dtype, self.device)
    self.runner = ModelRunner(self.spec, self.cache, self.dtype, self.device)

  def run_step(self, record: dict) -> Optional[np.ndarray]:
    """Runs one step; returns the wanted logits as float32 [wanted, vocab], or None."""
    items = []
    for e in record.get("entries", []):
      rid = e["id"]
      if not self.cache.has_request(rid):
        self.cache.admit(rid)
      items.append(StepItem(rid, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
    logits = None
    if items:
      out = self.runner.step(items)
      if out.shape[0] > 0:
        logits = out.float().cpu().numpy().astype("<f4", copy=False)
      elif self.device.type == "cuda":
        torch.cuda.synchronize()
      self.runner.check_status()
    for rid in record.get("end", []):
      if self.cache.has_request(rid):
        self.cache.release_request(rid)
    return logits


def main(argv=None, stdin: Optional[IO[str]] = None, stdout: Optional[IO[str]] = None) -> int:
  import argparse

  p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
  p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
  p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
  p.add_argument("--out", required=True, help="folder for <step>.f32 files")
  p.add_argument("--max-tokens", type=int, required=True,
                 help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
  p.add_argument("--page-size", type=int, default=TRACE_PAGE_SIZE, help="tokens per page of the cache (default 64)")
  p.add_argument("--num-pages", type=int, default=None,
                 help="pages of the cache pool (default: --max-tokens divided by the page size, rounded up)")
  p.add_argument("--device", default="cuda:0")
  args = p.parse_args(argv)
  stdin = stdin or sys.stdin
  stdout = stdout or sys.stdout
  os.makedirs(args.out, exist_ok=True)
  tr = TraceRunner(args.model, args.dtype, args.max_tokens, args.device, page_size=args.page_size, num_pages=args.num_pages)
  for line in stdin:
    line = line.strip()
    if not line:
      continue
    record = json.loads(line)
    logits = tr.run_step(record)
    if logits is not None:
      logits.tofile(os.path.join(args.out, f"{record['step']}.f32"))
    print(f"done {record['step']}", file=stdout, flush=True)
  return 0
