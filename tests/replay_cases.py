"""Traces for the replay tests: the same requests cut into steps in different ways, and the
comparison of what comes back with the plain implementation.

A trace is a list of records as ``bin/trace_run`` reads them:
``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}``.
"""

from __future__ import annotations

import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import plain_qwen3 as plain


def make_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
  g = torch.Generator().manual_seed(seed)
  return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def round_up(n: int, m: int = 64) -> int:
  return -(-n // m) * m


# ------------------------------------------------------------------------------ ways of cutting


def whole(reqs: Dict[str, List[int]]) -> List[dict]:
  """Each request alone and whole, one step each."""
  return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
          for i, (rid, ids) in enumerate(reqs.items())]


def tail_one_by_one(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
  """Most of a request in one step, its last ``tail`` tokens one by one."""
  trace, step = [], 0
  for rid, ids in reqs.items():
    k = min(tail, len(ids) - 1)
    head = ids[:len(ids) - k]
    trace.append({"step": step, "entries": [{"id": rid, "tokens": head, "want": list(range(len(head)))}],
                  "end": [rid] if k == 0 else []})
    step += 1
    for j in range(len(head), len(ids)):
      trace.append({"step": step, "entries": [{"id": rid, "tokens": [ids[j]], "want": [0]}],
                    "end": [rid] if j == len(ids) - 1 else []})
      step += 1
  return trace


def portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (13, 7, 2, 29, 3, 2, 5, 17, 2, 64, 1, 2)) -> List[dict]:
  """Each request alone, in portions of changing size, down to two tokens (and one)."""
  trace, step, k = [], 0, 0
  for rid, ids in reqs.items():
    pos = 0
    while pos < len(ids):
      n = min(sizes[k % len(sizes)], len(ids) - pos)
      k += 1
      trace.append({"step": step, "entries": [{"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))}],
                    "end": [rid] if pos + n == len(ids) else []})
      pos += n
      step += 1
  return trace


def mixed(reqs: Dict[str, List[int]], max_tokens: int, seed: int, max_live: int = 4, decode_tail: int = 6,
          granule: int = 64, preempt: bool = False) -> List[dict]:
  """Up to ``max_live`` requests at a time: portions of some beside single tokens of others, some left
  out of a step now and then, a new request starting as soon as one has ended and its room
  (``granule``-rounded) is free again - so that pages are used again.

  ``preempt``: every request of more than eight tokens is, once, ended mid-way (what a scheduler does
  when pages run out: everything the request holds is given back), waits behind the next request, and
  comes back under the same id with all the tokens it had been fed as ONE portion, then goes on
  where it was.  The logits of its second life must be those of its first at every position."""
  rng = random.Random(seed)
  prng = random.Random(seed + 1000)           # draws of its own, so that preempt=False gives the traces it always gave
  waiting = [(rid, ids, 0) for rid, ids in reqs.items()]
  live: Dict[str, dict] = {}
  cut_at = {rid: prng.randint(max(2, len(ids) // 3), len(ids) - 2) for rid, ids in reqs.items() if preempt and len(ids) > 8}
  trace, step = [], 0
  while waiting or live:
    held = sum(round_up(len(v["ids"]), granule) for v in live.values())
    while waiting and len(live) < max_live and held + round_up(len(waiting[0][1]), granule) <= max_tokens:
      rid, ids, resume = waiting.pop(0)
      live[rid] = {"ids": ids, "pos": 0, "resume": resume}
      held += round_up(len(ids), granule)
    assert live, "max_tokens is too small for the next request"
    entries, end, again = [], [], []
    chosen = [rid for rid in live if rng.random() < 0.8] or [next(iter(live))]
    for rid in chosen:
      st = live[rid]
      left = len(st["ids"]) - st["pos"]
      if st["resume"]:
        n, st["resume"] = st["resume"], 0       # the second life starts with everything fed so far, as one portion
      elif left <= decode_tail:
        n = 1
      else:
        n = min(left - decode_tail, rng.choice((2, 3, 5, 8, 13, 21, 40)))
      if rid in cut_at and st["pos"] < cut_at[rid] < st["pos"] + n:
        n = cut_at[rid] - st["pos"]
      toks = st["ids"][st["pos"]:st["pos"] + n]
      entries.append({"id": rid, "tokens": toks, "want": list(range(n)) if rng.random() < 0.8 or n > 64 else [n - 1]})
      st["pos"] += n
      if st["pos"] == len(st["ids"]):
        end.append(rid)
      elif cut_at.get(rid) == st["pos"]:
        del cut_at[rid]
        end.append(rid)
        again.append((rid, st["ids"], st["pos"]))
    for rid in end:
      del live[rid]
    # a preempted request waits behind the next one in line, so that its pages are taken meanwhile
    waiting[1:1] = again
    trace.append({"step": step, "entries": entries, "end": end})
    step += 1
  return trace


# ------------------------------------------------------------------------------ running and comparing


def collect(trace: List[dict], outputs: Dict[int, np.ndarray]) -> Dict[tuple, np.ndarray]:
  """(request, position) -> logits row, from the per-step outputs.  A request that was ended and came
  back under the same id starts again at position 0; rows of its later lives are kept under
  (request, position, life) beside those of the first."""
  pos: Dict[str, int] = {}
  life: Dict[str, int] = {}
  got: Dict[tuple, np.ndarray] = {}
  for rec in trace:
    rows = outputs.get(rec["step"])
    r = 0
    for e in rec["entries"]:
      start = pos.get(e["id"], 0)
      n = life.get(e["id"], 0)
      for w in e["want"]:
        got[(e["id"], start + w) if n == 0 else (e["id"], start + w, n)] = rows[r]
        r += 1
      pos[e["id"]] = start + len(e["tokens"])
    for rid in rec.get("end", []):
      if rid in pos:
        del pos[rid]
        life[rid] = life.get(rid, 0) + 1
    assert rows is None or r == rows.shape[0]
  return got


def run_in_process(runner, trace: List[dict]) -> Dict[Tuple[str, int], np.ndarray]:
  outputs = {}
  for rec in trace:
    out = runner.run_step(rec)
    if out is not None:
      outputs[rec["step"]] = np.array(out, copy=True)
  return collect(trace, outputs)


def reference_logits(model_dir: str, reqs: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
  w, c = plain.read_weights(model_dir), plain.read_config(model_dir)
  return {rid: plain.forward(w, c, ids) for rid, ids in reqs.items()}


def compare(got: Dict[Tuple[str, int], np.ndarray], ref: Dict[str, torch.Tensor], atol: float, what: str,
            check_argmax_margin: float = None) -> float:
  """Every wanted row against the plain implementation; says where the first wrong row is."""
  worst = 0.0
  assert got, "nothing was compared"
  for key, row in sorted(got.items()):
    rid, p = key[0], key[1]
    r = ref[rid][p].numpy()
    d = float(np.abs(row - r).max())
    worst = max(worst, d)
    assert np.isfinite(row).all(), f"{what}: request {rid} position {p}: logits are not finite"
    assert d <= atol, (f"{what}: request {rid} position {p}: max |diff| {d:.3e} > {atol:.1e} "
                       f"(first wrong row; earlier positions of this request agree)")
    if check_argmax_margin is not None:
      top2 = np.sort(r)[-2:]
      if top2[1] - top2[0] > check_argmax_margin:
        assert int(row.argmax()) == int(r.argmax()), f"{what}: request {rid} position {p}: another greedy token"
  return worst


def log_worst(what: str, worst: float, ref: Dict[str, torch.Tensor]) -> None:
  """With MINIINFER_B200_DIFF_LOG=<file> the largest difference of every comparison is appended there,
  beside the largest reference logit: the record from which the bfloat16 bounds of the tests are set."""
  path = os.environ.get("MINIINFER_B200_DIFF_LOG")
  if path:
    top = max(float(v.abs().max()) for v in ref.values())
    with open(path, "a") as f:
      f.write(f"{what} worst_abs_diff={worst:.6f} max_abs_logit={top:.4f}\n")
