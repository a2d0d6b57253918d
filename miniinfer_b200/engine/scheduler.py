"""Continuous batching on the host: admission, portions of prompts under a token budget, decode,
finishing, and what happens when pages run out.

The scheduler decides with host counters only; it asks the cache manager what an append would
cost and never touches the device (the reference allocates inside ``schedule()``,
miniinfer/scheduler/scheduler.py:290-517).

Policy, every step:
  1. every running request whose prompt is in the cache gets its one decode token
     (the reference tries to build a prefill batch first, scheduler.py:270-283, and lets decode
     tokens ride along only in its mixed mode, :417-434; here every step is mixed);
  2. what is left of ``max_num_batched_tokens`` goes to portions of running requests that are still
     in their prompt, oldest first, then to waiting requests in arrival order, each portion at most
     ``chunked_prefill_size`` tokens and cut anywhere (the reference rounds portions to whole pages,
     miniinfer/scheduler/prefill_adder.py:317-364);
  3. a request is admitted only while a slot is free, fewer than ``max_num_seqs`` are running and
     the pages for its first portion are free.

When pages run out: if a decode token cannot get its page, the most recently admitted running
request is preempted - its pages and slot go back, it keeps the tokens it has generated, and it
returns to the head of the waiting queue; when it is admitted again it runs prompt plus generated
tokens as a prompt and goes on from there.  (The reference retracts from the tail as well but throws
the generated tokens away, scheduler.py:553-598.)  The same happens when nothing at all could be
scheduled because prompts in progress hold all pages.  A request that could never fit the pool, or
is longer than ``max_model_len``, is refused when it is added.
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
  """One generation request (the reference's ``Req``, miniinfer/scheduler/scheduler_batch.py:45-119)."""

  req_id: Hashable
  prompt_ids: List[int]
  params: SamplingParams
  number: int = 0                     # arrival order; also feeds the default seed
  seed: int = 0
  output_ids: List[int] = field(default_factory=list)
  num_computed: int = 0               # tokens whose keys and values are in the cache
  status: str = WAITING
  finish_reason: Optional[str] = None
  max_tokens: int = 0                 # params.max_tokens clamped to max_model_len
  preemptions: int = 0

  def all_ids(self) -> List[int]:
    return self.prompt_ids + self.output_ids

  def ids(self, start: int, stop: int) -> List[int]:
    """Tokens ``start .. stop`` of prompt followed by output, without joining the two lists."""
    n = len(self.prompt_ids)
    if stop <= n:
      return self.prompt_ids[start:stop]
    if start >= n:
      return self.output_ids[start - n:stop - n]
    return self.prompt_ids[start:] + self.output_ids[:stop - n]

  @property
  def total_len(self) -> int:
    return len(self.prompt_ids) + len(self.output_ids)


@dataclass
class ScheduledItem:
  request: Request
  tokens: List[int]
  samples: bool          # True: the portion ends the known tokens, its last row is sampled


@dataclass
class SchedulerOutput:
  items: List[ScheduledItem]
  preempted: List[Request] = field(default_factory=list)
  num_prefill_tokens: int = 0
  num_decode_tokens: int = 0


class Scheduler:
  def __init__(self, cache, max_num_seqs: int, max_num_batched_tokens: int, chunked_prefill_size: int,
               max_model_len: int, eos_ids: Sequence[int] = ()):
    self.cache = cache
    self.max_num_seqs = max_num_seqs
    self.max_num_batched_tokens = max_num_batched_tokens
    self.chunked_prefill_size = chunked_prefill_size
    self.max_model_len = max_model_len
    self.eos_ids = set(int(e) for e in eos_ids)
    self.waiting: Deque[Request] = deque()
    self.running: List[Request] = []          # in order of admission
    self.finished: List[Request] = []
    self._numbers = itertools.count()
    self.num_preemptions = 0

  # ------------------------------------------------------------------ queue

  def add(self, req: Request) -> None:
    n = len(req.prompt_ids)
    if n < 1:
      raise ValueError("a prompt needs at least one token")
    if n >= self.max_model_len:
      raise ValueError(f"the prompt has {n} tokens; max_model_len={self.max_model_len} leaves no room to generate")
    req.max_tokens = min(req.params.max_tokens, self.max_model_len - n)
    # the whole request must fit the pool on its own, or it could never finish
    need = self.cache.pages_needed(None, n + req.max_tokens)
    total = [g.num_pages for g in self.cache.paged_groups]
    windowed = [g.spec.window is not None for g in self.cache.paged_groups]
    for g, (want, have) in enumerate(zip(need, total)):
      if want > have and not windowed[g]:
        raise ValueError(f"the request needs {want} pages of cache group {g}, the pool has {have}")
    req.number = next(self._numbers)
    req.status = WAITING
    self.waiting.append(req)

  def has_unfinished(self) -> bool:
    return bool(self.waiting or self.running)

  # ------------------------------------------------------------------ one step's decisions

  def _fits(self, req_id, n: int, pending: List[int]) -> bool:
    need = self.cache.pages_needed(req_id, n)
    free = self.cache.free_pages()
    return all(a + b <= f for a, b, f in zip(need, pending, free))

  def _take(self, req_id, n: int, pending: List[int]) -> None:
    for g, a in enumerate(self.cache.pages_needed(req_id, n)):
      pending[g] += a

  def _preempt(self, req: Request, out: SchedulerOutput) -> None:
    self.running.remove(req)
    self.cache.release_request(req.req_id)
    req.num_computed = 0
    req.status = WAITING
    req.preemptions += 1
    self.num_preemptions += 1
    self.waiting.appendleft(req)
    out.preempted.append(req)

  def _largest_fitting(self, req_id, want: int, pending: List[int]) -> int:
    """The largest portion <= want whose pages are free (0 if not even one token fits)."""
    if self._fits(req_id, want, pending):
      return want
    lo, hi = 0, want      # fits(lo) holds (lo = 0 costs nothing), fits(hi) fails
    while hi - lo > 1:
      mid = (lo + hi) // 2
      if self._fits(req_id, mid, pending):
        lo = mid
      else:
        hi = mid
    return lo

  def schedule(self) -> SchedulerOutput:
    out = SchedulerOutput(items=[])
    while True:
      out.num_decode_tokens = out.num_prefill_tokens = 0
      self._schedule_once(out)
      if out.items or not self.running:
        break
      # prompts in progress hold every page and none can move: give the newest one's pages back
      self._preempt(self.running[-1], out)
    return out

  def _schedule_once(self, out: SchedulerOutput) -> None:
    budget = self.max_num_batched_tokens
    pending = [0] * len(self.cache.paged_groups)
    items: List[ScheduledItem] = []
    scheduled = set()

    # 1. decode tokens; give the newest requests' pages back until all of them fit
    while True:
      decoders = [r for r in self.running if r.total_len - r.num_computed == 1][:budget]
      need = [0] * len(pending)
      for r in decoders:
        for g, a in enumerate(self.cache.pages_needed(r.req_id, 1)):
          need[g] += a
      if all(a <= f for a, f in zip(need, self.cache.free_pages())):
        break
      self._preempt(self.running[-1], out)
    for req in decoders:
      self._take(req.req_id, 1, pending)
      items.append(ScheduledItem(req, req.ids(req.total_len - 1, req.total_len), True))
      scheduled.add(req.req_id)
      budget -= 1
      out.num_decode_tokens += 1

    # 2. portions of prompts in progress, oldest first
    for req in self.running:
      if budget < 1:
        break
      remaining = req.total_len - req.num_computed
      if req.req_id in scheduled or remaining < 1:
        continue
      n = self._largest_fitting(req.req_id, min(remaining, budget, self.chunked_prefill_size), pending)
      if n < 1:
        continue
      self._take(req.req_id, n, pending)
      ids = req.ids(req.num_computed, req.num_computed + n)
      items.append(ScheduledItem(req, ids, n == remaining))
      scheduled.add(req.req_id)
      budget -= n
      out.num_prefill_tokens += n

    # 3. admission, in arrival order
    while self.waiting and budget >= 1 and len(self.running) < self.max_num_seqs and self.cache.num_free_slots > 0:
      req = self.waiting[0]
      remaining = req.total_len
      want = min(remaining, budget, self.chunked_prefill_size)
      n = self._largest_fitting(None, want, pending)
      if n < want and (n < 1 or self.running):
        break       # wait until pages come back, rather than start a prompt in small pieces
      self.waiting.popleft()
      self.cache.admit(req.req_id)
      req.status = RUNNING
      self.running.append(req)
      self._take(req.req_id, n, pending)
      items.append(ScheduledItem(req, req.ids(0, n), n == remaining))
      scheduled.add(req.req_id)
      budget -= n
      out.num_prefill_tokens += n

    out.items = items

  # ------------------------------------------------------------------ after the step

  def update(self, out: SchedulerOutput, sampled: Dict[Hashable, int]) -> List[Request]:
    """Records the step's tokens; returns the requests that finished (their pages are free again)."""
    done: List[Request] = []
    for item in out.items:
      req = item.request
      req.num_computed += len(item.tokens)
      if not item.samples:
        continue
      tok = int(sampled[req.req_id])
      req.output_ids.append(tok)
      reason = None
      if not req.params.ignore_eos and tok in self.eos_ids:
        reason = "eos"
      elif len(req.output_ids) >= req.max_tokens:
        reason = "max_tokens" if req.max_tokens == req.params.max_tokens else "length"
      if reason is not None:
        req.finish_reason = reason
        req.status = FINISHED
        self.running.remove(req)
        self.cache.release_request(req.req_id)
        self.finished.append(req)
        done.append(req)
    return done

  def get_stats(self) -> dict:
    return {"waiting": len(self.waiting), "running": len(self.running), "finished": len(self.finished),
            "preemptions": self.num_preemptions}
