"""The cache manager: pages of keys and values with a block table per request, one pool per group
of layers with the same need, and slots for per-request state of fixed size.

Against the reference (miniinfer/kvcache/kv_cache_manager.py, memory_pool.py):
  * the free list lives on the host (the reference keeps it in a device tensor and allocates with
    Triton kernels, memory_pool.py:245-459); allocating costs no device work;
  * the block table is direct, ``[slot, page index] -> page id`` (the reference maps token -> slot,
    memory_pool.py:476-478, and derives pages each step);
  * page 0 of every pool is a dummy that padded tokens may write to (memory_pool.py:422-424);
  * a request keeps its slot and pages from admission to release, also between portions of its
    prompt (the reference frees the slot between chunks, llm_engine.py:1178-1181);
  * pages behind a layer group's window are given back as soon as no later query can see them.

The manager does no scheduling: callers ask ``can_append`` and then ``append``; ``commit`` makes
the appended tokens part of the request after the step has run.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

STAGING_SLOTS = 8     # pinned snapshots of a block table that uploads in flight may still read

from .specs import CacheSpec, FixedStateSpec, PagedKVSpec


class OutOfPages(RuntimeError):
  """An append that the free pages of some group cannot cover.  Nothing was allocated."""


class OutOfSlots(RuntimeError):
  """No request slot is free."""


class PageAllocator:
  """Host free list of the page ids ``1..num_pages`` (0 is the dummy page).  Last freed, first
  reused.  Holding a page twice or freeing it twice is an error."""

  def __init__(self, num_pages: int):
    if num_pages < 1:
      raise ValueError("a pool needs at least one page")
    self.num_pages = num_pages
    self._free: List[int] = list(range(num_pages, 0, -1))
    self._held = bytearray(num_pages + 1)

  @property
  def num_free(self) -> int:
    return len(self._free)

  def alloc(self, n: int) -> List[int]:
    if n > len(self._free):
      raise OutOfPages(f"{n} pages wanted, {len(self._free)} free")
    out = [self._free.pop() for _ in range(n)]
    for p in out:
      if self._held[p]:
        raise AssertionError(f"page {p} handed out twice")
      self._held[p] = 1
    return out

  def free(self, pages: Sequence[int]) -> None:
    for p in pages:
      if p <= 0 or p > self.num_pages or not self._held[p]:
        raise AssertionError(f"page {p} freed but not held")
      self._held[p] = 0
      self._free.append(p)

  def held(self) -> List[int]:
    return [p for p in range(1, self.num_pages + 1) if self._held[p]]


class PagedGroup:
  """The pool, allocator and block table of the layers that share one ``PagedKVSpec``.

  Pool layout ``[layer, page, 2 (key, value), kv head, token in page, head_dim]``: the keys (or
  values) of one page and one head are one contiguous ``page_size x head_dim`` box."""

  def __init__(self, index: int, spec: PagedKVSpec, num_layers: int, page_size: int, num_pages: int,
               max_num_seqs: int, max_model_len: int, dtype: torch.dtype, device):
    self.index = index
    self.spec = spec
    self.num_layers = num_layers
    self.page_size = page_size
    self.num_pages = num_pages
    self.max_pages_per_seq = -(-max_model_len // page_size)
    self.allocator = PageAllocator(num_pages)
    self.kv = torch.zeros((num_layers, num_pages + 1, 2, spec.num_kv_heads, page_size, spec.head_dim),
                          dtype=dtype, device=device)
    self.block_table_host = np.zeros((max_num_seqs + 1, self.max_pages_per_seq), dtype=np.int32)
    self.block_table = torch.zeros((max_num_seqs + 1, self.max_pages_per_seq), dtype=torch.int32, device=device)
    self._dirty: set = set()
    # Uploads go through a ring of pinned copies of the table: the copy is queued on the stream and
    # reads host memory when the device gets to it, by when the host may have changed the table
    # again for a later step - so each upload reads a snapshot of its own, taken when it is queued.
    self._staging: List[torch.Tensor] = []
    self._staging_events: List[Optional[torch.cuda.Event]] = []
    self._staging_next = 0
    if torch.device(device).type == "cuda":
      for _ in range(STAGING_SLOTS):
        self._staging.append(torch.zeros((max_num_seqs + 1, self.max_pages_per_seq), dtype=torch.int32).pin_memory())
        self._staging_events.append(None)

  def bytes_per_token(self) -> int:
    return 2 * self.num_layers * self.spec.num_kv_heads * self.spec.head_dim * self.kv.element_size()

  def first_needed_page(self, length: int) -> int:
    """Index of the first page that a query at position ``length`` (the next one) can still see."""
    if self.spec.window is None:
      return 0
    return max(0, length - self.spec.window + 1) // self.page_size

  def sync(self) -> None:
    """Uploads the block-table rows that changed since the last call."""
    if not self._dirty:
      return
    rows = sorted(self._dirty)
    self._dirty.clear()
    lo, hi = rows[0], rows[-1] + 1
    if not self._staging:                 # a table on the host (tests of the host path): plain copy
      self.block_table[lo:hi].copy_(torch.from_numpy(self.block_table_host[lo:hi]))
      return
    k = self._staging_next
    self._staging_next = (k + 1) % len(self._staging)
    if self._staging_events[k] is not None:
      self._staging_events[k].synchronize()      # the upload that used this snapshot last has run (long ago, as a rule)
    else:
      self._staging_events[k] = torch.cuda.Event()
    snap = self._staging[k]
    snap.numpy()[lo:hi] = self.block_table_host[lo:hi]
    self.block_table[lo:hi].copy_(snap[lo:hi], non_blocking=True)
    self._staging_events[k].record()


class StateGroup:
  """Per-request state of fixed size: ``[layer, slot, *shape]``; the last slot is for padding."""

  def __init__(self, index: int, spec: FixedStateSpec, num_layers: int, max_num_seqs: int, device):
    self.index = index
    self.spec = spec
    self.num_layers = num_layers
    self.state = torch.zeros((num_layers, max_num_seqs + 1) + tuple(spec.shape),
                             dtype=getattr(torch, spec.dtype), device=device)


@dataclass
class LayerCache:
  """What a mixer gets for one entry of the run list."""

  kind: str                       # "paged", "state" or "none"
  group: int = -1                 # index among the groups of its kind
  tensor: Optional[torch.Tensor] = None   # paged: [page, 2, kv head, token, head_dim]; state: [slot, *shape]
  writes: bool = True             # False: the entry reads the cache another entry writes
  page_size: int = 0


@dataclass
class _Request:
  slot: int
  length: int = 0                 # committed tokens
  reserved: int = 0               # tokens appended but not committed
  pages: List[List[int]] = field(default_factory=list)   # per paged group: page ids by index, 0 = given back


def pages_in_flight(window: int, page_size: int, max_step_tokens: int) -> int:
  """The most pages a request holds in a group that keeps the last ``window`` positions: the window, what up to two
  steps of ``max_step_tokens`` tokens add before the first of them is committed and the pages behind the window go
  back, and one page for where the window starts inside a page."""
  return -(-(window + 2 * max_step_tokens) // page_size) + 1


class KVCacheManager:
  """``layer_specs[i]`` is the need of cache layer ``i`` (None: the layer keeps nothing).

  ``num_pages`` is the size of a group that keeps every key.  A group that keeps a window needs no more than its
  requests can hold at a time: with ``max_step_tokens`` (the most tokens a request gets in one step) such a group
  gets ``max_num_seqs * pages_in_flight(window, ...)`` pages, if that is less."""

  def __init__(self, layer_specs: Sequence[Optional[CacheSpec]], page_size: int, num_pages: int,
               max_num_seqs: int, max_model_len: int, dtype: torch.dtype, device="cpu",
               max_step_tokens: Optional[int] = None):
    self.page_size = page_size
    self.max_num_seqs = max_num_seqs
    self.max_model_len = max_model_len
    self.dtype = dtype
    self.device = device
    self.paged_groups: List[PagedGroup] = []
    self.state_groups: List[StateGroup] = []
    self._layer_place: List[Optional[tuple]] = []      # (kind, group index, layer index in group)
    by_spec: Dict[CacheSpec, List[int]] = {}
    for i, spec in enumerate(layer_specs):
      if spec is not None:
        by_spec.setdefault(spec, []).append(i)
    place: Dict[int, tuple] = {}
    for spec, layers in by_spec.items():
      if isinstance(spec, PagedKVSpec):
        g = PagedGroup(len(self.paged_groups), spec, len(layers), page_size,
                       self.group_pages(spec, page_size, num_pages, max_num_seqs, max_step_tokens),
                       max_num_seqs, max_model_len, dtype, device)
        self.paged_groups.append(g)
        for j, layer in enumerate(layers):
          place[layer] = ("paged", g.index, j)
      elif isinstance(spec, FixedStateSpec):
        s = StateGroup(len(self.state_groups), spec, len(layers), max_num_seqs, device)
        self.state_groups.append(s)
        for j, layer in enumerate(layers):
          place[layer] = ("state", s.index, j)
      else:
        raise TypeError(f"unknown cache spec {spec!r}")
    self._layer_place = [place.get(i) for i in range(len(layer_specs))]
    self._free_slots: List[int] = list(range(max_num_seqs - 1, -1, -1))
    self._requests: Dict[Hashable, _Request] = {}
    self.pad_slot = max_num_seqs

  # ------------------------------------------------------------------ sizing

  @staticmethod
  def group_pages(spec: PagedKVSpec, page_size: int, num_pages: int, max_num_seqs: int, max_step_tokens: Optional[int]) -> int:
    """Pages of the group of ``spec`` when a group that keeps every key has ``num_pages``."""
    if spec.window is None or max_step_tokens is None:
      return num_pages
    return min(num_pages, max_num_seqs * pages_in_flight(spec.window, page_size, max_step_tokens))

  @staticmethod
  def bytes_per_page(layer_specs: Sequence[Optional[CacheSpec]], page_size: int, dtype: torch.dtype,
                     windowed: Optional[bool] = None) -> int:
    """Bytes that one more page costs in every paged group (``windowed`` None), in the groups that keep a window
    (True) or in those that keep every key (False)."""
    size = torch.empty((), dtype=dtype).element_size()
    total = 0
    for spec in layer_specs:
      if isinstance(spec, PagedKVSpec) and (windowed is None or windowed == (spec.window is not None)):
        total += 2 * spec.num_kv_heads * spec.head_dim * page_size * size
    return total

  # ------------------------------------------------------------------ views for the model

  def layer_cache(self, cache_layer: Optional[int], writes: bool = True) -> LayerCache:
    if cache_layer is None or self._layer_place[cache_layer] is None:
      return LayerCache(kind="none", writes=False)
    kind, g, j = self._layer_place[cache_layer]
    if kind == "paged":
      return LayerCache("paged", g, self.paged_groups[g].kv[j], writes, self.page_size)
    return LayerCache("state", g, self.state_groups[g].state[j], writes, 0)

  # ------------------------------------------------------------------ requests

  def has_request(self, req_id: Hashable) -> bool:
    return req_id in self._requests

  @property
  def num_free_slots(self) -> int:
    return len(self._free_slots)

  def admit(self, req_id: Hashable) -> int:
    """Gives the request a slot; its state rows start at zero."""
    if req_id in self._requests:
      raise KeyError(f"request {req_id!r} is already admitted")
    if not self._free_slots:
      raise OutOfSlots("no free request slot")
    slot = self._free_slots.pop()
    self._requests[req_id] = _Request(slot=slot, pages=[[] for _ in self.paged_groups])
    for s in self.state_groups:
      s.state[:, slot].zero_()
    return slot

  def slot_of(self, req_id: Hashable) -> int:
    return self._requests[req_id].slot

  def length_of(self, req_id: Hashable) -> int:
    return self._requests[req_id].length

  def _pages_wanted(self, g: PagedGroup, r: _Request, new_total: int) -> int:
    have = len(r.pages[g.index])
    return max(0, -(-new_total // g.page_size) - have)

  def pages_needed(self, req_id: Optional[Hashable], n_new: int) -> List[int]:
    """Pages that each paged group must hand out so that the request (None: a new one) can take
    ``n_new`` more tokens."""
    r = self._requests[req_id] if req_id is not None else _Request(slot=-1, pages=[[] for _ in self.paged_groups])
    total = r.length + r.reserved + n_new
    return [self._pages_wanted(g, r, total) for g in self.paged_groups]

  def can_append(self, req_id: Optional[Hashable], n_new: int, keep_free: int = 0) -> bool:
    if req_id is not None:
      r = self._requests[req_id]
      if r.length + r.reserved + n_new > self.max_model_len:
        return False
    need = self.pages_needed(req_id, n_new)
    return all(n + keep_free <= g.allocator.num_free for n, g in zip(need, self.paged_groups))

  def append(self, req_id: Hashable, n_new: int) -> None:
    """Makes room for ``n_new`` more tokens in every group, or raises ``OutOfPages`` and changes
    nothing."""
    r = self._requests[req_id]
    total = r.length + r.reserved + n_new
    if total > self.max_model_len:
      raise ValueError(f"request {req_id!r} would hold {total} tokens, more than max_model_len={self.max_model_len}")
    need = [self._pages_wanted(g, r, total) for g in self.paged_groups]
    for n, g in zip(need, self.paged_groups):
      if n > g.allocator.num_free:
        raise OutOfPages(f"group {g.index}: {n} pages wanted for request {req_id!r}, "
                         f"{g.allocator.num_free} of {g.num_pages} free")
    for n, g in zip(need, self.paged_groups):
      if n == 0:
        continue
      new = g.allocator.alloc(n)
      have = len(r.pages[g.index])
      r.pages[g.index].extend(new)
      g.block_table_host[r.slot, have:have + n] = new
      g._dirty.add(r.slot)
    r.reserved += n_new

  def commit(self, req_id: Hashable, n_new: int) -> None:
    """The step has run: the tokens belong to the request.  Pages that a window has passed go back."""
    r = self._requests[req_id]
    if n_new > r.reserved:
      raise ValueError("commit of more tokens than were appended")
    r.reserved -= n_new
    r.length += n_new
    for g in self.paged_groups:
      if g.spec.window is None:
        continue
      first = min(g.first_needed_page(r.length), len(r.pages[g.index]))
      dead = [i for i in range(first) if r.pages[g.index][i] != 0]
      if dead:
        g.allocator.free([r.pages[g.index][i] for i in dead])
        for i in dead:
          r.pages[g.index][i] = 0
          g.block_table_host[r.slot, i] = 0
        g._dirty.add(r.slot)

  def cancel(self, req_id: Hashable, n_new: int) -> None:
    """Undoes an ``append`` whose step did not run: the pages it took go back."""
    r = self._requests[req_id]
    if n_new > r.reserved:
      raise ValueError("cancel of more tokens than were appended")
    r.reserved -= n_new
    for g in self.paged_groups:
      keep = -(-(r.length + r.reserved) // g.page_size)
      extra = r.pages[g.index][keep:]
      if extra:
        g.allocator.free([p for p in extra if p != 0])
        del r.pages[g.index][keep:]
        g.block_table_host[r.slot, keep:keep + len(extra)] = 0
        g._dirty.add(r.slot)

  def release_request(self, req_id: Hashable) -> None:
    """Gives back everything the request holds (miniinfer/kvcache/kv_cache_manager.py:664)."""
    r = self._requests.pop(req_id)
    for g in self.paged_groups:
      live = [p for p in r.pages[g.index] if p != 0]
      if live:
        g.allocator.free(live)
      n = len(r.pages[g.index])
      if n:
        g.block_table_host[r.slot, :n] = 0
        g._dirty.add(r.slot)
    self._free_slots.append(r.slot)

  # ------------------------------------------------------------------ step metadata

  def slot_mapping(self, req_id: Hashable, group: int, start: int, n: int) -> np.ndarray:
    """For the tokens at positions ``start .. start+n``: ``page id * page_size + offset``."""
    r = self._requests[req_id]
    g = self.paged_groups[group]
    pos = np.arange(start, start + n, dtype=np.int64)
    pages = np.asarray(r.pages[group], dtype=np.int64)[pos // g.page_size]
    return (pages * g.page_size + pos % g.page_size).astype(np.int32)

  def slot_at(self, req_id: Hashable, group: int, pos: int) -> int:
    """``slot_mapping`` for the one token at position ``pos``."""
    P = self.page_size
    return self._requests[req_id].pages[group][pos // P] * P + pos % P

  def sync(self) -> None:
    for g in self.paged_groups:
      g.sync()

  def get_page_table(self, group: int = 0) -> torch.Tensor:
    return self.paged_groups[group].block_table

  # ------------------------------------------------------------------ accounting

  def free_pages(self) -> List[int]:
    return [g.allocator.num_free for g in self.paged_groups]

  def available_tokens(self) -> int:
    """Tokens that the scarcest group could still take (kv_cache_manager.py:802-817)."""
    if not self.paged_groups:
      return self.max_model_len * self.max_num_seqs
    return min(g.allocator.num_free for g in self.paged_groups) * self.page_size

  def get_stats(self) -> dict:
    return {
      "live_requests": len(self._requests),
      "free_slots": len(self._free_slots),
      "free_pages": self.free_pages(),
      "total_pages": [g.num_pages for g in self.paged_groups],
    }

  def check_invariants(self) -> None:
    """No page lost, held twice, or in a block table without an owner."""
    for g in self.paged_groups:
      owned: List[int] = []
      for r in self._requests.values():
        live = [p for p in r.pages[g.index] if p != 0]
        owned.extend(live)
        row = g.block_table_host[r.slot]
        n = len(r.pages[g.index])
        assert list(row[:n]) == r.pages[g.index], "block table differs from the request's pages"
        assert not row[n:].any(), "block table has entries past the request's pages"
      assert len(owned) == len(set(owned)), "a page is held by two requests"
      assert sorted(owned) == g.allocator.held(), "allocator and requests disagree on held pages"
      assert len(owned) + g.allocator.num_free == g.num_pages, "a page was lost"
    slots = [r.slot for r in self._requests.values()]
    assert len(slots) == len(set(slots)), "a slot is held twice"
    assert sorted(slots + self._free_slots) == list(range(self.max_num_seqs)), "a slot was lost"
