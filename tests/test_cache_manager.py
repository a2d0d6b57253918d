import random

import numpy as np
import pytest
import torch

from miniinfer_b200.cache import FixedStateSpec, KVCacheManager, OutOfPages, OutOfSlots, PageAllocator, PagedKVSpec


def make(window=None, pages=6, page=4, seqs=3, max_len=64, extra=()):
  specs = [PagedKVSpec(2, 8), PagedKVSpec(2, 8)] + ([PagedKVSpec(2, 8, window)] if window else []) + list(extra)
  return KVCacheManager(specs, page, pages, seqs, max_len, torch.float32, "cpu")


def test_allocator_never_hands_a_page_out_twice():
  a = PageAllocator(5)
  got = a.alloc(3)
  assert sorted(got) == [1, 2, 3] and a.num_free == 2
  a.free([2])
  assert a.alloc(1) == [2]                      # last freed, first reused
  with pytest.raises(AssertionError):
    a.free([4])                                 # not held
  a.free([2])
  with pytest.raises(AssertionError):
    a.free([2])                                 # freed twice
  with pytest.raises(OutOfPages):
    a.alloc(10)
  assert a.num_free == 3


def test_groups_follow_the_specs():
  m = make(window=10, extra=[FixedStateSpec((3, 2)), None])
  assert len(m.paged_groups) == 2 and len(m.state_groups) == 1
  assert m.paged_groups[0].num_layers == 2 and m.paged_groups[1].spec.window == 10
  assert m.paged_groups[0].kv.shape == (2, 7, 2, 2, 4, 8)
  assert m.layer_cache(0).group == 0 and m.layer_cache(2).group == 1
  assert m.layer_cache(3).kind == "state" and m.layer_cache(3).tensor.shape == (4, 3, 2)
  assert m.layer_cache(4).kind == "none"
  assert m.layer_cache(1, writes=False).writes is False


def test_append_commit_release_and_block_table():
  m = make()
  s = m.admit("a")
  m.append("a", 6)
  assert m.free_pages() == [4]
  row = m.paged_groups[0].block_table_host[s]
  assert list(row[:2]) != [0, 0] and not row[2:].any()
  sm = m.slot_mapping("a", 0, 0, 6)
  assert list(sm) == [row[0] * 4 + i for i in range(4)] + [row[1] * 4, row[1] * 4 + 1]
  m.commit("a", 6)
  m.append("a", 2)                               # fills the second page, no new one
  assert m.free_pages() == [4]
  m.commit("a", 2)
  m.append("a", 1)
  assert m.free_pages() == [3]
  m.cancel("a", 1)                               # a step that did not run gives its page back
  assert m.free_pages() == [4] and m.length_of("a") == 8
  m.check_invariants()
  m.release_request("a")
  assert m.free_pages() == [6] and m.num_free_slots == 3
  assert not m.paged_groups[0].block_table_host.any()
  m.check_invariants()


def test_out_of_pages_changes_nothing_and_slots_run_out():
  m = make(pages=3)
  m.admit("a"); m.admit("b")
  m.append("a", 8)
  assert not m.can_append("b", 9) and m.can_append("b", 4)
  with pytest.raises(OutOfPages):
    m.append("b", 9)
  assert m.free_pages() == [1]
  m.check_invariants()
  m.admit("c")
  with pytest.raises(OutOfSlots):
    m.admit("d")
  with pytest.raises(KeyError):
    m.admit("a")
  with pytest.raises(ValueError):
    m.append("c", 65)                            # beyond max_model_len


def test_window_gives_pages_back_as_it_passes():
  m = make(window=6, pages=8, page=4)
  m.admit("a")
  m.append("a", 20); m.commit("a", 20)
  full, win = m.paged_groups
  assert full.allocator.num_free == 3
  # the next query (position 20) sees keys 15..20: pages 0..2 (keys 0..11) are dead
  assert win.allocator.num_free == 8 - 2
  assert list(win.block_table_host[m.slot_of("a")][:5]) [:3] == [0, 0, 0]
  for _ in range(12):
    m.append("a", 1); m.commit("a", 1)
    m.check_invariants()
  assert win.allocator.num_free >= 8 - 3
  assert full.allocator.num_free == 0
  m.release_request("a")
  assert m.free_pages() == [8, 8]
  m.check_invariants()


def test_a_windowed_group_is_as_large_as_its_requests_need():
  """With the most tokens a request gets in a step known, a group that keeps a window has a pool of its own size;
  requests that grow to the longest length in steps of that many tokens (two steps in flight before the first is
  committed) never find it empty, and the group that keeps every key keeps the size it was given."""
  from miniinfer_b200.cache.manager import pages_in_flight
  full, win = PagedKVSpec(2, 8), PagedKVSpec(2, 8, window=100)
  m = KVCacheManager([full, win, full, win], page_size=16, num_pages=1000, max_num_seqs=4, max_model_len=4000,
                     dtype=torch.float32, max_step_tokens=64)
  sizes = {g.spec.window: g.num_pages for g in m.paged_groups}
  assert sizes[None] == 1000 and sizes[100] == 4 * pages_in_flight(100, 16, 64) == 4 * 16
  same = KVCacheManager([full, win], page_size=16, num_pages=1000, max_num_seqs=4, max_model_len=4000, dtype=torch.float32)
  assert [g.num_pages for g in same.paged_groups] == [1000, 1000]          # without the bound: one size for all
  rng = random.Random(3)
  for r in range(4):
    m.admit(r)
  length = {r: 0 for r in range(4)}
  pending = {r: [] for r in range(4)}
  while any(length[r] + sum(pending[r]) < 4000 for r in range(4)):
    for r in range(4):
      left = 4000 - length[r] - sum(pending[r])
      if left > 0:
        n = min(left, rng.randint(1, 64))
        m.append(r, n)                                    # raises OutOfPages if the pool were too small
        pending[r].append(n)
      if len(pending[r]) == 2 or (left <= 0 and pending[r]):    # the older of two steps in flight is done
        n = pending[r].pop(0)
        m.commit(r, n)
        length[r] += n
    m.check_invariants()
  used = [g.num_pages - g.allocator.num_free for g in m.paged_groups]
  assert used[0] == 4 * 250 and used[1] <= 4 * 16


def test_state_rows_start_at_zero():
  m = make(extra=[FixedStateSpec((5,))])
  s = m.admit("a")
  m.layer_cache(2).tensor[s] += 3
  m.release_request("a")
  s2 = m.admit("b")
  assert s2 == s and not m.layer_cache(2).tensor[s2].any()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_double_a_page(seed):
  rng = random.Random(seed)
  m = make(window=7 if seed % 2 else None, pages=10, page=4, seqs=4, max_len=40)
  live = {}
  next_id = 0
  for _ in range(400):
    op = rng.random()
    if op < 0.25 and m.num_free_slots:
      m.admit(next_id); live[next_id] = 0; next_id += 1
    elif op < 0.8 and live:
      r = rng.choice(list(live))
      n = rng.randint(1, 9)
      if live[r] + n <= 40 and m.can_append(r, n):
        m.append(r, n)
        if rng.random() < 0.1:
          m.cancel(r, n)
        else:
          m.commit(r, n); live[r] += n
      else:
        before = m.free_pages()
        if live[r] + n <= 40:
          with pytest.raises(OutOfPages):
            m.append(r, n)
          assert m.free_pages() == before
    elif live:
      r = rng.choice(list(live))
      m.release_request(r); del live[r]
    m.check_invariants()
    for r, n in live.items():
      assert m.length_of(r) == n
  for r in list(live):
    m.release_request(r)
  m.check_invariants()
  assert m.free_pages() == [10] * len(m.paged_groups)
