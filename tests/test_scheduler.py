"""The scheduler's decisions, with the real cache manager on the CPU and a scripted runner."""
import torch

import pytest

from miniinfer_b200.cache import KVCacheManager, PagedKVSpec
from miniinfer_b200.engine.scheduler import Request, Scheduler
from miniinfer_b200.sampling import SamplingParams


def setup(pages=8, page=4, seqs=4, budget=16, chunk=None, max_len=64, eos=()):
  cache = KVCacheManager([PagedKVSpec(1, 8)], page, pages, seqs, max_len, torch.float32, "cpu")
  return cache, Scheduler(cache, seqs, budget, chunk or budget, max_len, eos)


def req(i, n, max_tokens=4, **kw):
  return Request(req_id=i, prompt_ids=list(range(1, n + 1)), params=SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw))


def run(cache, sched, token=lambda r: 7, max_steps=500):
  """Plays the runner: reserves and commits what was scheduled, hands back scripted tokens."""
  log = []
  for _ in range(max_steps):
    if not sched.has_unfinished():
      break
    out = sched.schedule()
    assert out.items, "a step with nothing to do while requests are unfinished"
    assert sum(len(i.tokens) for i in out.items) <= sched.max_num_batched_tokens
    for it in out.items:
      assert it.tokens == it.request.all_ids()[it.request.num_computed:it.request.num_computed + len(it.tokens)]
      cache.append(it.request.req_id, len(it.tokens))
    for it in out.items:
      cache.commit(it.request.req_id, len(it.tokens))
    cache.check_invariants()
    sampled = {it.request.req_id: token(it.request) for it in out.items if it.samples}
    done = sched.update(out, sampled)
    log.append((out, done))
  assert not sched.has_unfinished()
  return log


def test_prompts_are_cut_under_the_budget_and_decode_rides_along():
  cache, s = setup(pages=16, budget=10)
  s.add(req("a", 23, max_tokens=3)); s.add(req("b", 5, max_tokens=6))
  log = run(cache, s)
  first = log[0][0]
  assert [(i.request.req_id, len(i.tokens), i.samples) for i in first.items] == [("a", 10, False)]
  assert [(i.request.req_id, len(i.tokens)) for i in log[1][0].items] == [("a", 10)]
  third = log[2][0]
  assert [(i.request.req_id, len(i.tokens), i.samples) for i in third.items] == [("a", 3, True), ("b", 5, True)]
  fourth = log[3][0]                     # both decode now, one token each, in one batch
  assert [(i.request.req_id, len(i.tokens)) for i in fourth.items] == [("a", 1), ("b", 1)]
  assert fourth.num_decode_tokens == 2 and fourth.num_prefill_tokens == 0
  a, b = s.finished
  assert (a.req_id, len(a.output_ids), a.finish_reason) == ("a", 3, "max_tokens")
  assert len(b.output_ids) == 6
  assert cache.free_pages() == [16] and cache.num_free_slots == 4


def test_chunk_size_limits_one_prompt_not_the_step():
  cache, s = setup(pages=16, budget=12, chunk=5)
  s.add(req("a", 9)); s.add(req("b", 9))
  out = s.schedule()
  assert [(i.request.req_id, len(i.tokens)) for i in out.items] == [("a", 5), ("b", 5)]


def test_admission_waits_for_slots_and_pages():
  cache, s = setup(pages=4, seqs=2, budget=32)
  for i, n in enumerate((6, 6, 6)):
    s.add(req(i, n, max_tokens=2))
  out = s.schedule()
  assert [i.request.req_id for i in out.items] == [0, 1]      # two slots
  assert [r.req_id for r in s.waiting] == [2]
  log = run(cache, s)
  assert [r.req_id for r in s.finished] == [0, 1, 2]


def test_eos_max_tokens_and_length():
  cache, s = setup(pages=16, eos=(9,), max_len=12)
  s.add(req("eos", 3, max_tokens=10)); s.add(req("ignore", 3, max_tokens=3, ignore_eos=True)); s.add(req("len", 8, max_tokens=50, ignore_eos=True))
  run(cache, s, token=lambda r: 9)
  by = {r.req_id: r for r in s.finished}
  assert by["eos"].output_ids == [9] and by["eos"].finish_reason == "eos"
  assert by["ignore"].output_ids == [9, 9, 9] and by["ignore"].finish_reason == "max_tokens"
  assert len(by["len"].output_ids) == 4 and by["len"].finish_reason == "length"


def test_refusals():
  cache, s = setup(pages=4, max_len=64)
  with pytest.raises(ValueError, match="max_model_len"):
    s.add(req("x", 64))
  with pytest.raises(ValueError, match="pages"):
    s.add(req("y", 10, max_tokens=20))         # 30 tokens > 4 pages of 4
  with pytest.raises(ValueError):
    s.add(Request(req_id="z", prompt_ids=[], params=SamplingParams()))


def test_running_out_of_pages_preempts_the_newest_and_it_resumes():
  cache, s = setup(pages=6, page=4, budget=32)
  s.add(req("old", 8, max_tokens=12)); s.add(req("new", 8, max_tokens=12))
  counters = {"old": 0, "new": 0}

  def tok(r):
    counters[r.req_id] += 1
    return 100 + len(r.output_ids)

  log = run(cache, s, token=tok)
  assert s.num_preemptions >= 1
  pre = [r.req_id for out, _ in log for r in out.preempted]
  assert pre and set(pre) == {"new"}                          # only the newest pays
  by = {r.req_id: r for r in s.finished}
  # nothing generated was thrown away, and the outputs are what an undisturbed run gives
  assert by["old"].output_ids == [100 + i for i in range(12)]
  assert by["new"].output_ids == [100 + i for i in range(12)]
  assert counters == {"old": 12, "new": 12}
  # after a preemption the request runs prompt + outputs again as a prompt
  resumed = [it for out, _ in log for it in out.items if it.request.req_id == "new" and len(it.tokens) > 8]
  assert resumed and resumed[0].tokens[:8] == list(range(1, 9)) and resumed[0].tokens[8] == 100
  assert cache.free_pages() == [6]


def test_prompts_that_block_each_other_are_resolved():
  cache, s = setup(pages=5, page=4, budget=6, seqs=2)
  s.add(req("a", 14, max_tokens=2)); s.add(req("b", 14, max_tokens=2))
  log = run(cache, s)
  assert sorted(r.req_id for r in s.finished) == ["a", "b"]
  assert all(len(r.output_ids) == 2 for r in s.finished)
