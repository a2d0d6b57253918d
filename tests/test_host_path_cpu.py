"""The host side of the engine - cache manager, step metadata, scheduler, replay program - run on the
CPU with the kernels replaced by their PyTorch statements (tests/torch_ops.py), against the plain
implementation.  The CUDA kernels themselves are tested by the ``gpu`` tests."""
import io
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_cases as rc
from tiny_configs import ALL

LENGTHS = {"A": (5, 17, 33, 100, 64, 41), "B": (1, 9, 40, 71, 130, 65), "C": (90, 33, 150, 64, 7)}


def make_runner(model_dir, page_size, max_tokens):
  from miniinfer_b200.engine.replay import TraceRunner
  return TraceRunner(model_dir, "float32", max_tokens, device="cpu", page_size=page_size)


@pytest.mark.parametrize("tag,page", [("A", 16), ("B", 8), ("C", 8)])
def test_every_cut_gives_the_plain_logits(cpu_kernels, model_dirs, tag, page):
  d = model_dirs(tag)
  reqs = rc.make_requests(ALL[tag]["vocab_size"], LENGTHS[tag], seed=5)
  ref = rc.reference_logits(d, reqs)
  budget = 4 * rc.round_up(max(LENGTHS[tag]), page)
  for name, trace in (("whole", rc.whole(reqs)), ("tail", rc.tail_one_by_one(reqs)), ("portions", rc.portions(reqs)),
                      ("mixed", rc.mixed(reqs, budget // 2, seed=1, granule=page)),
                      ("preempted", rc.mixed(reqs, budget // 2, seed=2, granule=page, preempt=True))):
    runner = make_runner(d, page, budget if name not in ("mixed", "preempted") else budget // 2)
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, 2e-5, f"{tag}/{name}")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


def test_trace_program_reads_steps_and_writes_files(cpu_kernels, model_dirs, tmp_path):
  from miniinfer_b200.engine import replay
  d = model_dirs("A")
  reqs = rc.make_requests(256, (20, 9), seed=2)
  trace = rc.mixed(reqs, 128, seed=3)
  trace.append({"step": 99, "entries": [], "end": []})
  out = io.StringIO()
  code = replay.main(["--model", d, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128",
                      "--device", "cpu"], stdin=io.StringIO("\n".join(json.dumps(r) for r in trace) + "\n"), stdout=out)
  assert code == 0
  assert out.getvalue().split("\n")[:-1] == [f"done {r['step']}" for r in trace]
  outputs = {}
  for r in trace:
    path = tmp_path / "o" / f"{r['step']}.f32"
    wanted = sum(len(e["want"]) for e in r["entries"])
    assert path.exists() == (wanted > 0)
    if wanted:
      outputs[r["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, 256)
  rc.compare(rc.collect(trace, outputs), rc.reference_logits(d, reqs), 2e-5, "trace program")


def test_generate_equals_plain_generation(cpu_kernels, model_dirs):
  from miniinfer_b200 import LLMEngine, SamplingParams
  d = model_dirs("B")
  eng = LLMEngine(d, dtype="float32", device="cpu", page_size=8, num_pages=30, max_num_seqs=4, max_model_len=128,
                  max_num_batched_tokens=13)
  prompts = list(rc.make_requests(512, (1, 9, 40, 71), seed=0).values())
  w, c = plain.read_weights(d), plain.read_config(d)
  outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
  for p, o in zip(prompts, outs):
    assert o["token_ids"] == plain.generate(w, c, p, 6) and o["finish_reason"] == "max_tokens"
  sp = [SamplingParams(temperature=0.8, max_tokens=5, seed=i, top_k=(0, 20)[i % 2], top_p=(1.0, 0.9)[i // 2]) for i in range(4)]
  outs = eng.generate(prompts, sp)
  for p, o, s in zip(prompts, outs, sp):
    assert o["token_ids"] == plain.generate(w, c, p, 5, temperature=0.8, top_k=s.top_k, top_p=s.top_p, seed=s.seed)
  eng.cache.check_invariants()
  assert eng.cache.free_pages() == [30]


def test_generation_survives_preemption(cpu_kernels, model_dirs):
  from miniinfer_b200 import LLMEngine, SamplingParams
  d = model_dirs("A")
  prompts = list(rc.make_requests(256, (20, 24, 18), seed=4).values())
  w, c = plain.read_weights(d), plain.read_config(d)
  eng = LLMEngine(d, dtype="float32", device="cpu", page_size=16, num_pages=5, max_num_seqs=3, max_model_len=64,
                  max_num_batched_tokens=32)
  outs = eng.generate(prompts, SamplingParams(temperature=0.7, max_tokens=20, seed=9))
  assert eng.scheduler.num_preemptions >= 1
  for p, o in zip(prompts, outs):
    assert o["token_ids"] == plain.generate(w, c, p, 20, temperature=0.7, seed=9)
  assert eng.cache.free_pages() == [5]


def test_run_list_and_shared_cache(cpu_kernels, model_dirs):
  """A layer named twice and a layer that reads another layer's cache, against the plain implementation."""
  from miniinfer_b200.cache import KVCacheManager
  from miniinfer_b200.config import build_model_spec, load_model_config
  from miniinfer_b200.engine import ModelRunner, StepItem
  from miniinfer_b200.models import LayerRun
  from miniinfer_b200.weights import load_weights
  d = model_dirs("B")
  spec = build_model_spec(load_model_config(d))
  spec.run_list = [LayerRun(0), LayerRun(1, cache_of=0), LayerRun(2), LayerRun(1)]
  spec.__post_init__()
  load_weights(spec, d, torch.float32, "cpu")
  assert [s is not None for s in spec.cache_layer_specs()] == [True, False, True, True]
  cache = KVCacheManager(spec.cache_layer_specs(), 8, 20, 2, 128, torch.float32, "cpu")
  runner = ModelRunner(spec, cache, torch.float32, "cpu")
  ids = rc.make_requests(512, (45,), seed=6)["r0"]
  cache.admit("x")
  got = torch.cat([runner.step([StepItem("x", ids[:30], range(30))]).clone(),
                   runner.step([StepItem("x", ids[30:37], range(7))]).clone()] +
                  [runner.step([StepItem("x", [t], [0])]).clone() for t in ids[37:]])
  ref = plain.forward(plain.read_weights(d), plain.read_config(d), ids,
                      run_list=[(0, None), (1, 0), (2, None), (1, None)])
  assert (got - ref).abs().max() < 2e-5


def test_step_refuses_bad_input(cpu_kernels, model_dirs):
  from miniinfer_b200.cache import OutOfPages
  from miniinfer_b200.engine import StepItem
  r = make_runner(model_dirs("A"), 16, 64)
  r.cache.admit("a"); r.cache.admit("b")
  with pytest.raises(ValueError, match="vocabulary"):
    r.runner.step([StepItem("a", [256], [0])])
  with pytest.raises(ValueError, match="twice"):
    r.runner.step([StepItem("a", [1], []), StepItem("a", [2], [])])
  with pytest.raises(ValueError, match="wanted place"):
    r.runner.step([StepItem("a", [1, 2], [2])])
  with pytest.raises(OutOfPages):
    r.runner.step([StepItem("a", list(range(40)), []), StepItem("b", list(range(40)), [])])
  assert r.cache.length_of("a") == 0 and r.cache.free_pages() == [4]
  r.cache.check_invariants()


def test_decode_description_written_in_place_equals_the_general_one(cpu_kernels, model_dirs):
  """The decode-only steps of a captured graph write their description straight into the staging
  array; word for word it must be what the general description, padded, gives."""
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.engine.runner import _DecodeGraph
  from miniinfer_b200.sampling import Sampler, SamplingParams
  r = make_runner(model_dirs("A"), 16, 256)
  run = r.runner
  lengths = {"a": 5, "b": 33, "c": 16}
  for rid, n in lengths.items():
    r.cache.admit(rid)
    run.step([StepItem(rid, list(range(1, n + 1)), [])])
  g = _DecodeGraph(4, torch.device("cpu"))
  params = [SamplingParams(temperature=0.7, top_k=5, top_p=0.9), SamplingParams(), SamplingParams(temperature=1.3)]
  for step, rids in enumerate((["a", "b", "c"], ["c", "a"], ["b"], ["b", "c", "a"])):
    items = [StepItem(rid, [7 + step + i], (0,)) for i, rid in enumerate(rids)]
    packed = Sampler.pack(params[:len(rids)], [11, 2 ** 40 + 5, 3][:len(rids)], [step] * len(rids))
    starts = run._check_and_reserve(items)
    general = run._padded(run._describe(items, starts, packed), 4, Sampler.PAD_ROWS)
    if g.template is None:
      run._decode_layout(g, run._describe(items, starts, packed), Sampler.PAD_ROWS)
    want = np.zeros(g.total, dtype=np.int32)
    for k, v in general.items():
      o, n = g.offsets[k]
      assert n == len(v)
      want[o:o + n] = v
    start_np = np.zeros(4, dtype=np.int32)
    start_np[:len(starts)] = starts
    run._fill_decode(g, items, starts, packed, np.ones(4, dtype=np.int32), start_np)
    assert np.array_equal(g.meta.host.numpy()[:g.total], want), (step, rids)
    run._finish(items, True)
  for rid in lengths:
    r.cache.release_request(rid)
  r.cache.check_invariants()


def test_stream_generate_add_requests_and_submit_request(cpu_kernels, model_dirs):
  """The other entry points of the reference's engine: tokens streamed one by one (with requests
  that are handed in meanwhile from another thread), several requests added at once."""
  import threading
  from miniinfer_b200 import LLMEngine, RequestOutput, SamplingParams
  d = model_dirs("A", "float32")
  w, c = plain.read_weights(d), plain.read_config(d)
  prompts = [[5, 17, 3, 200, 9], list(range(40, 60)), [7]]
  eng = LLMEngine(d, dtype="float32", device="cpu", page_size=16, num_pages=24, max_num_seqs=4, max_model_len=128)
  sp = SamplingParams(temperature=0.0, max_tokens=6)
  late = {}
  seen = {}
  for out in eng.stream_generate(prompts[:2], sp):
    assert isinstance(out, RequestOutput)
    seen.setdefault(out.request_id, []).append(out.token_id)
    assert out.output_token_ids == seen[out.request_id]
    assert out.finished == (len(seen[out.request_id]) == 6) and (out.finish_reason == "max_tokens") == out.finished
    if not late:                       # from another thread, while the generator runs
      t = threading.Thread(target=lambda: late.setdefault("id", eng.submit_request(prompts[2], sp)))
      t.start(); t.join()
  assert sorted(seen) == [0, 1, late["id"]]
  for rid, p in zip((0, 1, late["id"]), prompts):
    assert seen[rid] == plain.generate(w, c, p, 6)
  ids = eng.add_requests(prompts, [sp] * 3)
  assert len(set(ids)) == 3 and not eng.is_finished()
  done = {}
  while not eng.is_finished():
    for o in eng.step():
      done[o["request_id"]] = o["token_ids"]
  assert [done[i] for i in ids] == [plain.generate(w, c, p, 6) for p in prompts]
  with pytest.raises(ValueError, match="mismatch"):
    eng.add_requests(prompts, [sp])
  assert eng.cache.free_pages() == [24]


def test_a_failing_step_leaves_a_structured_record(cpu_kernels, model_dirs, caplog):
  """When a step raises, the engine logs what it knew - queues, running requests, cache occupancy - and the
  error goes on unchanged; the dump itself never raises, whatever it is given."""
  import logging
  from miniinfer_b200 import LLMEngine, SamplingParams
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.utils import describe_step_failure, dump_step_failure, tensor_summary
  d = model_dirs("A", "float32")
  eng = LLMEngine(d, dtype="float32", device="cpu", page_size=16, num_pages=8, max_num_seqs=2, max_model_len=64)
  eng.add_request([5, 6, 7], SamplingParams(temperature=0.0, max_tokens=4))
  eng.step()

  def broken(*a, **k):
    raise ops.KernelError("a kernel refused its arguments (made up for this test)")

  logging.getLogger("miniinfer_b200").propagate = True
  with caplog.at_level(logging.ERROR, logger="miniinfer_b200"):
    import unittest.mock as mock
    with mock.patch.object(ops, "add_rmsnorm", broken):
      with pytest.raises(ops.KernelError, match="made up"):
        eng.step()
  text = caplog.text
  assert "a step failed" in text and "made up for this test" in text
  assert "running" in text and "'prompt': 3" in text and "free_pages" in text
  rec = describe_step_failure(RuntimeError("x"), scheduler=eng.scheduler, cache=eng.cache, runner=eng.runner)
  assert rec["error"] == "RuntimeError: x" and rec["cache"]["live_requests"] == 1
  assert dump_step_failure(RuntimeError("y"), scheduler=object(), cache=object(), runner=object(), items=[object()])["error"] == "RuntimeError: y"
  assert "shape=(2, 3)" in tensor_summary(torch.zeros(2, 3)) and tensor_summary(None) == "None"


def test_stage_ranges_and_the_profile_option(cpu_kernels, model_dirs, tmp_path):
  """Stage ranges are off by default and cost nothing; with --profile the command line writes the ranges'
  host times and the kernels' device times to a file."""
  import main as cli
  from miniinfer_b200.utils import stage, stages_enabled
  assert not stages_enabled()
  with stage("nothing"):
    pass
  out = tmp_path / "profile.txt"
  code = cli.main(["--model", model_dirs("A", "float32"), "--prompt-ids", "5,17,3", "--max-tokens", "4", "--temperature", "0",
                   "--dtype", "float32", "--device", "cpu", "--max-model-len", "64", "--page-size", "16", "--profile", str(out)])
  assert code == 0
  text = out.read_text()
  for name in ("stage::schedule", "stage::describe+launch", "stage::wait+update"):
    assert name in text
  assert not stages_enabled()


def test_the_attention_work_lists_of_a_step():
  """What the attention mixer declares for a step: the items that bring one token, and the tiles of 64 and of 128
  new tokens of the items that bring more (the 128-token tiles are the works of the tcgen05 prefill kernel where a
  block takes one head).  The keys - what the launches depend on - are the lists' lengths and the class of the
  longest decode context."""
  from miniinfer_b200.parts.base import HostStep
  from miniinfer_b200.parts.mixer import DecodeItems, PrefillTiles, PrefillWideTiles
  q_len = np.array([1, 130, 64, 2, 1], dtype=np.int32)
  start = np.array([99, 0, 500, 7, 1500], dtype=np.int32)
  step = HostStep(q_len, start, 4096)
  assert DecodeItems().build(step).tolist() == [0, 4]
  assert DecodeItems().key(step) == (2, 2048)            # the longest decode context, 1501 tokens, in classes of 1024
  tiles = PrefillTiles().build(step).reshape(-1, 2).tolist()
  assert tiles == [[1, 0], [1, 64], [1, 128], [2, 0], [3, 0]]
  assert PrefillTiles().key(step) == (5,)
  wide = PrefillWideTiles().build(step).reshape(-1, 2).tolist()
  assert wide == [[1, 0], [1, 128], [2, 0], [3, 0]]
  assert PrefillWideTiles().key(step) == (4,)
  assert PrefillTiles.name != PrefillWideTiles.name
  # a step of decode tokens only has neither kind of tile
  only = HostStep(np.ones(3, dtype=np.int32), np.array([5, 6, 7], dtype=np.int32), 4096)
  assert PrefillTiles().build(only).size == 0 and PrefillWideTiles().key(only) == (0,)
