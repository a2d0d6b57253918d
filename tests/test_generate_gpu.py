"""Generation through the Python entry point and the command line on the GPU."""
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
import replay_cases as rc
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine(d, dtype, **kw):
  from miniinfer_b200 import LLMEngine
  return LLMEngine(d, dtype=dtype, device=DEV, **kw)


def test_greedy_generation_float32_equals_plain(model_dirs):
  from miniinfer_b200 import SamplingParams
  for tag, page, lens in (("A", 16, (5, 17, 33)), ("B", 8, (1, 9, 40, 71))):
    d = model_dirs(tag)
    eng = engine(d, "float32", page_size=page, num_pages=40, max_num_seqs=4, max_model_len=128, max_num_batched_tokens=13)
    prompts = list(rc.make_requests(eng.model_config.vocab_size, lens, seed=0).values())
    w, c = plain.read_weights(d), plain.read_config(d)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    for p, o in zip(prompts, outs):
      assert o["token_ids"] == plain.generate(w, c, p, 8)
    assert eng.cache.free_pages() == [40]


def test_sampling_float32_equals_plain_and_ignores_batching(model_dirs):
  from miniinfer_b200 import SamplingParams
  d = model_dirs("B")
  prompts = list(rc.make_requests(512, (1, 9, 40, 71), seed=0).values())
  w, c = plain.read_weights(d), plain.read_config(d)
  sp = [SamplingParams(temperature=0.8, max_tokens=12, seed=100 + i, top_k=(0, 20)[i % 2], top_p=(1.0, 0.9)[i // 2]) for i in range(4)]
  together = engine(d, "float32", page_size=8, num_pages=40, max_num_seqs=4, max_model_len=128,
                    max_num_batched_tokens=13).generate(prompts, sp)
  alone = engine(d, "float32", page_size=8, num_pages=40, max_num_seqs=1, max_model_len=128)
  for p, s, o in zip(prompts, sp, together):
    assert alone.generate([p], s)[0]["token_ids"] == o["token_ids"]
    want = plain.generate(w, c, p, 12, temperature=0.8, top_k=s.top_k, top_p=s.top_p, seed=s.seed)
    assert o["token_ids"] == want


def test_greedy_generation_bfloat16_follows_plain_where_the_choice_is_clear(model_dirs):
  from miniinfer_b200 import SamplingParams
  d = model_dirs("A")
  eng = engine(d, "bfloat16", page_size=16, num_pages=40, max_num_seqs=4, max_model_len=128)
  prompts = list(rc.make_requests(256, (5, 17, 33), seed=0).values())
  w, c = plain.read_weights(d), plain.read_config(d)
  outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
  for p, o in zip(prompts, outs):
    ids = list(p)
    for tok in o["token_ids"]:
      logits = plain.forward(w, c, ids)[-1]
      top2 = torch.topk(logits, 2).values
      if top2[0] - top2[1] > 0.05 * logits.abs().max():
        assert tok == int(logits.argmax())
      ids.append(tok)          # follow the engine's own choice
    assert len(o["token_ids"]) == 8


def test_decode_with_the_norm_and_the_residual_add_fused_to_the_products(model_dirs, monkeypatch):
  """The optional decode path of six launches per layer (MINIINFER_B200_FUSE_FEW_ROWS=1): every token is the
  plain implementation's greedy choice or within the bfloat16 bound of it, for a model with head size 64
  (TMA and cluster attention kernels) and one with head size 16."""
  from miniinfer_b200 import SamplingParams
  monkeypatch.setenv("MINIINFER_B200_FUSE_FEW_ROWS", "1")
  for tag, page, bound in (("D", 64, 0.0103), ("A", 16, 0.0072)):
    d = model_dirs(tag)
    eng = engine(d, "bfloat16", page_size=page, num_pages=40, max_num_seqs=4, max_model_len=256)
    prompts = list(rc.make_requests(eng.model_config.vocab_size, (70, 5, 33), seed=3).values())
    w, c = plain.read_weights(d), plain.read_config(d)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    launches = eng.runner.last_launches
    exact = sum(plain.check_greedy_tokens(w, c, p, o["token_ids"], margin=2 * bound) for p, o in zip(prompts, outs))
    assert exact >= 30
    if DEV != "cpu":
      L = eng.model_config.num_hidden_layers
      assert launches <= 6 * L + 5, launches        # the last step was a decode step: six launches per layer


def test_preemption_on_the_gpu_keeps_the_tokens(model_dirs):
  from miniinfer_b200 import SamplingParams
  d = model_dirs("A")
  prompts = list(rc.make_requests(256, (20, 24, 18), seed=4).values())
  w, c = plain.read_weights(d), plain.read_config(d)
  eng = engine(d, "float32", page_size=16, num_pages=5, max_num_seqs=3, max_model_len=64, max_num_batched_tokens=32)
  outs = eng.generate(prompts, SamplingParams(temperature=0.7, max_tokens=20, seed=9))
  assert eng.scheduler.num_preemptions >= 1
  for p, o in zip(prompts, outs):
    assert o["token_ids"] == plain.generate(w, c, p, 20, temperature=0.7, seed=9)


def test_overlap_gives_the_same_tokens_also_when_a_request_ends_with_a_stop_token(model_dirs):
  """With enable_overlap a decode step is launched before the tokens of the step before are read; a
  request that ends with a stop token is then run once more and that token dropped.  Same tokens,
  same finish reasons, every page back."""
  from miniinfer_b200 import SamplingParams
  d = model_dirs("B")
  prompts = list(rc.make_requests(512, (9, 40, 71, 3), seed=2).values())
  sp = [SamplingParams(temperature=0.8, max_tokens=(16, 24, 9, 30)[i], seed=50 + i) for i in range(4)]
  kw = dict(page_size=8, num_pages=60, max_num_seqs=4, max_model_len=160)
  plain_loop, overlapped = engine(d, "float32", enable_overlap=False, **kw), engine(d, "float32", enable_overlap=True, **kw)
  first = plain_loop.generate(prompts, sp)
  stop = first[1]["token_ids"][6]              # becomes a stop token: at least the second request ends early
  for e in (plain_loop, overlapped):
    e.scheduler.eos_ids = {stop}
  a, b = plain_loop.generate(prompts, sp), overlapped.generate(prompts, sp)
  assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]
  assert [o["finish_reason"] for o in a] == [o["finish_reason"] for o in b]
  assert a[1]["finish_reason"] == "eos" and len(a[1]["token_ids"]) <= 7
  assert overlapped.cache.free_pages() == [60] and plain_loop.cache.free_pages() == [60]
  overlapped.cache.check_invariants()
  assert overlapped.runner.num_graphs() >= 1


def test_command_line(model_dirs):
  d = model_dirs("A")
  proc = subprocess.run([sys.executable, os.path.join(ROOT, "main.py"), "--model", d, "--prompt-ids", "5,17,3,200",
                         "--prompt-len", "9", "--max-tokens", "6", "--temperature", "0", "--dtype", "float32",
                         "--max-model-len", "64", "--page-size", "16"], capture_output=True, text=True, timeout=900)
  assert proc.returncode == 0, proc.stderr[-3000:]
  assert proc.stdout.count("[Token count]: 6") == 2
  w, c = plain.read_weights(d), plain.read_config(d)
  assert str(plain.generate(w, c, [5, 17, 3, 200], 6)) in proc.stdout


def test_smoke_entry():
  import __graft_entry__
  __graft_entry__.smoke()
