"""The plain implementation against the reference's own model code (stored outputs) and itself."""
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from golden.make_reference_golden import checksum, draw_weights
from tiny_configs import TINY_A, TINY_B, TINY_C

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("tag,cfg", [("A", TINY_A), ("B", TINY_B)])
def test_plain_equals_reference_model_code(tag, cfg):
  g = np.load(os.path.join(GOLDEN, f"reference_logits_{tag}.npz"))
  sd = {k[2:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("w:")}      # the weights the reference ran with
  assert abs(checksum(sd) - float(g["weight_checksum"])) <= 1e-9 * float(g["weight_checksum"])
  logits = plain.forward(sd, cfg, g["ids"].tolist())
  ref = torch.from_numpy(g["logits"])
  assert logits.shape == ref.shape
  assert (logits - ref).abs().max().item() < 2e-5
  assert torch.equal(logits.argmax(-1), ref.argmax(-1))


def test_fused_and_split_names_agree():
  sd = draw_weights(TINY_A, 5)
  fused = dict(sd)
  for i in range(TINY_A["num_hidden_layers"]):
    p = f"model.layers.{i}"
    fused[f"{p}.self_attn.qkv_proj.weight"] = torch.cat([fused.pop(f"{p}.self_attn.{n}_proj.weight") for n in "qkv"])
    fused[f"{p}.mlp.gate_up_proj.weight"] = torch.cat([fused.pop(f"{p}.mlp.{n}_proj.weight") for n in ("gate", "up")])
  ids = list(range(3, 40))
  assert torch.allclose(plain.forward(sd, TINY_A, ids), plain.forward(fused, TINY_A, ids), atol=1e-6)


def test_causality_and_window():
  sd = draw_weights(TINY_C, 7)
  ids = torch.randint(0, TINY_C["vocab_size"], (90,), generator=torch.Generator().manual_seed(0)).tolist()
  full = plain.forward(sd, TINY_C, ids)
  # a later token never changes an earlier position
  assert torch.allclose(plain.forward(sd, TINY_C, ids[:50]), full[:50], atol=1e-5)
  # the window matters: without it the late positions differ
  no_window = dict(TINY_C, use_sliding_window=False)
  other = plain.forward(sd, no_window, ids)
  assert torch.allclose(other[:40], full[:40], atol=1e-5)
  assert (other[60:] - full[60:]).abs().max() > 1e-4
  assert plain.layer_window(TINY_C, 0) is None and plain.layer_window(TINY_C, 2) == 40


def test_run_list_shared_cache_changes_result():
  sd = draw_weights(TINY_B, 9)
  ids = list(range(10, 40))
  base = plain.forward(sd, TINY_B, ids)
  same = plain.forward(sd, TINY_B, ids, run_list=[(0, None), (1, None), (2, None)])
  assert torch.equal(base, same)
  shared = plain.forward(sd, TINY_B, ids, run_list=[(0, None), (1, 0), (2, None), (1, None)])
  assert shared.shape == base.shape and (shared - base).abs().max() > 1e-4


def test_sampler_statement():
  logits = torch.tensor([0.1, 2.0, 1.9, -1.0, 0.5])
  assert plain.sample_token(logits, 0.0, 0, 1.0, 0, 0)[0] == 1
  z = plain.filter_logits(logits, 1.0, 2, 1.0)
  assert torch.isfinite(z).tolist() == [False, True, True, False, False]
  z = plain.filter_logits(logits, 1.0, 0, 0.5)
  assert torch.isfinite(z).tolist() == [False, True, True, False, False]   # 0.41 + 0.37 reaches 0.5
  z = plain.filter_logits(logits, 1.0, 0, 0.3)
  assert torch.isfinite(z).tolist() == [False, True, False, False, False]
  # the draw is a function of (seed, counter) only and follows the distribution
  counts = torch.zeros(5)
  for c in range(400):
    counts[plain.sample_token(logits, 1.0, 0, 1.0, 3, c)[0]] += 1
  p = torch.softmax(logits, -1)
  assert (counts / 400 - p).abs().max() < 0.08
  assert plain.sample_token(logits, 1.0, 0, 1.0, 3, 7)[0] == plain.sample_token(logits, 1.0, 0, 1.0, 3, 7)[0]


def test_uniform_numbers_stay_inside_the_unit_interval_in_float32():
  """The hash's extreme values must not give u = 0 or u = 1 once rounded to float32: the Gumbel noise
  -log(-log(u)) would be infinite and that vocabulary entry would win (or lose) whatever its logit."""
  for bits in (0, (1 << 64) - 1, (1 << 41) - 1, ((1 << 23) - 1) << 41):
    u = np.float32(plain.uniform_from_bits(bits))
    assert float(u) == plain.uniform_from_bits(bits)                  # exact in float32
    assert np.float32(0) < u < np.float32(1)
    noise = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
    assert np.isfinite(noise) and -3.0 < float(noise) < 17.4
