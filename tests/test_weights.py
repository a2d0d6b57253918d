import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from miniinfer_b200.config import build_model_spec, load_model_config
from miniinfer_b200.weights import WeightLoadError, load_weights, write_random_model
from tiny_configs import TINY_A, TINY_B


def _load(d, dtype=torch.float32):
  spec = build_model_spec(load_model_config(d))
  load_weights(spec, d, dtype, "cpu")
  return spec


def _rewrite(d, fn):
  path = os.path.join(d, "model.safetensors")
  sd = load_file(path)
  sd = fn(sd) or sd
  save_file({k: v.contiguous() for k, v in sd.items()}, path)


def test_random_model_folder_is_reproducible(tmp_path):
  a = write_random_model(dict(TINY_A), str(tmp_path / "a"), seed=3)
  b = write_random_model(dict(TINY_A), str(tmp_path / "b"), seed=3)
  c = write_random_model(dict(TINY_A), str(tmp_path / "c"), seed=4)
  sa, sb, sc = (load_file(os.path.join(x, "model.safetensors")) for x in (a, b, c))
  assert sorted(sa) == sorted(sb) and all(torch.equal(sa[k], sb[k]) for k in sa)
  assert not torch.equal(sa["model.embed_tokens.weight"], sc["model.embed_tokens.weight"])
  assert "lm_head.weight" not in sa                       # tied
  assert sa["model.embed_tokens.weight"].dtype == torch.bfloat16
  assert sa["model.norm.weight"].dtype == torch.float32
  assert abs(float(sa["model.norm.weight"].mean()) - 1.0) < 0.1
  assert abs(float(sa["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
  cfg = json.load(open(os.path.join(a, "config.json")))
  assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["head_dim"] == TINY_A["head_dim"]


def test_kept_dtypes_and_fused_rows(tmp_path):
  d = write_random_model(dict(TINY_B), str(tmp_path / "m"), seed=1)
  sd = load_file(os.path.join(d, "model.safetensors"))
  spec = _load(d, torch.bfloat16)
  m = spec.blocks[1].mixer
  assert m.qkv.dtype == torch.bfloat16 and m.q_norm.dtype == torch.float32
  nh, nkv, hd = TINY_B["num_attention_heads"], TINY_B["num_key_value_heads"], TINY_B["head_dim"]
  p = "model.layers.1.self_attn"
  assert torch.equal(m.qkv[:nh * hd], sd[f"{p}.q_proj.weight"])
  assert torch.equal(m.qkv[nh * hd:(nh + nkv) * hd], sd[f"{p}.k_proj.weight"])
  assert torch.equal(m.qkv[(nh + nkv) * hd:], sd[f"{p}.v_proj.weight"])
  f = spec.blocks[2].ffn
  I = TINY_B["intermediate_size"]
  assert torch.equal(f.gate_up[:I], sd["model.layers.2.mlp.gate_proj.weight"])
  assert torch.equal(f.gate_up[I:], sd["model.layers.2.mlp.up_proj.weight"])
  assert spec.lm_head.table() is spec.lm_head.weight
  spec32 = _load(d, torch.float32)
  assert spec32.blocks[0].mixer.o.dtype == torch.float32
  assert torch.equal(spec32.blocks[0].mixer.o, sd["model.layers.0.self_attn.o_proj.weight"].float())


def test_fused_names_and_missing_prefix_are_accepted(tmp_path):
  d = write_random_model(dict(TINY_A), str(tmp_path / "m"), seed=1)
  ref = _load(d)

  def fuse(sd):
    out = {}
    for k, v in sd.items():
      out[k[len("model."):] if k.startswith("model.") else k] = v
    for i in range(TINY_A["num_hidden_layers"]):
      p = f"layers.{i}"
      out[f"{p}.self_attn.qkv_proj.weight"] = torch.cat([out.pop(f"{p}.self_attn.{n}_proj.weight") for n in "qkv"])
      out[f"{p}.mlp.gate_up_proj.weight"] = torch.cat([out.pop(f"{p}.mlp.{n}_proj.weight") for n in ("gate", "up")])
    return out

  _rewrite(d, fuse)
  got = _load(d)
  assert torch.equal(got.blocks[1].mixer.qkv, ref.blocks[1].mixer.qkv)
  assert torch.equal(got.blocks[0].ffn.gate_up, ref.blocks[0].ffn.gate_up)
  assert torch.equal(got.embedding.weight, ref.embedding.weight)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
  d = write_random_model(dict(TINY_B), str(tmp_path / "m"), seed=1)

  def damage(sd):
    del sd["model.layers.0.self_attn.k_proj.weight"]
    del sd["model.norm.weight"]
    sd["model.layers.9.extra.weight"] = torch.zeros(3)
    sd["model.layers.1.mlp.down_proj.weight"] = torch.zeros(5, 7)
    sd["lm_head.weight"] = sd["lm_head.weight"][:-1]

  _rewrite(d, damage)
  with pytest.raises(WeightLoadError) as e:
    _load(d)
  err = e.value
  assert err.missing == ["model.layers.0.self_attn.k_proj.weight", "model.norm.weight"]
  assert err.unexpected == ["model.layers.9.extra.weight"]
  assert len(err.wrong_shape) == 2
  text = str(err)
  for word in ("k_proj", "model.norm.weight", "layers.9.extra", "down_proj", "[5, 7]", "lm_head.weight", "missing",
               "unexpected", "wrong shapes"):
    assert word in text, word


def test_tied_head_rules(tmp_path):
  d = write_random_model(dict(TINY_A), str(tmp_path / "m"), seed=1)
  _rewrite(d, lambda sd: dict(sd, **{"lm_head.weight": sd["model.embed_tokens.weight"].clone()}))
  spec = _load(d)                                           # equal copy: accepted, the table is shared
  assert spec.lm_head.table() is spec.embedding.weight
  _rewrite(d, lambda sd: dict(sd, **{"lm_head.weight": sd["lm_head.weight"] + 1}))
  with pytest.raises(WeightLoadError, match="ties"):
    _load(d)
  d2 = write_random_model(dict(TINY_B), str(tmp_path / "u"), seed=1)
  _rewrite(d2, lambda sd: {k: v for k, v in sd.items() if k != "lm_head.weight"})
  with pytest.raises(WeightLoadError, match="lm_head.weight"):
    _load(d2)


def test_no_file_and_wrong_kind(tmp_path):
  d = write_random_model(dict(TINY_A), str(tmp_path / "m"), seed=1)
  os.remove(os.path.join(d, "model.safetensors"))
  with pytest.raises(FileNotFoundError):
    _load(d)
  d = write_random_model(dict(TINY_A), str(tmp_path / "n"), seed=1)
  _rewrite(d, lambda sd: dict(sd, **{"model.norm.weight": torch.ones(TINY_A["hidden_size"], dtype=torch.int32)}))
  with pytest.raises(WeightLoadError, match="floating"):
    _load(d)
