import json
import os

import pytest
import torch

from miniinfer_b200.config import (ConfigError, EngineConfig, Qwen3Config, build_model_spec, known_architectures,
                                   load_model_config, lookup, register_model, unregister_model)
from miniinfer_b200.config.model_config import ModelConfig
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_every_key_is_read(tmp_path):
  d = dict(TINY_B, eos_token_id=[5, 7], bos_token_id=1, torch_dtype="bfloat16", some_future_key=3)
  (tmp_path / "config.json").write_text(json.dumps(d))
  cfg = load_model_config(str(tmp_path))
  assert isinstance(cfg, Qwen3Config)
  for k in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
            "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps", "max_position_embeddings",
            "tie_word_embeddings"):
    assert getattr(cfg, k) == d[k], k
  assert cfg.eos_ids() == [5, 7] and cfg.extra == {"some_future_key": 3}
  assert cfg.to_dict()["some_future_key"] == 3


def test_defaults_follow_the_architecture():
  cfg = Qwen3Config.from_dict({"architectures": ["Qwen3ForCausalLM"]})
  assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.head_dim, cfg.vocab_size) == (1024, 28, 128, 151936)
  cfg = Qwen3Config.from_dict({"hidden_size": 96, "num_attention_heads": 4, "head_dim": None, "num_key_value_heads": None})
  assert cfg.head_dim == 24 and cfg.num_key_value_heads == 4


@pytest.mark.parametrize("bad,word", [
  ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
  ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
  ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"head_dim": 15}, "head_dim"),
  ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
  ({"layer_types": ["full_attention"]}, "layer_types"), ({"vocab_size": 0}, "vocab_size")])
def test_unsupported_values_name_the_key(bad, word):
  with pytest.raises(ConfigError, match=word):
    Qwen3Config.from_dict(dict(TINY_A, **bad))


def test_window_per_layer():
  cfg = Qwen3Config.from_dict(TINY_C)
  assert [cfg.window_of_layer(i) for i in range(4)] == [None, None, 40, 40]
  cfg = Qwen3Config.from_dict(dict(TINY_C, layer_types=["sliding_attention", "full_attention"] * 2))
  assert [cfg.window_of_layer(i) for i in range(4)] == [40, None, 40, None]
  assert Qwen3Config.from_dict(TINY_A).window_of_layer(1) is None


def test_registry():
  assert "Qwen3ForCausalLM" in known_architectures()
  with pytest.raises(ConfigError, match="NoSuchLM.*known.*Qwen3ForCausalLM"):
    lookup("NoSuchLM")
  from miniinfer_b200.config.registry import architecture_of
  with pytest.raises(ConfigError, match="architectures"):
    architecture_of({})

  @register_model("ToyLM", ModelConfig)
  def build(cfg):
    return "toy"

  try:
    assert lookup("ToyLM")[1](None) == "toy"
    with pytest.raises(ValueError):
      register_model("ToyLM", ModelConfig)(build)
  finally:
    unregister_model("ToyLM")


def test_spec_is_built_from_the_configuration_alone():
  for d in (TINY_A, TINY_B, TINY_C):
    cfg = Qwen3Config.from_dict(d)
    spec = build_model_spec(cfg)
    assert len(spec.blocks) == d["num_hidden_layers"]
    m = spec.blocks[-1].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim) == (d["num_attention_heads"], d["num_key_value_heads"], d["head_dim"])
    assert m.scale == d["head_dim"] ** -0.5 and m.qk_norm_eps == d["rms_norm_eps"]
    assert m.position.theta == d["rope_theta"]
    assert spec.blocks[0].ffn.intermediate_size == d["intermediate_size"]
    assert (spec.lm_head.tied_to is not None) == d["tie_word_embeddings"]
  spec = build_model_spec(Qwen3Config.from_dict(TINY_C))
  assert [b.mixer.window for b in spec.blocks] == [None, None, 40, 40]
  assert len(set(spec.cache_layer_specs())) == 2


def test_engine_config():
  c = EngineConfig.from_kwargs("/m", dtype="float32", max_model_len=99, page_size=8)
  assert c.dtype == torch.float32 and c.max_context_len == 99 and c.max_model_len == 99
  assert c.chunked_prefill_size == c.max_num_batched_tokens
  with pytest.raises(TypeError, match="max_modle_len"):
    EngineConfig.from_kwargs("/m", max_modle_len=5)
  with pytest.raises(ValueError, match="dtype"):
    EngineConfig.from_kwargs("/m", dtype="float16")
  with pytest.raises(TypeError):
    EngineConfig.from_kwargs("/m", max_model_len=5, max_context_len=6)


def test_sizes_the_kernels_cannot_take_are_refused_when_the_engine_is_built(tmp_path):
  """head_dim 6 is a valid Qwen3 configuration for config.json, but no attention kernel takes it; a
  hidden size of 36 cannot be read 16 bytes at a time in bfloat16.  Both are refused with the
  offending size in the message when the step function is built, before any step."""
  import torch
  from miniinfer_b200.cache import KVCacheManager
  from miniinfer_b200.config import build_model_spec
  from miniinfer_b200.config.model_config import Qwen3Config
  from miniinfer_b200.engine import ModelRunner
  from tiny_configs import TINY_A

  def runner(cfg, dtype):
    spec = build_model_spec(Qwen3Config.from_dict(cfg))
    cache = KVCacheManager(spec.cache_layer_specs(), 16, 4, 2, 64, dtype, "cpu")
    return ModelRunner(spec, cache, dtype, "cpu")

  with pytest.raises(ValueError, match="head_dim=6"):
    runner(dict(TINY_A, head_dim=6), torch.float32)
  with pytest.raises(ValueError, match="head_dim=260"):
    runner(dict(TINY_A, head_dim=260), torch.bfloat16)
  with pytest.raises(ValueError, match="hidden_size=36"):
    runner(dict(TINY_A, hidden_size=36), torch.bfloat16)
  with pytest.raises(ValueError, match="intermediate_size=100"):
    runner(dict(TINY_A, intermediate_size=100), torch.bfloat16)
  runner(dict(TINY_A, hidden_size=36, intermediate_size=100), torch.float32)      # the 32-bit kernels take both
  runner(dict(TINY_A, head_dim=20), torch.bfloat16)                               # a head size of 20 runs on the general kernel
