"""A mixer with state of its own, defined here, registered, built and stepped without a change to
the package: the cache manager gives it a fixed-size state per request, the step function hands it
the batch, and a whole architecture around it is registered by name."""
import json
from dataclasses import dataclass
from typing import Dict, Optional

import pytest
import torch

from gpu_helpers import DEV

pytestmark = pytest.mark.gpu


def define_toy():
  from miniinfer_b200.cache import FixedStateSpec
  from miniinfer_b200.config import register_model
  from miniinfer_b200.config.model_config import ModelConfig
  from miniinfer_b200.models import LayerRun, ModelSpec
  from miniinfer_b200.parts import (MIXERS, LMHead, Mixer, ParamSpec, PreNormBlock, RMSNorm, SwiGLUFeedForward,
                                    TokenEmbedding, make, register_mixer, whole)

  if "toy_decay" not in MIXERS:
    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
      """out_t = W (s_t), s_t = decay * s_{t-1} + x_t: a running sum per request, kept in a state slot."""

      reads_step_on_host = True      # forward walks the items of the step in Python

      def __init__(self, name, hidden_size, decay):
        super().__init__(name)
        self.hidden_size, self.decay = hidden_size, decay

      def cache_spec(self):
        return FixedStateSpec((self.hidden_size,), "float32")

      def param_specs(self) -> Dict[str, ParamSpec]:
        H = self.hidden_size
        return {"w": ParamSpec((H, H), "matrix", [whole(f"{self.name}.w", (H, H))])}

      def forward(self, x, ctx, cache):
        assert cache.kind == "state"
        out = torch.empty_like(x)
        for b, (q0, n) in enumerate(zip(ctx.host["q_start"], ctx.host["q_len"])):
          slot = ctx.host["seq_slot"][b]
          s = cache.tensor[slot]
          for t in range(q0, q0 + n):
            s.mul_(self.decay).add_(x[t].float())
            out[t] = (s.to(x.dtype) @ self.w.t())
        return out

  @dataclass
  class ToyConfig(ModelConfig):
    hidden_size: int = 32
    num_hidden_layers: int = 2
    decay: float = 0.5
    rms_norm_eps: float = 1e-5
    intermediate_size: int = 48

  from miniinfer_b200.config.registry import _MODELS
  if "ToyDecayLM" not in _MODELS:
    @register_model("ToyDecayLM", ToyConfig)
    def build(cfg):
      H = cfg.hidden_size
      emb = TokenEmbedding("emb", cfg.vocab_size, H)
      blocks = [PreNormBlock(f"l{i}", RMSNorm(f"l{i}.n1", H, cfg.rms_norm_eps), make(MIXERS, "toy_decay", f"l{i}.mix", H, cfg.decay),
                             RMSNorm(f"l{i}.n2", H, cfg.rms_norm_eps), SwiGLUFeedForward(f"l{i}.mlp", H, cfg.intermediate_size))
                for i in range(cfg.num_hidden_layers)]
      return ModelSpec(config=cfg, embedding=emb, blocks=blocks, final_norm=RMSNorm("norm", H, cfg.rms_norm_eps),
                       lm_head=LMHead("head", cfg.vocab_size, H, tied_to=emb))
  return ToyConfig


def plain_toy(weights, cfg, ids):
  """The toy model on one whole sequence, no cache."""
  import plain_qwen3 as plain
  res = weights["emb.weight"][torch.tensor(ids)]
  h = None
  for i in range(cfg["num_hidden_layers"]):
    if h is not None:
      res = h + res
    x = plain.rms_norm(res, weights[f"l{i}.n1.weight"], cfg["rms_norm_eps"])
    s = torch.zeros(cfg["hidden_size"])
    a = []
    for t in range(len(ids)):
      s = cfg["decay"] * s + x[t]
      a.append(s @ weights[f"l{i}.mix.w"].t())
    res = torch.stack(a) + res
    x = plain.rms_norm(res, weights[f"l{i}.n2.weight"], cfg["rms_norm_eps"])
    h = plain.swiglu_mlp(x, weights, f"l{i}")
  x = plain.rms_norm(h + res, weights["norm.weight"], cfg["rms_norm_eps"])
  return x @ weights["emb.weight"].t()


def test_toy_mixer_with_state_runs_through_the_engine(tmp_path):
  define_toy()
  import plain_qwen3 as plain
  import replay_cases as rc
  from miniinfer_b200.engine.replay import TraceRunner
  from miniinfer_b200.weights import write_random_model
  cfg = dict(architectures=["ToyDecayLM"], model_type="toy", vocab_size=97, max_position_embeddings=256, hidden_size=32,
             num_hidden_layers=2, decay=0.5, rms_norm_eps=1e-5, intermediate_size=48)
  d = write_random_model(cfg, str(tmp_path / "toy"), seed=3, dtype=torch.float32)
  weights = plain.read_weights(d)
  reqs = rc.make_requests(97, (40, 23, 9), seed=1)
  ref = {rid: plain_toy(weights, cfg, ids) for rid, ids in reqs.items()}
  runner = TraceRunner(d, "float32", 256, device=DEV)
  assert not runner.runner.graphs_allowed        # its mixer reads the step on the host: no CUDA graphs for it
  assert runner.cache.paged_groups == [] and len(runner.cache.state_groups) == 1
  assert runner.cache.state_groups[0].state.shape == (2, 9, 32)
  for trace in (rc.whole(reqs), rc.portions(reqs), rc.mixed(reqs, 256, seed=2)):
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, 1e-4, "toy")
    assert runner.cache.num_free_slots == 8
