"""A mixer that keeps per-request state and updates it in place ON THE DEVICE, without reading the step
on the host - so its steps are recorded into CUDA graphs and replayed like any other model's.

This is what the state slots of the cache manager are for (a recurrent or linear-attention layer).
The test is about the step function: recording a graph must not run the step's tokens through the
model a second time (the state would advance twice), padding entries of a decode graph must not
touch a live request's state, and the step that records must give what every other step gives.
Defined, registered and run here without a change to the package."""
from dataclasses import dataclass
from typing import Dict

import pytest
import torch

from gpu_helpers import DEV
from test_toy_mixer_gpu import plain_toy

pytestmark = pytest.mark.gpu


def define_device_toy():
  from miniinfer_b200.cache import FixedStateSpec
  from miniinfer_b200.config import register_model
  from miniinfer_b200.config.model_config import ModelConfig
  from miniinfer_b200.config.registry import _MODELS
  from miniinfer_b200.models import ModelSpec
  from miniinfer_b200.parts import (MIXERS, LMHead, Mixer, ParamSpec, PreNormBlock, RMSNorm, SwiGLUFeedForward,
                                    TokenEmbedding, make, register_mixer, whole)

  if "toy_decay_device" not in MIXERS:
    @register_mixer("toy_decay_device")
    class DeviceDecayMixer(Mixer):
      """out_t = W s_t, s_t = decay * s_{t-1} + x_t per request; all of it as device operations whose
      shapes depend only on the numbers of tokens and items, so a recorded step can be replayed."""

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
        T = x.shape[0]
        item = ctx.token_item.long()
        slot = ctx.seq_slot.long()
        j = (torch.arange(T, device=x.device) - ctx.q_start.long()[item]).float()          # place within the item's portion
        same = item[:, None] == item[None, :]
        lag = j[:, None] - j[None, :]
        w = torch.where(same & (lag >= 0), torch.pow(torch.full_like(lag, self.decay), lag.clamp(min=0)), torch.zeros_like(lag))
        before = cache.tensor[slot][item]                                                   # the state each token's request came with
        s = w @ x.float() + torch.pow(torch.full_like(j, self.decay), j + 1)[:, None] * before
        last = (ctx.q_start + ctx.q_len - 1).long()
        cache.tensor.index_copy_(0, slot, s[last])                                          # in place: the state after the portion
        return (s.to(x.dtype) @ self.w.t()).contiguous()

  @dataclass
  class ToyDeviceConfig(ModelConfig):
    hidden_size: int = 32
    num_hidden_layers: int = 2
    decay: float = 0.5
    rms_norm_eps: float = 1e-5
    intermediate_size: int = 48

  if "ToyDeviceDecayLM" not in _MODELS:
    @register_model("ToyDeviceDecayLM", ToyDeviceConfig)
    def build(cfg):
      H = cfg.hidden_size
      emb = TokenEmbedding("emb", cfg.vocab_size, H)
      blocks = [PreNormBlock(f"l{i}", RMSNorm(f"l{i}.n1", H, cfg.rms_norm_eps), make(MIXERS, "toy_decay_device", f"l{i}.mix", H, cfg.decay),
                             RMSNorm(f"l{i}.n2", H, cfg.rms_norm_eps), SwiGLUFeedForward(f"l{i}.mlp", H, cfg.intermediate_size))
                for i in range(cfg.num_hidden_layers)]
      return ModelSpec(config=cfg, embedding=emb, blocks=blocks, final_norm=RMSNorm("norm", H, cfg.rms_norm_eps),
                       lm_head=LMHead("head", cfg.vocab_size, H, tied_to=emb))


CFG = dict(architectures=["ToyDeviceDecayLM"], model_type="toy", vocab_size=97, max_position_embeddings=256, hidden_size=32,
           num_hidden_layers=2, decay=0.5, rms_norm_eps=1e-5, intermediate_size=48)


def test_state_updated_on_the_device_survives_graph_recording(tmp_path):
  define_device_toy()
  import plain_qwen3 as plain
  import replay_cases as rc
  from miniinfer_b200.engine.replay import TraceRunner
  from miniinfer_b200.weights import write_random_model
  d = write_random_model(dict(CFG), str(tmp_path / "toy"), seed=3, dtype=torch.float32)
  weights = plain.read_weights(d)
  reqs = rc.make_requests(97, (40, 23, 9, 40, 23), seed=1)
  ref = {rid: plain_toy(weights, CFG, ids) for rid, ids in reqs.items()}
  runner = TraceRunner(d, "float32", 256, device=DEV)
  assert runner.runner.graphs_allowed == True
  assert runner.cache.paged_groups == [] and len(runner.cache.state_groups) == 1
  # whole: the prompts of 40 and of 23 tokens come twice, the second time their step is recorded, and
  # a recorded step is replayed for the decode tail; portions and mixed steps repeat shapes as well
  for name, trace in (("whole", rc.whole(reqs)), ("tail", rc.tail_one_by_one(reqs, tail=20)), ("portions", rc.portions(reqs)),
                      ("mixed", rc.mixed(reqs, 256, seed=2)), ("preempted", rc.mixed(reqs, 256, seed=3, preempt=True))):
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, 1e-4, f"device toy/{name}")
    assert runner.cache.num_free_slots == 8
  if DEV != "cpu":
    assert runner.runner.num_graphs() >= 2          # steps were recorded and replayed along the way


def test_state_mixer_decodes_from_graphs_through_the_entry_point(tmp_path):
  """Twenty greedy tokens for three requests: the decode steps are CUDA graphs (one is recorded on
  the way, padded to its bucket); tokens equal to the plain statement run on whole sequences."""
  define_device_toy()
  import plain_qwen3 as plain
  from miniinfer_b200 import LLMEngine, SamplingParams
  from miniinfer_b200.weights import write_random_model
  d = write_random_model(dict(CFG), str(tmp_path / "toy"), seed=4, dtype=torch.float32)
  weights = plain.read_weights(d)
  prompts = [[5, 17, 3, 90, 9], list(range(40, 63)), [7, 8, 9]]

  def plain_generate(ids, n):
    ids = list(ids)
    for _ in range(n):
      ids.append(int(plain_toy(weights, CFG, ids)[-1].argmax()))
    return ids[-n:]

  want = [plain_generate(p, 20) for p in prompts]
  for eager in (False, True):
    eng = LLMEngine(d, dtype="float32", device=DEV, page_size=16, num_pages=8, max_num_seqs=4, max_model_len=128,
                    enforce_eager=eager)
    got = [o["token_ids"] for o in eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=20))]
    assert got == want, f"enforce_eager={eager}"
    if DEV != "cpu":
      assert (eng.runner.num_graphs() >= 1) == (not eager)
