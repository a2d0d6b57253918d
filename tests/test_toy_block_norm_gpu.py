"""A norm and an arrangement of a layer defined here, in the test, and run through the engine without a
change to the package: a centred norm with a bias (mean and variance, not a plain RMSNorm, so no part may
take its place in a kernel of its own) and a block whose mixer and feed-forward both read ONE normalised
copy of the residual stream and whose outputs are added together (a "parallel" layer).  The model puts
such a layer beside a layer of the package's usual arrangement, with the package's attention (rotary
encoding, QK norm, grouped heads; a window in the second layer) and SwiGLU feed-forward inside both, and
ends in the centred norm too.  Compared with a plain whole-sequence statement under every way of cutting
the requests into steps, and through greedy generation from CUDA graphs."""
from dataclasses import dataclass
from typing import Dict, List, Optional

import pytest
import torch

from gpu_helpers import DEV

pytestmark = pytest.mark.gpu


def define_parts():
  from miniinfer_b200.config import register_model
  from miniinfer_b200.config.model_config import ModelConfig
  from miniinfer_b200.config.registry import _MODELS
  from miniinfer_b200.models import ModelSpec
  from miniinfer_b200.parts import (AttentionMixer, Block, LMHead, Norm, ParamSpec, PreNormBlock, RotaryEncoding,
                                    SwiGLUFeedForward, TokenEmbedding, whole)

  class CentredNorm(Norm):
    """y = weight * (x - mean(x)) / sqrt(var(x) + eps) + bias, in float32."""

    def __init__(self, name, dim, eps):
      super().__init__(name)
      self.dim, self.eps = dim, float(eps)

    def param_specs(self) -> Dict[str, ParamSpec]:
      return {"weight": ParamSpec((self.dim,), "vector", [whole(f"{self.name}.weight", (self.dim,))], init="ones_noise"),
              "bias": ParamSpec((self.dim,), "vector", [whole(f"{self.name}.bias", (self.dim,))])}

    def _norm(self, x, ctx):
      mu = x.mean(-1, keepdim=True)
      var = ((x - mu) ** 2).mean(-1, keepdim=True)
      return (self.weight * (x - mu) * torch.rsqrt(var + self.eps) + self.bias).to(ctx.dtype)

    def add_norm(self, resid, delta, ctx):
      if delta is not None:
        resid += delta.float()
      return self._norm(resid, ctx)

    def norm_rows(self, resid, delta, rows, ctx):
      x = resid[rows.long()]
      if delta is not None:
        x = x + delta[rows.long()].float()
      return self._norm(x, ctx)

  class ParallelBlock(Block):
    """pending = mixer(x) + feed_forward(x) with x = norm(residual + what was pending): one norm a layer."""

    def __init__(self, name, norm, mixer, ffn):
      super().__init__(name)
      self.norm, self.mixer, self.ffn = norm, mixer, ffn

    def sub_parts(self) -> List:
      return [self.norm, self.mixer, self.ffn]

    def mixer_part(self):
      return self.mixer

    def forward(self, resid, pending, ctx, cache) -> Optional[torch.Tensor]:
      x = self.norm.add_norm(resid, pending, ctx)
      a = self.mixer.forward(x, ctx, cache)
      f = self.ffn.forward(x, ctx)
      return a + f

  @dataclass
  class ToyParallelConfig(ModelConfig):
    hidden_size: int = 40
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 16
    intermediate_size: int = 56
    norm_eps: float = 1e-3
    rope_theta: float = 5000.0
    window: int = 24

  if "ToyParallelLM" not in _MODELS:
    @register_model("ToyParallelLM", ToyParallelConfig)
    def build(cfg):
      H, hd = cfg.hidden_size, cfg.head_dim
      emb = TokenEmbedding("emb", cfg.vocab_size, H)
      rope = RotaryEncoding("rope", hd, cfg.rope_theta, cfg.max_position_embeddings)

      def attn(name, window):
        return AttentionMixer(name, H, cfg.num_heads, cfg.num_kv_heads, hd, hd ** -0.5, cfg.norm_eps, rope, window)

      b0 = ParallelBlock("l0", CentredNorm("l0.n", H, cfg.norm_eps), attn("l0.self_attn", None),
                         SwiGLUFeedForward("l0.mlp", H, cfg.intermediate_size))
      b1 = PreNormBlock("l1", CentredNorm("l1.n1", H, cfg.norm_eps), attn("l1.self_attn", cfg.window),
                        CentredNorm("l1.n2", H, cfg.norm_eps), SwiGLUFeedForward("l1.mlp", H, cfg.intermediate_size))
      return ModelSpec(config=cfg, embedding=emb, blocks=[b0, b1], final_norm=CentredNorm("norm", H, cfg.norm_eps),
                       lm_head=LMHead("head", cfg.vocab_size, H, tied_to=emb), position_encodings=[rope])
  return ToyParallelConfig


def plain_parallel_model(w, cfg, ids):
  """The toy architecture on one whole sequence, no cache."""
  import plain_qwen3 as plain
  T, eps = len(ids), cfg["norm_eps"]
  acfg = dict(num_attention_heads=cfg["num_heads"], num_key_value_heads=cfg["num_kv_heads"], head_dim=cfg["head_dim"], rms_norm_eps=eps)
  cos, sin = plain.rope_table(T, cfg["head_dim"], cfg["rope_theta"])

  def norm(x, name):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return w[f"{name}.weight"] * (x - mu) * torch.rsqrt(var + eps) + w[f"{name}.bias"]

  res = w["emb.weight"][torch.tensor(ids)]
  x = norm(res, "l0.n")
  a, _ = plain.attention_part(x, w, "l0", acfg, cos, sin, None)
  pending = a + plain.swiglu_mlp(x, w, "l0")
  res = pending + res
  x = norm(res, "l1.n1")
  a, _ = plain.attention_part(x, w, "l1", acfg, cos, sin, cfg["window"])
  res = a + res
  pending = plain.swiglu_mlp(norm(res, "l1.n2"), w, "l1")
  return norm(pending + res, "norm") @ w["emb.weight"].t()


CFG = dict(architectures=["ToyParallelLM"], model_type="toy_parallel", vocab_size=97, max_position_embeddings=192, hidden_size=40,
           num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=56, norm_eps=1e-3, rope_theta=5000.0, window=24)


@pytest.mark.parametrize("dtype,bound", [("float32", 2e-4), ("bfloat16", 0.06)])
def test_a_norm_and_a_block_of_the_tests_own_run_through_the_engine(tmp_path, dtype, bound):
  define_parts()
  import plain_qwen3 as plain
  import replay_cases as rc
  from miniinfer_b200.engine.replay import TraceRunner
  from miniinfer_b200.weights import write_random_model
  d = write_random_model(CFG, str(tmp_path / "toy_parallel"), seed=6, dtype=torch.float32)
  weights = plain.read_weights(d)
  if dtype == "bfloat16":                      # the engine rounds matrices and tables to bfloat16: so does the statement
    weights = {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in weights.items()}
  reqs = rc.make_requests(97, (90, 41, 17, 6), seed=8)
  ref = {rid: plain_parallel_model(weights, CFG, ids) for rid, ids in reqs.items()}
  runner = TraceRunner(d, dtype, 320, device=DEV, page_size=16)
  # the layer with a window keeps pages of its own, apart from the layer that keeps every key
  assert len(runner.cache.paged_groups) == 2
  for trace in (rc.whole(reqs), rc.tail_one_by_one(reqs), rc.portions(reqs), rc.mixed(reqs, 320, seed=5, granule=16)):
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, bound, f"toy parallel/{dtype}")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


def test_generation_with_the_tests_own_norm_and_block_runs_from_graphs(tmp_path):
  define_parts()
  import plain_qwen3 as plain
  import replay_cases as rc
  from miniinfer_b200 import LLMEngine, SamplingParams
  from miniinfer_b200.weights import write_random_model
  d = write_random_model(CFG, str(tmp_path / "toy_parallel"), seed=6, dtype=torch.float32)
  weights = plain.read_weights(d)
  prompts = list(rc.make_requests(97, (30, 9, 51), seed=3).values())
  eng = LLMEngine(d, dtype="float32", device=DEV, page_size=16, num_pages=40, max_num_seqs=4, max_model_len=192)
  outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24))
  if DEV != "cpu":
    assert eng.runner.num_graphs() >= 1, "the decode steps were not replayed from a CUDA graph"
  for p, o in zip(prompts, outs):
    ids, toks = list(p), o["token_ids"]
    assert len(toks) == 24
    logits = plain_parallel_model(weights, CFG, ids + toks[:-1])
    for i, t in enumerate(toks):
      row = logits[len(ids) - 1 + i]
      assert t == int(row.argmax()) or float(row.max() - row[t]) < 2e-4
  eng.runner.check_status()
