"""Parts defined here, in the test, and put together into an architecture of their own without a
change to the package: a feed-forward with routing (a router in float32 picks two of four small
experts per token), a learned absolute position encoding that acts on the hidden state after the
embedding, and a model whose layers differ - the package's attention (no rotation, no QK norm) with
a dense feed-forward in one layer, the toy mixer with state and the routed feed-forward in the other.
The frame is the test's own too: an embedding that adds two tables (tokens, and token classes) and a head
that caps its logits softly.  The run list names the first block twice.  Compared with a plain whole-sequence statement under
every way of cutting the requests into steps."""
from dataclasses import dataclass
from typing import Dict

import pytest
import torch

from gpu_helpers import DEV
from test_toy_mixer_gpu import define_toy

pytestmark = pytest.mark.gpu


def define_parts():
  define_toy()                                   # registers the "toy_decay" mixer
  from miniinfer_b200.config import register_model
  from miniinfer_b200.config.model_config import ModelConfig
  from miniinfer_b200.config.registry import _MODELS
  from miniinfer_b200.models import LayerRun, ModelSpec
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.parts import (FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, AttentionMixer, Embedding, FeedForward, Head,
                                    ParamSpec, PositionEncoding, PreNormBlock, RMSNorm, SwiGLUFeedForward,
                                    make, register_feed_forward, register_position_encoding, whole)

  class TwoTableEmbedding(Embedding):
    """hidden_t = tokens[id_t] + classes[id_t mod num_classes]: a frame that starts from more than one table."""

    def __init__(self, name, vocab_size, hidden_size, num_classes):
      super().__init__(name)
      self.vocab_size, self.hidden_size, self.num_classes = vocab_size, hidden_size, num_classes

    def param_specs(self) -> Dict[str, ParamSpec]:
      V, H, C = self.vocab_size, self.hidden_size, self.num_classes
      return {"tokens": ParamSpec((V, H), "table", [whole(f"{self.name}.tokens", (V, H))]),
              "classes": ParamSpec((C, H), "table", [whole(f"{self.name}.classes", (C, H))])}

    def forward(self, ids, ctx):
      out = ctx.ws.buffer("resid", (ids.shape[0], self.hidden_size), torch.float32)
      ops.embedding(out, self.tokens, ids)
      out += self.classes[(ids % self.num_classes).long()].float()
      return out

  class SoftCapHead(Head):
    """logits = cap * tanh((x W^T) / cap), W the embedding's token table."""

    def __init__(self, name, vocab_size, hidden_size, cap, tied_to):
      super().__init__(name)
      self.vocab_size, self.hidden_size, self.cap, self.tied_to = vocab_size, hidden_size, cap, tied_to

    def forward(self, x, ctx):
      out = ctx.ws.buffer("logits", (x.shape[0], self.vocab_size), torch.float32)
      ops.linear(out, x, self.tied_to.tokens)
      out.copy_(self.cap * torch.tanh(out / self.cap))
      return out

  if "toy_routed" not in FEED_FORWARDS:
    @register_feed_forward("toy_routed")
    class RoutedFeedForward(FeedForward):
      """out = sum over the top-k experts e of softmax(router(x))_e * W2_e relu(W1_e x); router in float32."""

      def __init__(self, name, hidden_size, expert_size, num_experts, top_k):
        super().__init__(name)
        self.hidden_size, self.expert_size, self.num_experts, self.top_k = hidden_size, expert_size, num_experts, top_k

      def param_specs(self) -> Dict[str, ParamSpec]:
        H, I, E = self.hidden_size, self.expert_size, self.num_experts
        return {"router": ParamSpec((E, H), "vector", [whole(f"{self.name}.router", (E, H))]),
                "w1": ParamSpec((E * I, H), "matrix", [whole(f"{self.name}.w1", (E * I, H))]),
                "w2": ParamSpec((E * H, I), "matrix", [whole(f"{self.name}.w2", (E * H, I))])}

      def forward(self, x, ctx):
        H, I, E = self.hidden_size, self.expert_size, self.num_experts
        probs = torch.softmax(x.float() @ self.router.float().t(), dim=-1)
        top_p, top_e = probs.topk(self.top_k, dim=-1)
        out = torch.zeros(x.shape[0], H, dtype=torch.float32, device=x.device)
        w1, w2 = self.w1.view(E, I, H), self.w2.view(E, H, I)
        for e in range(E):
          weight = (top_p * (top_e == e)).sum(-1, keepdim=True)          # 0 where the token did not pick e
          rows = weight.squeeze(-1).nonzero().squeeze(-1)
          if rows.numel():
            h = torch.relu(x[rows].float() @ w1[e].float().t())
            out[rows] += weight[rows] * (h @ w2[e].float().t())
        return out.to(x.dtype)

  if "toy_learned" not in POSITION_ENCODINGS:
    @register_position_encoding("toy_learned")
    class LearnedPositions(PositionEncoding):
      """hidden_t += table[position_t], right after the embedding."""

      def __init__(self, name, hidden_size, num_positions):
        super().__init__(name)
        self.hidden_size, self.num_positions = hidden_size, num_positions

      def param_specs(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((self.num_positions, self.hidden_size), "vector",
                                   [whole(f"{self.name}.table", (self.num_positions, self.hidden_size))])}

      def max_positions(self):
        return self.num_positions

      def apply_to_hidden(self, resid, ctx):
        resid += self.table[ctx.positions.long()]

  @dataclass
  class ToyPartsConfig(ModelConfig):
    hidden_size: int = 48
    num_heads: int = 3
    num_kv_heads: int = 1
    head_dim: int = 16
    intermediate_size: int = 40
    expert_size: int = 24
    num_experts: int = 4
    top_k: int = 2
    decay: float = 0.25
    rms_norm_eps: float = 1e-5
    num_positions: int = 160
    num_classes: int = 7
    logit_cap: float = 3.0

  if "ToyPartsLM" not in _MODELS:
    @register_model("ToyPartsLM", ToyPartsConfig)
    def build(cfg):
      H = cfg.hidden_size
      emb = TwoTableEmbedding("emb", cfg.vocab_size, H, cfg.num_classes)
      pos = make(POSITION_ENCODINGS, "toy_learned", "pos", H, cfg.num_positions)
      attn = AttentionMixer("l0.attn", H, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.head_dim ** -0.5, None, None)
      b0 = PreNormBlock("l0", RMSNorm("l0.n1", H, cfg.rms_norm_eps), attn, RMSNorm("l0.n2", H, cfg.rms_norm_eps),
                        SwiGLUFeedForward("l0.mlp", H, cfg.intermediate_size))
      b1 = PreNormBlock("l1", RMSNorm("l1.n1", H, cfg.rms_norm_eps), make(MIXERS, "toy_decay", "l1.mix", H, cfg.decay),
                        RMSNorm("l1.n2", H, cfg.rms_norm_eps),
                        make(FEED_FORWARDS, "toy_routed", "l1.moe", H, cfg.expert_size, cfg.num_experts, cfg.top_k))
      # the attention block runs twice, with a cache of its own each time
      return ModelSpec(config=cfg, embedding=emb, blocks=[b0, b1], final_norm=RMSNorm("norm", H, cfg.rms_norm_eps),
                       lm_head=SoftCapHead("head", cfg.vocab_size, H, cfg.logit_cap, emb), position_encodings=[pos],
                       run_list=[LayerRun(0), LayerRun(1), LayerRun(0)])
  return ToyPartsConfig


def plain_parts_model(w, cfg, ids):
  """The toy architecture on one whole sequence, no cache."""
  import plain_qwen3 as plain
  T, H = len(ids), cfg["hidden_size"]
  nh, nkv, hd = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
  res = w["emb.tokens"][torch.tensor(ids)] + w["emb.classes"][torch.tensor(ids) % cfg["num_classes"]] + w["pos.table"][:T]

  def attention_block(res, pending):
    if pending is not None:
      res = pending + res
    x = plain.rms_norm(res, w["l0.n1.weight"], cfg["rms_norm_eps"])
    q = (x @ w["l0.attn.q_proj.weight"].t()).view(T, nh, hd)
    k = (x @ w["l0.attn.k_proj.weight"].t()).view(T, nkv, hd).repeat_interleave(nh // nkv, dim=1)
    v = (x @ w["l0.attn.v_proj.weight"].t()).view(T, nkv, hd).repeat_interleave(nh // nkv, dim=1)
    s = torch.einsum("thd,shd->hts", q, k) * hd ** -0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    a = torch.einsum("hts,shd->thd", torch.softmax(s, -1), v).reshape(T, nh * hd) @ w["l0.attn.o_proj.weight"].t()
    res = a + res
    x = plain.rms_norm(res, w["l0.n2.weight"], cfg["rms_norm_eps"])
    return res, plain.swiglu_mlp(x, w, "l0")

  def decay_block(res, pending):
    res = pending + res
    x = plain.rms_norm(res, w["l1.n1.weight"], cfg["rms_norm_eps"])
    s, a = torch.zeros(H), []
    for t in range(T):
      s = cfg["decay"] * s + x[t]
      a.append(s @ w["l1.mix.w"].t())
    res = torch.stack(a) + res
    x = plain.rms_norm(res, w["l1.n2.weight"], cfg["rms_norm_eps"])
    E, I = cfg["num_experts"], cfg["expert_size"]
    probs = torch.softmax(x @ w["l1.moe.router"].t(), -1)
    top_p, top_e = probs.topk(cfg["top_k"], -1)
    out = torch.zeros(T, H)
    for t in range(T):
      for p, e in zip(top_p[t], top_e[t]):
        w1, w2 = w["l1.moe.w1"].view(E, I, H)[e], w["l1.moe.w2"].view(E, H, I)[e]
        out[t] += p * (torch.relu(x[t] @ w1.t()) @ w2.t())
    return res, out

  res, pending = attention_block(res, None)
  res, pending = decay_block(res, pending)
  res, pending = attention_block(res, pending)
  x = plain.rms_norm(pending + res, w["norm.weight"], cfg["rms_norm_eps"])
  return cfg["logit_cap"] * torch.tanh((x @ w["emb.tokens"].t()) / cfg["logit_cap"])


def test_toy_parts_run_through_the_engine(tmp_path):
  define_parts()
  import plain_qwen3 as plain
  import replay_cases as rc
  from miniinfer_b200.engine.replay import TraceRunner
  from miniinfer_b200.weights import write_random_model
  cfg = dict(architectures=["ToyPartsLM"], model_type="toy_parts", vocab_size=101, max_position_embeddings=160, hidden_size=48,
             num_heads=3, num_kv_heads=1, head_dim=16, intermediate_size=40, expert_size=24, num_experts=4, top_k=2,
             decay=0.25, rms_norm_eps=1e-5, num_positions=160, num_classes=7, logit_cap=3.0)
  d = write_random_model(cfg, str(tmp_path / "toy_parts"), seed=4, dtype=torch.float32)
  weights = plain.read_weights(d)
  reqs = rc.make_requests(101, (70, 33, 12, 5), seed=2)
  ref = {rid: plain_parts_model(weights, cfg, ids) for rid, ids in reqs.items()}
  runner = TraceRunner(d, "float32", 256, device=DEV, page_size=16)
  # two run-list entries name the attention block: two cache layers in one paged group; one state layer
  assert len(runner.cache.paged_groups) == 1 and runner.cache.paged_groups[0].num_layers == 2
  assert len(runner.cache.state_groups) == 1
  assert runner.runner.max_position == 160
  for trace in (rc.whole(reqs), rc.tail_one_by_one(reqs), rc.portions(reqs), rc.mixed(reqs, 256, seed=3, granule=16)):
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, 2e-4, "toy parts")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]
