"""Each part of a layer alone on the GPU against the plain implementation's function for it, at
sizes of its own, in float32 and bfloat16."""
from types import SimpleNamespace

import pytest
import torch

import plain_qwen3 as plain
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu


def bind_random(part, dtype, seed):
  from miniinfer_b200.weights.loader import role_dtype
  g = torch.Generator().manual_seed(seed)
  params, host = {}, {}
  for name, ps in part.param_specs().items():
    t = torch.randn(ps.shape, generator=g)
    t = (1 + 0.1 * t) if ps.init == "ones_noise" else 0.05 * t
    t = t.to(role_dtype(ps.role, dtype))
    params[name] = t.to(DEV)
    host[name] = t.float()
  part.bind(params)
  return host


def context_for(mixers, rope, dtype, T, page_size=16, start=0):
  """A step context for one request with T new tokens at positions start.., through the real
  cache manager and step preparation."""
  from miniinfer_b200.cache import KVCacheManager
  from miniinfer_b200.engine import ModelRunner, StepItem
  from miniinfer_b200.models import LayerRun
  blocks = [SimpleNamespace(mixer_part=lambda m=m: m) for m in mixers]
  spec = SimpleNamespace(position_encodings=[rope] if rope else [], run_list=[LayerRun(i) for i in range(len(mixers))],
                         blocks=blocks, config=SimpleNamespace(vocab_size=10), all_parts=lambda: list(mixers))
  cache = KVCacheManager([m.cache_spec() for m in mixers], page_size, 40, 2, 512, dtype, DEV)
  runner = ModelRunner(spec, cache, dtype, DEV)
  cache.admit("x")
  if start:
    cache.append("x", start); cache.commit("x", start)
  ctx = runner.prepare([StepItem("x", [1] * T, [])])
  return ctx, runner, cache


TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
  from miniinfer_b200.parts import RMSNorm
  part = RMSNorm("n", 200, 1e-5)
  w = bind_random(part, dtype, 1)["weight"]
  ctx, _, _ = context_for([], None, dtype, 9)
  resid = torch.randn(9, 200, device=DEV)
  delta = torch.randn(9, 200, device=DEV).to(dtype)
  want_sum = resid.cpu() + delta.float().cpu()
  out = part.add_norm(resid, delta, ctx)
  assert torch.allclose(resid.cpu(), want_sum, atol=1e-6)
  want = plain.rms_norm(want_sum, w, 1e-5)
  assert (out.float().cpu() - want).abs().max() < TOL[dtype] * 4
  rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
  out = part.norm_rows(resid, None, rows, ctx)
  assert (out.float().cpu() - want[[8, 2]]).abs().max() < TOL[dtype] * 4


def test_rotary_table_equals_the_plain_one():
  from miniinfer_b200.parts import RotaryEncoding
  rope = RotaryEncoding("r", 48, 50000.0, 4096)
  rope.prepare(DEV, 300)
  cos, sin = plain.rope_table(300, 48, 50000.0)
  t = rope.rotary_table().cpu()
  assert t.shape == (300, 48) and torch.equal(t[:, :24], cos) and torch.equal(t[:, 24:], sin)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,H,window", [(6, 2, 48, 80, None), (4, 1, 32, 136, 20), (8, 8, 16, 64, None)])
def test_attention_mixer_part(dtype, nh, nkv, hd, H, window):
  from miniinfer_b200.parts import AttentionMixer, RotaryEncoding
  rope = RotaryEncoding("r", hd, 10000.0, 512)
  m = AttentionMixer("a", H, nh, nkv, hd, hd ** -0.5, 1e-6, rope, window)
  host = bind_random(m, dtype, 2)
  T = 57
  x = (torch.randn(T, H, generator=torch.Generator().manual_seed(3))).to(dtype)
  weights = {"a.self_attn.qkv_proj.weight": host["qkv"], "a.self_attn.o_proj.weight": host["o"],
             "a.self_attn.q_norm.weight": host["q_norm"], "a.self_attn.k_norm.weight": host["k_norm"]}
  cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rms_norm_eps": 1e-6}
  cos, sin = plain.rope_table(T, hd, 10000.0)
  want, _ = plain.attention_part(x.float(), weights, "a", cfg, cos, sin, window)
  # whole, and in two portions (the second reads the first from the cache)
  ctx, runner, cache = context_for([m], rope, dtype, T)
  got = m.forward(x.to(DEV), ctx, runner.layer_caches[0]).float().cpu()
  assert (got - want).abs().max() < TOL[dtype]
  ctx, runner, cache = context_for([m], rope, dtype, 40)
  first = m.forward(x[:40].contiguous().to(DEV), ctx, runner.layer_caches[0]).float().cpu().clone()
  cache.commit("x", 40)
  from miniinfer_b200.engine import StepItem
  ctx = runner.prepare([StepItem("x", [1] * (T - 40), [])])
  second = m.forward(x[40:].contiguous().to(DEV), ctx, runner.layer_caches[0]).float().cpu()
  assert (torch.cat([first, second]) - want).abs().max() < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
  from miniinfer_b200.parts import SwiGLUFeedForward
  f = SwiGLUFeedForward("f.mlp", 136, 176)
  host = bind_random(f, dtype, 4)
  x = torch.randn(21, 136, generator=torch.Generator().manual_seed(5)).to(dtype)
  ctx, _, _ = context_for([], None, dtype, 21)
  got = f.forward(x.to(DEV), ctx).float().cpu()
  want = plain.swiglu_mlp(x.float(), {"f.mlp.gate_up_proj.weight": host["gate_up"], "f.mlp.down_proj.weight": host["down"]}, "f")
  assert (got - want).abs().max() < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_lm_head_parts(dtype, tied):
  from miniinfer_b200.parts import LMHead, TokenEmbedding
  e = TokenEmbedding("e", 1000, 72)
  table = bind_random(e, dtype, 6)["weight"]
  h = LMHead("h", 1000, 72, tied_to=e if tied else None)
  head = table if tied else bind_random(h, dtype, 7)["weight"]
  ctx, _, _ = context_for([], None, dtype, 5)
  ids = torch.tensor([3, 999, 0, 17, 500], dtype=torch.int32, device=DEV)
  assert torch.equal(e.forward(ids, ctx).cpu(), plain.embedding(table, ids.cpu()))
  x = torch.randn(5, 72, generator=torch.Generator().manual_seed(8)).to(dtype)
  got = h.forward(x.to(DEV), ctx)
  assert got.dtype == torch.float32
  assert (got.cpu() - x.float() @ head.t()).abs().max() < (1e-5 if dtype == torch.float32 else 1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_arrangement(dtype):
  from miniinfer_b200.parts import AttentionMixer, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLUFeedForward
  H, nh, nkv, hd, I, T = 80, 6, 2, 48, 176, 33
  rope = RotaryEncoding("r", hd, 10000.0, 512)
  blk = PreNormBlock("b", RMSNorm("b.input_layernorm", H, 1e-5), AttentionMixer("b.self_attn", H, nh, nkv, hd, hd ** -0.5, 1e-5, rope),
                     RMSNorm("b.post_attention_layernorm", H, 1e-5), SwiGLUFeedForward("b.mlp", H, I))
  w = {}
  for i, part in enumerate(blk.sub_parts()):
    for k, v in bind_random(part, dtype, 10 + i).items():
      w[f"{part.name}.{ {'qkv': 'qkv_proj', 'o': 'o_proj', 'gate_up': 'gate_up_proj', 'down': 'down_proj'}.get(k, k)}.weight".replace(".weight.weight", ".weight")] = v
  resid0 = torch.randn(T, H, generator=torch.Generator().manual_seed(1))
  pend0 = torch.randn(T, H, generator=torch.Generator().manual_seed(2)).to(dtype)
  ctx, runner, _ = context_for([blk.mixer], rope, dtype, T)
  resid = resid0.clone().to(DEV)
  pending = blk.forward(resid, pend0.to(DEV), ctx, runner.layer_caches[0])
  # the same arrangement with the plain parts (miniinfer/models/fused_qwen3.py:175-196)
  cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rms_norm_eps": 1e-5}
  cos, sin = plain.rope_table(T, hd, 10000.0)
  r = resid0 + pend0.float()
  a, _ = plain.attention_part(plain.rms_norm(r, w["b.input_layernorm.weight"], 1e-5), w, "b", cfg, cos, sin, None)
  r = r + a
  want = plain.swiglu_mlp(plain.rms_norm(r, w["b.post_attention_layernorm.weight"], 1e-5), w, "b")
  assert (resid.cpu() - r).abs().max() < TOL[dtype]
  assert (pending.float().cpu() - want).abs().max() < TOL[dtype]
