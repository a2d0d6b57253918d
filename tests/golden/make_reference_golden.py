"""Makes tests/golden/reference_logits_{A,B}.npz with tom-jerr/MiniInfer's OWN model code on the CPU.

Run once, by hand, where the reference checkout is available:

    python tests/golden/make_reference_golden.py /path/to/MiniInfer

It builds ``miniinfer.models.fused_qwen3.Qwen3ForCausalLM`` in float32 from a tiny configuration,
loads random weights drawn from a seeded CPU generator, runs one whole sequence and stores the
token ids, the logits at every position, and the weights themselves (under ``w:<tensor name>``; they
are small), so that tests/test_plain.py does not depend on what a torch build draws from a seed.

The reference's forward needs a GPU in three places; each is replaced by the same formula in torch,
and the attention library by the reference's own dense grouped attention:
  * ``RMSNorm.rms_forward`` is ``@torch.compile``d (miniinfer/layers/layernorm.py:22): run eagerly,
    same body;
  * ``add_rms_norm_forward`` is a Triton kernel (kernels/triton/rms_norm.py:66-149): acc = x + res,
    out = w * (acc * rsqrt(mean(acc^2) + eps));
  * ``SiluAndMul`` is a Triton kernel (kernels/triton/silu_mul.py:6-74): silu(gate) * up;
  * the attention backend: ``scaled_dot_product_attention_grouped(..., mask="causal")``
    (miniinfer/layers/attention.py:131-191), as the reference's tests do (tests/utils.py:196-276).
To get logits at every position the sequence is passed with ``extend_seq_lens_cpu = [1] * T``
(the model keeps the last row of each sequence, fused_qwen3.py:317-334).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from tiny_configs import TINY_A, TINY_B  # noqa: E402


def draw_weights(cfg: dict, seed: int) -> dict:
  """Split (q/k/v, gate/up) float32 tensors by name, from one seeded generator, in this order."""
  g = torch.Generator().manual_seed(seed)
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

  def n(*s):
    return torch.randn(*s, generator=g) * 0.02

  def w1(d):
    return 1 + 0.1 * torch.randn(d, generator=g)

  sd = {"model.embed_tokens.weight": n(V, H)}
  for i in range(cfg["num_hidden_layers"]):
    p = f"model.layers.{i}"
    sd[f"{p}.input_layernorm.weight"] = w1(H)
    sd[f"{p}.self_attn.q_proj.weight"] = n(nh * hd, H)
    sd[f"{p}.self_attn.k_proj.weight"] = n(nkv * hd, H)
    sd[f"{p}.self_attn.v_proj.weight"] = n(nkv * hd, H)
    sd[f"{p}.self_attn.o_proj.weight"] = n(H, nh * hd)
    sd[f"{p}.self_attn.q_norm.weight"] = w1(hd)
    sd[f"{p}.self_attn.k_norm.weight"] = w1(hd)
    sd[f"{p}.post_attention_layernorm.weight"] = w1(H)
    sd[f"{p}.mlp.gate_proj.weight"] = n(I, H)
    sd[f"{p}.mlp.up_proj.weight"] = n(I, H)
    sd[f"{p}.mlp.down_proj.weight"] = n(H, I)
  sd["model.norm.weight"] = w1(H)
  if not cfg["tie_word_embeddings"]:
    sd["lm_head.weight"] = n(V, H)
  return sd


def checksum(sd: dict) -> float:
  return float(sum(v.double().abs().sum() for v in sd.values()))


def main(ref_root: str) -> None:
  sys.path.insert(0, ref_root)
  os.environ.update(HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1", MINIINFER_EAGER_IMPORT="0")
  import miniinfer.layers.layernorm as ln
  import miniinfer.models.fused_qwen3 as fq3
  from miniinfer.config.model.qwen3 import Qwen3Config
  from miniinfer.layers.attention import scaled_dot_product_attention_grouped
  from miniinfer.loader.weight import _merge_state_dict
  from miniinfer.scheduler.scheduler_batch import ForwardBatch, ForwardMode

  def add_rms(x, residual, weight, eps):
    acc = x + residual
    a = acc.float()
    return (a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps)).to(acc.dtype) * weight, acc

  def rms_forward(self, x):
    d = x.dtype
    x = x.float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
    return self.weight * x.to(d)

  def silu_mul(x):
    n = x.shape[-1] // 2
    g, u = x[..., :n], x[..., n:]
    return (g.float() * torch.sigmoid(g.float())).to(g.dtype) * u

  ln.add_rms_norm_forward = add_rms
  ln.RMSNorm.rms_forward = rms_forward

  class Dense:
    def forward(self, q, k, v, layer, fb, save_kv_cache=True, **kw):
      T = q.shape[0]
      q = q.view(1, T, layer.tp_q_head_num, layer.head_dim).transpose(1, 2)
      k = k.view(1, T, layer.tp_k_head_num, layer.head_dim).transpose(1, 2)
      v = v.view(1, T, layer.tp_v_head_num, layer.head_dim).transpose(1, 2)
      o = scaled_dot_product_attention_grouped(q, k, v, scale=layer.scaling, mask="causal")
      return o.transpose(1, 2).reshape(T, -1)

  for tag, cfg, seed, T in (("A", TINY_A, 11, 33), ("B", TINY_B, 12, 71)):
    keys = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "max_position_embeddings",
            "tie_word_embeddings")
    rc = Qwen3Config(**{k: cfg[k] for k in keys})
    sd = draw_weights(cfg, seed)
    model = fq3.Qwen3ForCausalLM(rc, device=torch.device("cpu"), precision=torch.float32)
    model.load_weights(_merge_state_dict({k: v.clone() for k, v in sd.items()}))
    model.eval()
    for m in model.modules():
      if isinstance(m, fq3.Qwen3MLP):
        m.act_fn = silu_mul
    ids = torch.randint(0, cfg["vocab_size"], (T,), generator=torch.Generator().manual_seed(seed + 100))
    pos = torch.arange(T)
    fb = ForwardBatch(forward_mode=ForwardMode.EXTEND, batch_size=1, input_ids=ids, positions=pos)
    fb.attn_backend = Dense()
    fb.extend_seq_lens_cpu = [1] * T
    logits = model(ids, pos, fb).logits
    assert logits.shape == (T, cfg["vocab_size"]), logits.shape
    np.savez_compressed(os.path.join(HERE, f"reference_logits_{tag}.npz"), ids=ids.numpy().astype(np.int32),
                        logits=logits.float().numpy(), weight_checksum=np.float64(checksum(sd)),
                        seed=np.int64(seed), **{f"w:{k}": v.numpy() for k, v in sd.items()})
    print(tag, logits.shape, float(logits.abs().max()))


if __name__ == "__main__":
  if len(sys.argv) != 2:
    sys.exit("usage: make_reference_golden.py <path of a checkout of tom-jerr/MiniInfer>")
  main(sys.argv[1])
