"""A plain, slow statement of the Qwen3 dense decoder, used as the oracle of the tests.

Whole sequences, no cache, float32 arithmetic (or float64 on request), one function per part.
Nothing here imports the engine package: weights are read straight from ``model.safetensors``
and the configuration straight from ``config.json``.

Every function cites the place in tom-jerr/MiniInfer whose formula it states (paths are relative
to that project's root).  The numbers of ``tests/golden/`` were made by that project's own model
code on the CPU and pin this file to it (see ``tests/golden/make_reference_golden.py``).

Two things go beyond what MiniInfer computes, and are marked where they occur:
  * a sliding window (``use_sliding_window``/``sliding_window``/``max_window_layers``/``layer_types``
    are carried by MiniInfer's configuration, ``miniinfer/config/model/base.py:29-31``, but never
    read), stated here the way the keys are documented for the architecture: a query at position
    ``p`` sees the keys ``j`` with ``p - window < j <= p``;
  * a run list that may name a layer twice or let a layer read another layer's keys and values.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- model folder


def read_config(model_dir: str) -> dict:
  """config.json as a dict (miniinfer/config/model/base.py:56-60)."""
  with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as f:
    return json.load(f)


def read_weights(model_dir: str, dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
  """All tensors of every ``*.safetensors`` file, by name (miniinfer/loader/weight.py:109-158)."""
  from safetensors import safe_open

  out: Dict[str, torch.Tensor] = {}
  for name in sorted(os.listdir(model_dir)):
    if not name.endswith(".safetensors"):
      continue
    with safe_open(os.path.join(model_dir, name), framework="pt", device="cpu") as f:
      for key in f.keys():
        t = f.get_tensor(key)
        out[key] = t.to(dtype) if t.is_floating_point() else t
  return out


def _w(weights: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
  """Names may or may not carry the ``model.`` prefix (miniinfer/models/fused_qwen3.py:225-226)."""
  if name in weights:
    return weights[name]
  if name.startswith("model.") and name[len("model."):] in weights:
    return weights[name[len("model."):]]
  raise KeyError(name)


# --------------------------------------------------------------------------- parts


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
  """``h[t] = E[ids[t]]`` (miniinfer/layers/embedding.py:23-27)."""
  return table[ids.long(), :]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
  """``w * x * rsqrt(mean(x^2) + eps)`` (miniinfer/layers/layernorm.py:27-32)."""
  var = x.pow(2).mean(-1, keepdim=True)
  return weight * (x * torch.rsqrt(var + eps))


def rope_table(max_pos: int, head_dim: int, theta: float,
               dtype: torch.dtype = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
  """cos and sin of ``pos * theta^(-2j/head_dim)`` (miniinfer/layers/position_encoding.py:29-45).

  The table is always made in float32, as there, and then cast."""
  inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
  t = torch.arange(max_pos, dtype=torch.float)
  freqs = torch.einsum("i,j -> ij", t, inv_freq)
  return freqs.cos().to(dtype), freqs.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
  """Half-split (NeoX) rotation over the whole head (position_encoding.py:91-116).

  ``x``: [T, heads, head_dim]; ``cos``/``sin``: [T, head_dim/2]."""
  c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
  x1, x2 = torch.chunk(x, 2, dim=-1)
  return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def attention_scores_mask(q_pos: torch.Tensor, k_pos: torch.Tensor, window: Optional[int]) -> torch.Tensor:
  """True where a query may see a key: causal (miniinfer/layers/attention.py:112-128), and inside
  the window if there is one (beyond MiniInfer, see the header)."""
  ok = k_pos.unsqueeze(0) <= q_pos.unsqueeze(1)
  if window is not None:
    ok = ok & (k_pos.unsqueeze(0) > q_pos.unsqueeze(1) - window)
  return ok


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                  window: Optional[int] = None) -> torch.Tensor:
  """Grouped-query causal attention over one whole sequence
  (miniinfer/layers/attention.py:131-191; query head h reads kv head h // (nh/nkv)).

  q: [T, nh, hd]; k, v: [T, nkv, hd]  ->  [T, nh*hd]."""
  T, nh, hd = q.shape
  nkv = k.shape[1]
  g = nh // nkv
  pos = torch.arange(T)
  ok = attention_scores_mask(pos, pos, window)                      # [T, T]
  qh = q.permute(1, 0, 2).reshape(nkv, g, T, hd)
  kh = k.permute(1, 0, 2).reshape(nkv, 1, T, hd)
  vh = v.permute(1, 0, 2).reshape(nkv, 1, T, hd)
  s = torch.matmul(qh, kh.transpose(-2, -1)) * scale               # [nkv, g, T, T]
  s = s.masked_fill(~ok, float("-inf"))
  p = torch.softmax(s, dim=-1)
  o = torch.matmul(p, vh)                                          # [nkv, g, T, hd]
  return o.reshape(nh, T, hd).permute(1, 0, 2).reshape(T, nh * hd)


def qkv_project(x: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
  """q, k, v projections without bias (miniinfer/models/fused_qwen3.py:51-53,95-96); the fused
  matrix of MiniInfer is cat(q_proj, k_proj, v_proj) (miniinfer/loader/weight.py:78-86)."""
  q = x @ _w(weights, f"{prefix}.self_attn.q_proj.weight").t()
  k = x @ _w(weights, f"{prefix}.self_attn.k_proj.weight").t()
  v = x @ _w(weights, f"{prefix}.self_attn.v_proj.weight").t()
  return q, k, v


def attention_part(x: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                   cos: torch.Tensor, sin: torch.Tensor, window: Optional[int],
                   shared_kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                   ) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
  """QKV -> per-head RMSNorm of q and k -> RoPE -> attention -> o_proj
  (miniinfer/models/fused_qwen3.py:95-108).  Returns the output and the (k, v) it used."""
  T = x.shape[0]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  eps = cfg["rms_norm_eps"]
  fused = f"{prefix}.self_attn.qkv_proj.weight"
  if fused in weights or fused[len("model."):] in weights:
    qkv = x @ _w(weights, fused).t()
    q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
  else:
    q, k, v = qkv_project(x, weights, prefix)
  q = rms_norm(q.reshape(T, nh, hd), _w(weights, f"{prefix}.self_attn.q_norm.weight"), eps)
  q = apply_rope(q, cos, sin)
  if shared_kv is None:
    k = rms_norm(k.reshape(T, nkv, hd), _w(weights, f"{prefix}.self_attn.k_norm.weight"), eps)
    k = apply_rope(k, cos, sin)
    v = v.reshape(T, nkv, hd)
  else:
    k, v = shared_kv
  o = gqa_attention(q, k, v, hd ** -0.5, window)                    # scale: fused_qwen3.py:47
  return o @ _w(weights, f"{prefix}.self_attn.o_proj.weight").t(), (k, v)


def swiglu_mlp(x: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
  """``down(silu(gate(x)) * up(x))`` (miniinfer/models/fused_qwen3.py:134-138;
  kernels/triton/silu_mul.py:35-37; fused matrix = cat(gate, up), loader/weight.py:87-93)."""
  fused = f"{prefix}.mlp.gate_up_proj.weight"
  if fused in weights or fused[len("model."):] in weights:
    gu = x @ _w(weights, fused).t()
    g, u = gu.chunk(2, dim=-1)
  else:
    g = x @ _w(weights, f"{prefix}.mlp.gate_proj.weight").t()
    u = x @ _w(weights, f"{prefix}.mlp.up_proj.weight").t()
  act = g * torch.sigmoid(g) * u
  return act @ _w(weights, f"{prefix}.mlp.down_proj.weight").t()


def layer_window(cfg: dict, layer: int) -> Optional[int]:
  """The window of a layer, or None (beyond MiniInfer, see the header).  ``layer_types`` wins if
  it is given; else the layers from ``max_window_layers`` on are windowed when
  ``use_sliding_window`` is set."""
  if not cfg.get("use_sliding_window", False) or cfg.get("sliding_window") is None:
    return None
  types = cfg.get("layer_types")
  if types is not None:
    return int(cfg["sliding_window"]) if types[layer] == "sliding_attention" else None
  return int(cfg["sliding_window"]) if layer >= cfg.get("max_window_layers", 0) else None


def lm_head_weight(weights: Dict[str, torch.Tensor]) -> torch.Tensor:
  """``lm_head.weight`` if the file has it, else the embedding table
  (miniinfer/layers/embedding.py:41-48)."""
  if "lm_head.weight" in weights:
    return weights["lm_head.weight"]
  return _w(weights, "model.embed_tokens.weight")


def forward(weights: Dict[str, torch.Tensor], cfg: dict, ids: Sequence[int],
            run_list: Optional[List[Tuple[int, Optional[int]]]] = None,
            dtype: torch.dtype = torch.float32, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
  """Logits [T, V] of one whole sequence (miniinfer/models/fused_qwen3.py:243-259,344); with
  ``rows``, only at those positions (the reference keeps the last row of a sequence,
  fused_qwen3.py:317-334): the layers still run on the whole sequence.

  The block is pre-norm with the residual carried beside the hidden state
  (fused_qwen3.py:175-196): ``res = h (+ res)``; ``x = norm1(res)``; ``a = attn(x)``;
  ``res = a + res``; ``x = norm2(res)``; ``h = mlp(x)``; after the last layer
  ``norm(h + res)``.

  ``run_list`` (beyond MiniInfer): entries ``(layer, kv_of)``; entry ``i`` runs the weights of
  ``layer``; if ``kv_of`` is an earlier entry's index it uses that entry's keys and values instead
  of making its own.  Default: every layer once, in order."""
  weights = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
  ids_t = torch.as_tensor(list(ids), dtype=torch.long)
  T = ids_t.shape[0]
  hd = cfg["head_dim"]
  cos, sin = rope_table(max(T, 1), hd, float(cfg["rope_theta"]), dtype)
  eps = cfg["rms_norm_eps"]
  if run_list is None:
    run_list = [(i, None) for i in range(cfg["num_hidden_layers"])]

  res = embedding(_w(weights, "model.embed_tokens.weight"), ids_t)
  h = None
  kv_of_entry: List[Tuple[torch.Tensor, torch.Tensor]] = []
  for layer, kv_of in run_list:
    p = f"model.layers.{layer}"
    if h is not None:
      res = h + res
    x = rms_norm(res, _w(weights, f"{p}.input_layernorm.weight"), eps)
    shared = kv_of_entry[kv_of] if kv_of is not None else None
    a, kv = attention_part(x, weights, p, cfg, cos[:T], sin[:T], layer_window(cfg, layer), shared)
    kv_of_entry.append(kv)
    res = a + res
    x = rms_norm(res, _w(weights, f"{p}.post_attention_layernorm.weight"), eps)
    h = swiglu_mlp(x, weights, p)
  if h is not None:
    res = h + res
  if rows is not None:
    res = res[torch.as_tensor(list(rows), dtype=torch.long)]
  x = rms_norm(res, _w(weights, "model.norm.weight"), eps)
  return (x @ lm_head_weight(weights).t()).float()


# --------------------------------------------------------------------------- sampling


def _mix64(x: int) -> int:
  """The 64-bit finaliser the engine's sampler documents for its counter-based random numbers
  (splitmix64's output function); restated here from the documented constants."""
  m = (1 << 64) - 1
  x &= m
  x ^= x >> 30
  x = (x * 0xBF58476D1CE4E5B9) & m
  x ^= x >> 27
  x = (x * 0x94D049BB133111EB) & m
  x ^= x >> 31
  return x


def uniform_for(seed: int, counter: int, index: int) -> float:
  """The uniform number in (0, 1) that belongs to (seed, output index, vocabulary index)."""
  key = _mix64((seed & ((1 << 64) - 1)) ^ _mix64(counter + 0x9E3779B97F4A7C15))
  bits = _mix64(key ^ ((index * 0xD1342543DE82EF95) & ((1 << 64) - 1)))
  return uniform_from_bits(bits)


def uniform_from_bits(bits: int) -> float:
  """The top 23 bits of a 64-bit hash as a number strictly inside (0, 1): (n + 0.5) / 2^23 has 24
  significant bits, so float32 holds it exactly and the largest value is 1 - 2^-24, not 1."""
  return ((bits >> 41) + 0.5) * (1.0 / (1 << 23))


def filter_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
  """Temperature, then top-k, then top-p, as MiniInfer's sampler applies them
  (miniinfer/layers/sample.py:115-122: softmax(logits/T), top-k first, then top-p).  Returns the
  scaled logits with the excluded entries at -inf.  Ties at either threshold are all kept."""
  z = logits.double() / max(temperature, 1e-10)
  if top_k and top_k > 0 and top_k < z.numel():
    kth = torch.topk(z, top_k).values[-1]
    z = torch.where(z >= kth, z, torch.full_like(z, float("-inf")))
  if top_p < 1.0:
    probs = torch.softmax(z, dim=-1)
    sp, _ = torch.sort(probs, descending=True)
    before = torch.cumsum(sp, 0) - sp                # mass strictly ahead of each entry
    last_kept = int((before < top_p).nonzero().max())
    z = torch.where(probs >= sp[last_kept], z, torch.full_like(z, float("-inf")))
  return z


def sample_token(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                 seed: int, counter: int) -> Tuple[int, torch.Tensor]:
  """One token.  ``temperature == 0`` is the arg-max with the lowest index among equals
  (miniinfer/layers/sample.py:111-112).  Otherwise the Gumbel-max form of sampling from
  softmax(filtered logits): argmax(z_i - log(-log u_i)), which draws from the same distribution
  as sample.py:115-128.  Also returns the perturbed scores, for tests that accept near-ties."""
  if temperature <= 0.0:
    return int(torch.argmax(logits.float())), logits.double()
  z = filter_logits(logits, temperature, top_k, top_p)
  u = torch.tensor([uniform_for(seed, counter, i) for i in range(z.numel())], dtype=torch.float64)
  score = z - torch.log(-torch.log(u))
  return int(torch.argmax(score)), score


def generate(weights: Dict[str, torch.Tensor], cfg: dict, prompt: Sequence[int], max_tokens: int,
             temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
             eos: Optional[Sequence[int]] = None) -> List[int]:
  """Token-by-token generation by running the whole sequence again for every new token."""
  ids = list(prompt)
  out: List[int] = []
  for n in range(max_tokens):
    logits = forward(weights, cfg, ids, rows=[len(ids) - 1])[0]
    tok, _ = sample_token(logits, temperature, top_k, top_p, seed, n)
    out.append(tok)
    ids.append(tok)
    if eos is not None and tok in eos:
      break
  return out


def check_greedy_tokens(weights: Dict[str, torch.Tensor], cfg: dict, prompt: Sequence[int], tokens: Sequence[int],
                        margin: float) -> int:
  """Whether ``tokens`` are a greedy continuation of ``prompt``, by ONE pass over prompt + tokens:
  each token must be the arg-max of the logits at the position before it, or lie within ``margin`` of
  the largest logit there (a choice that rounding may turn).  If every token is the arg-max, this is
  what ``generate`` gives token by token, since equal prefixes give equal logits.  Returns how many
  tokens were the arg-max itself."""
  ids = list(prompt) + list(tokens)
  P, n = len(prompt), len(tokens)
  logits = forward(weights, cfg, ids[:-1], rows=range(P - 1, P - 1 + n))
  exact = 0
  for i, tok in enumerate(tokens):
    row = logits[i]
    best = int(row.argmax())
    if tok == best:
      exact += 1
      continue
    gap = float(row[best] - row[tok])
    assert gap <= margin, f"output token {i}: engine chose {tok} (logit {float(row[tok]):.5f}), plain chooses {best} ({float(row[best]):.5f}): gap {gap:.2e} > {margin:.1e}"
  return exact
