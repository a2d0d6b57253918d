"""Grouped-query attention over the paged cache as a mixer part.

Order of the computation as in the reference (miniinfer/models/fused_qwen3.py:95-108): fused QKV
projection without bias; per-head RMSNorm of q and k (optional here); rotary encoding (from the
position-encoding part, optional here); k and v into the cache; attention with
``scale`` over the keys a token may see (all earlier ones, or the last ``window``); output
projection.  Head counts, head size, scale, eps and window are constructor arguments.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.specs import CacheSpec, PagedKVSpec
from ..kernels import ops
from .base import Mixer, ParamSpec, Piece, PositionEncoding, whole


class AttentionMixer(Mixer):
  def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
               scale: float, qk_norm_eps: Optional[float], position: Optional[PositionEncoding],
               window: Optional[int] = None):
    super().__init__(name)
    if num_heads % num_kv_heads:
      raise ValueError("num_heads must be a multiple of num_kv_heads")
    self.hidden_size = hidden_size
    self.num_heads = num_heads
    self.num_kv_heads = num_kv_heads
    self.head_dim = head_dim
    self.scale = float(scale)
    self.qk_norm_eps = qk_norm_eps
    self.position = position
    self.window = window

  def cache_spec(self) -> Optional[CacheSpec]:
    return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

  def param_specs(self) -> Dict[str, ParamSpec]:
    H, nh, nkv, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
    n = self.name
    specs = {
      "qkv": ParamSpec(((nh + 2 * nkv) * hd, H), "matrix", [
        [Piece(f"{n}.q_proj.weight", 0, (nh * hd, H)), Piece(f"{n}.k_proj.weight", nh * hd, (nkv * hd, H)),
         Piece(f"{n}.v_proj.weight", (nh + nkv) * hd, (nkv * hd, H))],
        whole(f"{n}.qkv_proj.weight", ((nh + 2 * nkv) * hd, H)),
      ]),
      "o": ParamSpec((H, nh * hd), "matrix", [whole(f"{n}.o_proj.weight", (H, nh * hd))]),
    }
    if self.qk_norm_eps is not None:
      specs["q_norm"] = ParamSpec((hd,), "vector", [whole(f"{n}.q_norm.weight", (hd,))], init="ones_noise")
      specs["k_norm"] = ParamSpec((hd,), "vector", [whole(f"{n}.k_norm.weight", (hd,))], init="ones_noise")
    return specs

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
    if cache.kind != "paged":
      raise RuntimeError(f"{self.name}: attention needs a paged cache, got {cache.kind!r}")
    qkv = ctx.ws.buffer("qkv", (T, (nh + 2 * nkv) * hd), ctx.dtype)
    ops.linear(qkv, x, self.qkv)
    table = self.position.rotary_table() if self.position is not None else None
    qn = self.q_norm if self.qk_norm_eps is not None else None
    kn = self.k_norm if self.qk_norm_eps is not None else None
    ops.qk_norm_rope_store(qkv, qn, kn, table, ctx.positions,
                           ctx.slot_mapping[cache.group] if cache.writes else None,
                           cache.tensor if cache.writes else None, nh, nkv, hd,
                           self.qk_norm_eps if self.qk_norm_eps is not None else 1.0)
    attn = ctx.ws.buffer("attn_out", (T, nh * hd), ctx.dtype)
    ops.attention(attn, qkv, cache.tensor, ctx.block_tables[cache.group], ctx.attn, nh, nkv, hd,
                  self.scale, self.window)
    out = ctx.ws.buffer("mixer_out", (T, self.hidden_size), ctx.dtype)
    ops.linear(out, attn, self.o)
    return out
