"""Grouped-query attention over the paged cache as a mixer part.

Order of the computation as in the reference (miniinfer/models/fused_qwen3.py:95-108): fused QKV
projection without bias; per-head RMSNorm of q and k (optional here); rotary encoding (from the
position-encoding part, optional here); k and v into the cache; attention with
``scale`` over the keys a token may see (all earlier ones, or the last ``window``); output
projection.  Head counts, head size, scale, eps and window are constructor arguments.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..cache.specs import CacheSpec, PagedKVSpec
from ..kernels import ops
from ..kernels.ops import AttentionBatch
from .base import HostStep, Mixer, ParamSpec, Piece, PositionEncoding, StepWork, whole

DECODE_CONTEXT_STEP = 1024   # the split-KV grid of a step is sized for its longest context rounded up to this


class DecodeItems(StepWork):
  """The items that bring one token: the split-KV decode kernel works through these.  Its grid is
  sized from their number and from a bound on their context lengths, so both are the list's key."""

  name = "attention_decode_items"

  def build(self, step: HostStep) -> np.ndarray:
    return step.decode_items()

  def key(self, step: HostStep) -> tuple:
    return (int((step.q_len == 1).sum()), step.context_class(step.longest_decode_context(), DECODE_CONTEXT_STEP))


class PrefillTiles(StepWork):
  """(item, first row) of every tile of ``ops.PREFILL_TILE`` query rows of the items that bring
  several tokens: one block of the prefill attention kernel per tile and head."""

  name = "attention_prefill_tiles"
  tile = ops.PREFILL_TILE

  def build(self, step: HostStep) -> np.ndarray:
    pairs = [(b, o) for b in np.flatnonzero(step.q_len > 1) for o in range(0, int(step.q_len[b]), self.tile)]
    return np.array(pairs, dtype=np.int32).reshape(-1)

  def key(self, step: HostStep) -> tuple:
    n = step.q_len[step.q_len > 1]
    return (int((-(-n // self.tile)).sum()),)


class PrefillWideTiles(PrefillTiles):
  """The same in steps of ``ops.PREFILL_WIDE_TILE`` rows: the works of the tcgen05 prefill kernel when a block, or each
  block of a pair, takes 128 tokens of one head."""

  name = "attention_prefill_wide_tiles"
  tile = ops.PREFILL_WIDE_TILE


_WORK = [DecodeItems(), PrefillTiles(), PrefillWideTiles()]


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

  def validate(self, dtype: torch.dtype) -> None:
    hd, H = self.head_dim, self.hidden_size
    if hd % 4 or not (4 <= hd <= 256):
      raise ValueError(f"{self.name}: head_dim={hd} is not supported: the attention kernels take multiples of 4 up to 256 "
                       f"(multiples of 16 run on the tensor cores in bfloat16)")
    if dtype == torch.bfloat16:
      for what, k in (("hidden_size", H), ("num_attention_heads * head_dim", self.num_heads * hd),
                      ("(num_attention_heads + 2 * num_key_value_heads) * head_dim", (self.num_heads + 2 * self.num_kv_heads) * hd)):
        if k % 8:
          raise ValueError(f"{self.name}: {what}={k} must be a multiple of 8 in bfloat16 (rows are read 16 bytes at a time)")
    rotary = getattr(self.position, "rotary_dim", None)
    if rotary is not None and rotary > hd:
      raise ValueError(f"{self.name}: the rotary encoding covers {rotary} values, more than head_dim={hd}")

  def step_work(self) -> List[StepWork]:
    return _WORK

  @staticmethod
  def _batch(ctx) -> AttentionBatch:
    """The step as the attention kernels take it; made once per step and shared by all layers."""
    batch = ctx.shared.get("attention_batch")
    if batch is None:
      dec, tiles, wide = ctx.work[DecodeItems.name], ctx.work[PrefillTiles.name], ctx.work[PrefillWideTiles.name]
      batch = AttentionBatch(
        token_item=ctx.token_item, positions=ctx.positions, seq_slot=ctx.seq_slot, q_start=ctx.q_start, q_len=ctx.q_len,
        ctx_len=ctx.ctx_len, num_tokens=ctx.num_tokens, num_items=ctx.num_items,
        prefill_tiles=tiles.view(-1, 2), num_prefill_tiles=tiles.shape[0] // 2,
        prefill_wide_tiles=wide.view(-1, 2), num_prefill_wide_tiles=wide.shape[0] // 2, decode_items=dec, num_decode=dec.shape[0],
        max_ctx_len=max(1, ctx.work_key[DecodeItems.name][1]), scratch=ctx.ws)
      ctx.shared["attention_batch"] = batch
    return batch

  def takes_residual(self, norm, ctx) -> bool:
    return norm.as_rms() is not None and ops.fuses_few_rows(ctx.num_tokens, ctx.dtype)

  def forward_on_residual(self, resid: torch.Tensor, norm, ctx, cache) -> None:
    """The norm in the QKV product's prologue, the residual add in the output product's epilogue."""
    weight, eps = norm.as_rms()
    nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
    qkv = ctx.ws.buffer("qkv", (resid.shape[0], (nh + 2 * nkv) * hd), ctx.dtype)
    ops.linear_normed(qkv, resid, weight, eps, self.qkv)
    attn = self._attend(qkv, ctx, cache)
    ops.linear_add(resid, attn, self.o)

  def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
    T = x.shape[0]
    nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
    qkv = ctx.ws.buffer("qkv", (T, (nh + 2 * nkv) * hd), ctx.dtype)
    ops.linear(qkv, x, self.qkv)
    attn = self._attend(qkv, ctx, cache)
    out = ctx.ws.buffer("mixer_out", (T, self.hidden_size), ctx.dtype)
    ops.linear(out, attn, self.o)
    return out

  def _attend(self, qkv: torch.Tensor, ctx, cache) -> torch.Tensor:
    """From the fused QKV rows to the attention output rows: QK norm, rotation, cache store, attention."""
    T = qkv.shape[0]
    nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
    if cache.kind != "paged":
      raise RuntimeError(f"{self.name}: attention needs a paged cache, got {cache.kind!r}")
    table = self.position.rotary_table() if self.position is not None else None
    qn = self.q_norm if self.qk_norm_eps is not None else None
    kn = self.k_norm if self.qk_norm_eps is not None else None
    attn = ctx.ws.buffer("attn_out", (T, nh * hd), ctx.dtype)
    ops.rope_store_attention(attn, qkv, qn, kn, table, ctx.positions, ctx.slot_mapping[cache.group], cache.tensor,
                             cache.writes, ctx.block_tables[cache.group], self._batch(ctx), nh, nkv, hd,
                             self.qk_norm_eps if self.qk_norm_eps is not None else 1.0, self.scale, self.window)
    return attn
