"""The step function: one batch of (request, its next tokens) through the model, from the cache.

``ModelRunner.step(items)`` runs exactly the tokens it is given - portions of prompts beside single
decode tokens, cut anywhere - as one batch, reading what earlier steps left in the cache, and
returns float32 logits at the places asked for.  It is the only forward pass of the package: the
scheduler's loop, the Python entry point, the benchmark and the trace-replay program all call it.

The reference has three entry modes (EXTEND, DECODE, MIXED: miniinfer/engine/model_runner.py:123-186,
miniinfer/scheduler/scheduler_batch.py:320-429) and returns the last row of every sequence
(miniinfer/models/fused_qwen3.py:317-342); here there is one mode and any set of rows.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import KVCacheManager, OutOfPages
from ..kernels.ops import AttentionBatch
from ..models.spec import ModelSpec
from .context import StepContext, Workspace

PREFILL_TILE = 64   # query rows of one prefill-attention tile


@dataclass
class StepItem:
  """The next tokens of one request and the places among them whose logits are wanted."""

  req_id: Hashable
  tokens: Sequence[int]
  want: Sequence[int] = field(default_factory=tuple)


def _pad4(n: int) -> int:
  return (n + 3) & ~3


class ModelRunner:
  def __init__(self, spec: ModelSpec, cache: KVCacheManager, dtype: torch.dtype, device):
    self.spec = spec
    self.cache = cache
    self.dtype = dtype
    self.device = torch.device(device)
    self.vocab_size = spec.config.vocab_size
    self.ws = Workspace(self.device)
    for pe in spec.position_encodings:
      pe.prepare(self.device, cache.max_model_len)
    limits = [pe.max_positions() for pe in spec.position_encodings if pe.max_positions() is not None]
    self.max_position = min([cache.max_model_len] + limits)
    self.layer_caches = []
    for i, run in enumerate(spec.run_list):
      if run.cache_of is None:
        self.layer_caches.append(cache.layer_cache(i, writes=True))
      else:
        self.layer_caches.append(cache.layer_cache(run.cache_of, writes=False))
    self._meta_host: Optional[torch.Tensor] = None
    self._meta_dev: Optional[torch.Tensor] = None
    self._copy_done = None

  # ------------------------------------------------------------------ metadata

  def _meta_buffers(self, n: int):
    if self._meta_host is None or self._meta_host.numel() < n:
      cap = max(n, 4096)
      pin = self.device.type == "cuda"
      self._meta_host = torch.empty(cap, dtype=torch.int32, pin_memory=pin)
      self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
    return self._meta_host, self._meta_dev

  def prepare(self, items: Sequence[StepItem], extras: Optional[dict] = None) -> StepContext:
    """Reserves cache room for the items' tokens and builds the step's device-side description
    with one host-to-device copy."""
    cache = self.cache
    if not items:
      raise ValueError("a step needs at least one item")
    seen = set()
    for it in items:
      if it.req_id in seen:
        raise ValueError(f"request {it.req_id!r} appears twice in one step")
      seen.add(it.req_id)
      if len(it.tokens) < 1:
        raise ValueError(f"request {it.req_id!r} brings no tokens")
      for w in it.want:
        if not (0 <= w < len(it.tokens)):
          raise ValueError(f"request {it.req_id!r}: wanted place {w} is outside its {len(it.tokens)} tokens")
    # all or nothing: the pages of every group must cover the whole step
    need = [0] * len(cache.paged_groups)
    for it in items:
      for g, n in enumerate(cache.pages_needed(it.req_id, len(it.tokens))):
        need[g] += n
    for g, n in enumerate(need):
      if n > cache.paged_groups[g].allocator.num_free:
        raise OutOfPages(f"group {g}: the step needs {n} new pages, {cache.paged_groups[g].allocator.num_free} are free")
    ids = np.concatenate([np.asarray(it.tokens, dtype=np.int64) for it in items])
    if ids.min() < 0 or ids.max() >= self.vocab_size:
      raise ValueError(f"token id outside the vocabulary of {self.vocab_size}")
    starts = []
    for it in items:
      start = cache.length_of(it.req_id)
      if start + len(it.tokens) > self.max_position:
        raise ValueError(f"request {it.req_id!r} would reach position {start + len(it.tokens)}, "
                         f"beyond the limit of {self.max_position}")
      starts.append(start)
    for it in items:
      cache.append(it.req_id, len(it.tokens))

    B = len(items)
    T = sum(len(it.tokens) for it in items)
    R = sum(len(it.want) for it in items)
    G = len(cache.paged_groups)
    q_len = np.array([len(it.tokens) for it in items], dtype=np.int32)
    q_start = np.zeros(B, dtype=np.int32)
    q_start[1:] = np.cumsum(q_len)[:-1]
    start_np = np.array(starts, dtype=np.int32)
    token_item = np.repeat(np.arange(B, dtype=np.int32), q_len)
    positions = (np.arange(T, dtype=np.int32) - np.repeat(q_start, q_len) + np.repeat(start_np, q_len)).astype(np.int32)
    seq_slot = np.array([cache.slot_of(it.req_id) for it in items], dtype=np.int32)
    rows = np.array([q_start[b] + w for b, it in enumerate(items) for w in it.want], dtype=np.int32)
    pre_tiles = [(b, o) for b in range(B) if q_len[b] > 1 for o in range(0, int(q_len[b]), PREFILL_TILE)]
    dec_items = [b for b in range(B) if q_len[b] == 1]

    sizes = [("ids", T), ("positions", T), ("token_item", T)]
    sizes += [(f"slot_mapping{g}", T) for g in range(G)]
    sizes += [("q_start", B), ("q_len", B), ("ctx_len", B), ("seq_slot", B), ("logit_rows", R),
              ("decode_items", len(dec_items)), ("prefill_tiles", 2 * len(pre_tiles))]
    extras = extras or {}
    sizes += [(f"extra:{k}", len(v)) for k, v in extras.items()]
    offsets = {}
    total = 0
    for name, n in sizes:
      offsets[name] = (total, n)
      total += _pad4(n)
    host, dev = self._meta_buffers(total)
    if self._copy_done is not None:
      self._copy_done.synchronize()    # the staging buffer may still be feeding the previous copy
    h = host.numpy()

    def put(name, arr):
      o, n = offsets[name]
      h[o:o + n] = arr

    put("ids", ids.astype(np.int32))
    put("positions", positions)
    put("token_item", token_item)
    for g in range(G):
      put(f"slot_mapping{g}", np.concatenate(
        [cache.slot_mapping(it.req_id, g, s, len(it.tokens)) for it, s in zip(items, starts)]))
    put("q_start", q_start)
    put("q_len", q_len)
    put("ctx_len", start_np + q_len)
    put("seq_slot", seq_slot)
    put("logit_rows", rows)
    put("decode_items", np.array(dec_items, dtype=np.int32))
    put("prefill_tiles", np.array(pre_tiles, dtype=np.int32).reshape(-1))
    for k, v in extras.items():
      put(f"extra:{k}", v)
    dev[:total].copy_(host[:total], non_blocking=True)
    if self.device.type == "cuda":
      self._copy_done = torch.cuda.Event()
      self._copy_done.record()
    cache.sync()

    def view(name):
      o, n = offsets[name]
      return dev[o:o + n]

    ctx = StepContext(self.dtype, self.device, self.ws)
    ctx.num_tokens, ctx.num_items = T, B
    ctx.ids, ctx.positions, ctx.token_item = view("ids"), view("positions"), view("token_item")
    ctx.q_start, ctx.q_len, ctx.ctx_len, ctx.seq_slot = view("q_start"), view("q_len"), view("ctx_len"), view("seq_slot")
    ctx.logit_rows = view("logit_rows")
    ctx.slot_mapping = [view(f"slot_mapping{g}") for g in range(G)]
    ctx.block_tables = [g.block_table for g in cache.paged_groups]
    ctx.host = {"q_len": q_len.tolist(), "q_start": q_start.tolist(), "start": starts,
                "seq_slot": seq_slot.tolist(), "logit_rows": rows.tolist()}
    ctx.extra = {k: view(f"extra:{k}") for k in extras}
    ctx.attn = AttentionBatch(
      token_item=ctx.token_item, positions=ctx.positions, seq_slot=ctx.seq_slot, q_start=ctx.q_start,
      q_len=ctx.q_len, ctx_len=ctx.ctx_len, num_tokens=T, num_items=B,
      prefill_tiles=view("prefill_tiles").view(-1, 2), num_prefill_tiles=len(pre_tiles),
      decode_items=view("decode_items"), num_decode=len(dec_items),
      max_ctx_len=int((start_np + q_len).max()), scratch=self.ws)
    return ctx

  # ------------------------------------------------------------------ the forward pass

  def forward(self, ctx: StepContext) -> torch.Tensor:
    """Runs the layers in run-list order; returns logits [wanted rows, vocab] in float32."""
    spec = self.spec
    resid = spec.embedding.forward(ctx.ids, ctx)
    for pe in spec.position_encodings:
      pe.apply_to_hidden(resid, ctx)
    pending = None
    for run, layer_cache in zip(spec.run_list, self.layer_caches):
      pending = spec.blocks[run.block].forward(resid, pending, ctx, layer_cache)
    if ctx.logit_rows.shape[0] == 0:
      return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
    x = spec.final_norm.norm_rows(resid, pending, ctx.logit_rows, ctx)
    return spec.lm_head.forward(x, ctx)

  @torch.no_grad()
  def step(self, items: Sequence[StepItem], extras: Optional[dict] = None, return_ctx: bool = False):
    ctx = self.prepare(items, extras)
    try:
      logits = self.forward(ctx)
    except BaseException:
      for it in items:
        self.cache.cancel(it.req_id, len(it.tokens))
      raise
    for it in items:
      self.cache.commit(it.req_id, len(it.tokens))
    return (logits, ctx) if return_ctx else logits
