"""The step function: one batch of (request, its next tokens) through the model, from the cache.

``ModelRunner.step(items)`` runs exactly the tokens it is given - portions of prompts beside single
decode tokens, cut anywhere - as one batch, reading what earlier steps left in the cache, and
returns float32 logits at the places asked for.  It is the only forward pass of the package: the
scheduler's loop, the Python entry point, the benchmark and the trace-replay program all call it.

The reference has three entry modes (EXTEND, DECODE, MIXED: miniinfer/engine/model_runner.py:123-186,
miniinfer/scheduler/scheduler_batch.py:320-429) and returns the last row of every sequence
(miniinfer/models/fused_qwen3.py:317-342); here there is one mode and any set of rows.

Steps that hold only decode tokens can be replayed from a CUDA graph (``step_and_sample`` with
``use_graphs``): the same forward pass, captured once per batch-size bucket with the batch padded
by entries that read and write the dummy page (the reference captures decode at power-of-two batch
sizes as well, miniinfer/engine/cuda_graph_runner.py:121-131,289-381).  Such a step may take its
token ids from a device buffer - the tokens the step before has sampled - so that the host need not
have read them yet.  Any other step (a prompt portion, a mixed step) is recorded as a graph of its
own once its shape has been seen twice, and replayed when that shape comes again
(``_shape_step``); kernel by kernel a step is bound by the host's time per launch.

Recording a graph touches nothing of the live requests: the run that prepares the recording works on
a step of the same shape whose items all sit in the padding slot and the dummy page, and the real
step then runs once, as the first replay.  So a step's tokens pass through the model exactly once
whether or not it is the step that records, which mixers with per-request state updated in place
rely on.

What a part's kernels need per step beyond the common description - attention's lists of decode
items and prefill tiles, say - the part declares (``Part.step_work``); the step function knows no
part's tiling.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import KVCacheManager, OutOfPages
from ..kernels import ops
from ..models.spec import ModelSpec
from ..parts.base import HostStep, StepWork
from .context import StepContext, Workspace

GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
DECODE_GRAPHS_KEPT = 12     # graphs of decode-only steps that are kept (each holds buffers of its own, logits included)
STEP_GRAPHS_KEPT = 8        # graphs of steps other than decode-only ones (prompt portions, mixed steps) that are kept
STEP_GRAPH_AFTER = 2        # a step of a shape is recorded once that shape has been seen this many times ...
STEP_GRAPH_WINDOW = 64      # ... no more than this many steps apart: recording costs about twenty steps' worth of host
                            # time, which a shape that comes back once in a few hundred steps never repays


@dataclass
class StepItem:
  """The next tokens of one request and the places among them whose logits are wanted."""

  req_id: Hashable
  tokens: Sequence[int]
  want: Sequence[int] = field(default_factory=tuple)


def _pad4(n: int) -> int:
  return (n + 3) & ~3


class _MetaBuffers:
  """A pinned host array and its device twin; one copy moves a whole step's description."""

  def __init__(self, device: torch.device, capacity: int = 4096):
    self.device = device
    self.host: Optional[torch.Tensor] = None
    self.dev: Optional[torch.Tensor] = None
    self.copy_done = None
    self.bytes_copied = 0
    self._ensure(capacity)

  def _ensure(self, n: int) -> None:
    if self.host is None or self.host.numel() < n:
      cap = max(n, 4096)
      self.host = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
      self.dev = torch.empty(cap, dtype=torch.int32, device=self.device)

  def begin(self) -> np.ndarray:
    """The staging array, once the copy that last read it has finished."""
    if self.copy_done is not None:
      self.copy_done.synchronize()
    return self.host.numpy()

  def send(self, total: int) -> None:
    """One host-to-device copy of the first ``total`` words."""
    self.dev[:total].copy_(self.host[:total], non_blocking=True)
    if self.device.type == "cuda":
      if self.copy_done is None:
        self.copy_done = torch.cuda.Event()
      self.copy_done.record()
    self.bytes_copied = 4 * total

  @staticmethod
  def layout(arrays: "OrderedDict[str, np.ndarray]") -> Tuple[Dict[str, Tuple[int, int]], int]:
    offsets: Dict[str, Tuple[int, int]] = {}
    total = 0
    for name, arr in arrays.items():
      offsets[name] = (total, len(arr))
      total += _pad4(len(arr))
    return offsets, total

  def upload(self, arrays: "OrderedDict[str, np.ndarray]", fixed_capacity: bool = False) -> Dict[str, Tuple[int, int]]:
    offsets, total = self.layout(arrays)
    if fixed_capacity and total > self.host.numel():
      raise RuntimeError("step description is larger than the captured buffers")
    if total > self.host.numel():
      if self.copy_done is not None:
        self.copy_done.synchronize()
      self.copy_done = None
      self._ensure(total)
    h = self.begin()
    for name, arr in arrays.items():
      o, n = offsets[name]
      h[o:o + n] = arr
    self.send(total)
    return offsets


class _DecodeGraph:
  """A captured decode step for one batch-size bucket, with buffers of its own."""

  def __init__(self, bucket: int, device: torch.device):
    self.bucket = bucket
    self.meta = _MetaBuffers(device)
    self.ws = Workspace(device)
    self.graph = None
    self.ctx: Optional[StepContext] = None
    self.logits: Optional[torch.Tensor] = None
    self.tokens: Optional[torch.Tensor] = None
    self.launches = 0
    self.work_keys: Dict[str, tuple] = {}
    # the description of a step with no live entry (all padding) and where each array lies in it
    self.template: Optional[np.ndarray] = None
    self.offsets: Dict[str, Tuple[int, int]] = {}
    self.total = 0


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
    self.meta = _MetaBuffers(self.device)
    parts = spec.all_parts() if hasattr(spec, "all_parts") else []
    # sizes that a part's kernels cannot take are refused here, before any step
    for p in parts:
      p.validate(dtype)
    # the work lists the parts declare, one of each name
    self.work: "OrderedDict[str, StepWork]" = OrderedDict()
    for p in parts:
      for w in p.step_work():
        self.work.setdefault(w.name, w)
    # a part that reads the step on the host would have its decisions frozen into a recorded graph
    self.graphs_allowed = not any(getattr(p, "reads_step_on_host", False) for p in parts)
    self._graphs: "OrderedDict[tuple, _DecodeGraph]" = OrderedDict()
    # steps of any other kind, by shape (see _shape_key): how often seen, and the graphs of the repeated ones
    self._shape_seen: Dict[tuple, Tuple[int, int]] = {}      # shape -> (times seen, step it was last seen at)
    self._shape_steps = 0
    self._step_graphs: "OrderedDict[tuple, _DecodeGraph]" = OrderedDict()
    self.last_h2d_bytes = 0
    self.last_launches = 0

  # ------------------------------------------------------------------ reserving and describing a step

  def _check_and_reserve(self, items: Sequence[StepItem]) -> List[int]:
    """Checks the items, then makes room for their tokens in every cache group (all or nothing).
    Returns each request's length before the step."""
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
    need = [0] * len(cache.paged_groups)
    for it in items:
      for g, n in enumerate(cache.pages_needed(it.req_id, len(it.tokens))):
        need[g] += n
    for g, n in enumerate(need):
      if n > cache.paged_groups[g].allocator.num_free:
        raise OutOfPages(f"group {g}: the step needs {n} new pages, {cache.paged_groups[g].allocator.num_free} are free")
    starts = []
    for it in items:
      lo, hi = min(it.tokens), max(it.tokens)
      if lo < 0 or hi >= self.vocab_size:
        raise ValueError(f"token id outside the vocabulary of {self.vocab_size}")
      start = cache.length_of(it.req_id)
      if start + len(it.tokens) > self.max_position:
        raise ValueError(f"request {it.req_id!r} would reach position {start + len(it.tokens)}, "
                         f"beyond the limit of {self.max_position}")
      starts.append(start)
    for it in items:
      cache.append(it.req_id, len(it.tokens))
    return starts

  def _describe(self, items: Sequence[StepItem], starts: Sequence[int], extras: Optional[dict]
                ) -> "OrderedDict[str, np.ndarray]":
    """The step as int32 arrays, in the order they are laid out on the device."""
    cache = self.cache
    B = len(items)
    G = len(cache.paged_groups)
    q_len = np.array([len(it.tokens) for it in items], dtype=np.int32)
    T = int(q_len.sum())
    q_start = np.zeros(B, dtype=np.int32)
    q_start[1:] = np.cumsum(q_len)[:-1]
    start_np = np.array(starts, dtype=np.int32)
    a: "OrderedDict[str, np.ndarray]" = OrderedDict()
    a["ids"] = np.concatenate([np.asarray(it.tokens, dtype=np.int32) for it in items])
    a["positions"] = (np.arange(T, dtype=np.int32) - np.repeat(q_start, q_len) + np.repeat(start_np, q_len)).astype(np.int32)
    a["token_item"] = np.repeat(np.arange(B, dtype=np.int32), q_len)
    for g in range(G):
      a[f"slot_mapping{g}"] = np.concatenate(
        [cache.slot_mapping(it.req_id, g, s, len(it.tokens)) for it, s in zip(items, starts)])
    a["q_start"] = q_start
    a["q_len"] = q_len
    a["ctx_len"] = start_np + q_len
    a["seq_slot"] = np.array([cache.slot_of(it.req_id) for it in items], dtype=np.int32)
    a["logit_rows"] = np.array([q_start[b] + w for b, it in enumerate(items) for w in it.want], dtype=np.int32)
    host = HostStep(q_len, start_np, cache.max_model_len)
    for name, w in self.work.items():
      a[f"work:{name}"] = np.asarray(w.build(host), dtype=np.int32).reshape(-1)
    for k, v in (extras or {}).items():
      a[f"extra:{k}"] = np.asarray(v, dtype=np.int32)
    return a

  def _work_keys(self, q_len: np.ndarray, start: np.ndarray) -> Dict[str, tuple]:
    host = HostStep(q_len, start, self.cache.max_model_len)
    return {name: tuple(w.key(host)) for name, w in self.work.items()}

  def _context(self, a: "OrderedDict[str, np.ndarray]", offsets: Dict[str, Tuple[int, int]], dev: torch.Tensor,
               ws: Workspace, work_keys: Optional[Dict[str, tuple]] = None, captured: bool = False) -> StepContext:
    def view(name):
      o, n = offsets[name]
      return dev[o:o + n]

    cache = self.cache
    G = len(cache.paged_groups)
    ctx = StepContext(self.dtype, self.device, ws)
    ctx.num_tokens, ctx.num_items = len(a["ids"]), len(a["q_len"])
    ctx.ids, ctx.positions, ctx.token_item = view("ids"), view("positions"), view("token_item")
    ctx.q_start, ctx.q_len, ctx.ctx_len, ctx.seq_slot = view("q_start"), view("q_len"), view("ctx_len"), view("seq_slot")
    ctx.logit_rows = view("logit_rows")
    ctx.slot_mapping = [view(f"slot_mapping{g}") for g in range(G)]
    ctx.block_tables = [g.block_table for g in cache.paged_groups]
    ctx.host = {"q_len": a["q_len"].tolist(), "q_start": a["q_start"].tolist(),
                "start": (a["ctx_len"] - a["q_len"]).tolist(), "seq_slot": a["seq_slot"].tolist(),
                "logit_rows": a["logit_rows"].tolist()}
    ctx.extra = {k[len("extra:"):]: view(k) for k in a if k.startswith("extra:")}
    ctx.work = {k[len("work:"):]: view(k) for k in a if k.startswith("work:")}
    ctx.work_key = work_keys if work_keys is not None else self._work_keys(a["q_len"], a["ctx_len"] - a["q_len"])
    ctx.captured = captured
    return ctx

  def prepare(self, items: Sequence[StepItem], extras: Optional[dict] = None) -> StepContext:
    """Reserves cache room for the items' tokens and builds the step's device-side description
    with one host-to-device copy."""
    self._reserved_starts = self._check_and_reserve(items)
    return self._prepare_reserved(items, extras)

  def _prepare_reserved(self, items: Sequence[StepItem], extras: Optional[dict] = None) -> StepContext:
    starts = self._reserved_starts
    try:
      return self._prepare_described(items, starts, extras)
    except BaseException:
      self._finish(items, False)
      raise

  def _prepare_described(self, items, starts, extras) -> StepContext:
    arrays = self._describe(items, starts, extras)
    offsets = self.meta.upload(arrays)
    self.last_h2d_bytes = self.meta.bytes_copied
    self.cache.sync()
    return self._context(arrays, offsets, self.meta.dev, self.ws)

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

  def _finish(self, items: Sequence[StepItem], ok: bool) -> None:
    for it in items:
      if ok:
        self.cache.commit(it.req_id, len(it.tokens))
      else:
        self.cache.cancel(it.req_id, len(it.tokens))

  # ------------------------------------------------------------------ steps of a repeated shape, from CUDA graphs

  def _shape_key(self, items: Sequence[StepItem], starts: Sequence[int], sampled: bool) -> Tuple[tuple, Dict[str, tuple]]:
    """What the launches of a step depend on: the counts of tokens, items and wanted rows, whether
    the sampler runs, and the keys of the work lists that the parts declare (for attention: the
    numbers of decode items and prefill tiles and the class of the longest decode context, which
    sizes the split-KV grid).  Everything else about the step is in the description on the device."""
    q_len = np.array([len(it.tokens) for it in items], dtype=np.int32)
    keys = self._work_keys(q_len, np.array(starts, dtype=np.int32))
    R = sum(len(it.want) for it in items)
    return (int(q_len.sum()), len(items), R, sampled) + tuple(keys.values()), keys

  def _shape_step(self, items: Sequence[StepItem], extras: Optional[dict], sample_fn) -> Optional[_DecodeGraph]:
    """Runs the step from a CUDA graph if a step of its shape has been recorded, records it if the
    shape has been seen often enough; returns the graph (logits and tokens in its buffers), or None
    if the step is to run kernel by kernel.  The items' cache room is reserved on return either way;
    a returned graph means the step has run and is committed."""
    starts = self._check_and_reserve(items)
    self._reserved_starts = starts
    self._shape_steps += 1
    if not (self.graphs_allowed and self.device.type == "cuda"):
      return None
    key, work_keys = self._shape_key(items, starts, sample_fn is not None)
    g = self._step_graphs.get(key)
    if g is None:
      seen, last = self._shape_seen.get(key, (0, 0))
      seen = seen + 1 if seen and self._shape_steps - last <= STEP_GRAPH_WINDOW else 1
      if len(self._shape_seen) > 4096:
        self._shape_seen.clear()
      self._shape_seen[key] = (seen, self._shape_steps)
      if seen < STEP_GRAPH_AFTER:
        return None
    try:
      arrays = self._describe(items, starts, extras)
      if g is None:
        g = _DecodeGraph(len(items), self.device)
        g.work_keys = work_keys
        g.offsets, g.total = g.meta.layout(arrays)
        self.cache.sync()
        self._capture(g, arrays, g.offsets, sample_fn, rows=key[2])
        self._step_graphs[key] = g
        while len(self._step_graphs) > STEP_GRAPHS_KEPT:
          self._step_graphs.popitem(last=False)
      else:
        self._step_graphs.move_to_end(key)
      offsets = g.meta.upload(arrays, fixed_capacity=True)
      if offsets != g.offsets:
        raise RuntimeError("a step's description does not have the layout its shape was recorded with")
      self.cache.sync()
      self.last_h2d_bytes = g.meta.bytes_copied
      g.graph.replay()
      self.last_launches = g.launches
    except BaseException:
      self._finish(items, False)
      raise
    self._finish(items, True)
    return g

  @torch.no_grad()
  def step(self, items: Sequence[StepItem], extras: Optional[dict] = None, return_ctx: bool = False,
           use_graphs: bool = True):
    """Runs one step; returns the float32 logits of the wanted rows.  A step whose shape repeats is
    replayed from a CUDA graph; its logits then live in a buffer that the next step of the same
    shape overwrites."""
    if use_graphs and not return_ctx:
      g = self._shape_step(items, extras, None)
      if g is not None:
        return g.logits
      ctx = self._prepare_reserved(items, extras)
    else:
      ctx = self.prepare(items, extras)
    before = ops.launch_count()
    try:
      logits = self.forward(ctx)
    except BaseException:
      self._finish(items, False)
      raise
    self._finish(items, True)
    self.last_launches = ops.launch_count() - before
    return (logits, ctx) if return_ctx else logits

  # ------------------------------------------------------------------ sampling steps, with CUDA graphs for decode

  @torch.no_grad()
  def graph_decode_bucket(self, items: Sequence[StepItem]) -> Optional[int]:
    """The batch-size bucket whose CUDA graph runs this step, if it is a step of decode tokens only,
    each wanting its one row; else None."""
    if not (self.graphs_allowed and self.device.type == "cuda"):
      return None
    if not all(len(it.tokens) == 1 and tuple(it.want) == (0,) for it in items):
      return None
    return next((b for b in GRAPH_BUCKETS if b >= len(items)), None)

  def step_and_sample(self, items: Sequence[StepItem], sampling: Dict[str, np.ndarray],
                      sample_fn: Callable[..., None],
                      tokens_out: torch.Tensor, use_graphs: bool = True,
                      ids_on_device: Optional[torch.Tensor] = None,
                      sampling_pad: Optional[Dict[str, np.ndarray]] = None) -> torch.Tensor:
    """Runs the step and samples one token for each wanted row into ``tokens_out`` (int32, device).
    ``sampling``: packed per-row options (``Sampler.pack``).  ``sampling_pad``: for each option the
    words of a row that samples harmlessly, for the padding rows of a captured decode step (default:
    zero words).  Returns the tokens' device view.
    A step of decode tokens only, each wanting its one row, is replayed from a CUDA graph; for such
    a step ``ids_on_device`` (int32, one per item) may give the tokens instead of the items: the
    tokens a step before has sampled and the host has not read yet."""
    R = sum(len(it.want) for it in items)
    bucket = self.graph_decode_bucket(items) if use_graphs else None
    if ids_on_device is not None and bucket is None:
      raise ValueError("tokens on the device are taken by graph decode steps only")
    if bucket is not None:
      return self._graph_step(items, sampling, sample_fn, tokens_out, bucket, ids_on_device, sampling_pad)
    if use_graphs and R:
      g = self._shape_step(items, sampling, sample_fn)      # a step of a repeated shape: forward pass and sampler from one graph
      if g is not None:
        return g.tokens[:R]
      ctx = self._prepare_reserved(items, sampling)
    else:
      ctx = self.prepare(items, sampling)
    before = ops.launch_count()
    try:
      logits = self.forward(ctx)
      if R:
        sample_fn(logits, ctx.extra, tokens_out[:R], self.ws)
    except BaseException:
      self._finish(items, False)
      raise
    self._finish(items, True)
    self.last_launches = ops.launch_count() - before
    return tokens_out[:R]

  def _padded(self, a: "OrderedDict[str, np.ndarray]", bucket: int, sampling_pad: Optional[Dict[str, np.ndarray]] = None
              ) -> "OrderedDict[str, np.ndarray]":
    """Fills a decode-only description up to ``bucket`` entries.  The extra entries belong to the
    padding slot, whose block table points at the dummy page: they read one key there and write
    there; their state rows are the padding slot's.  Work lists are made anew for the padded step;
    the sampler's options get the rows their owner declared harmless (zero words otherwise)."""
    B = len(a["q_len"])
    n = bucket - B

    def pad(arr, value, count=n):
      return np.concatenate([arr, np.full(count, value, dtype=np.int32)])

    out: "OrderedDict[str, np.ndarray]" = OrderedDict()
    for k, v in a.items():
      if k in ("ids", "positions") or k.startswith("slot_mapping"):
        out[k] = pad(v, 0)
      elif k in ("token_item", "q_start", "logit_rows"):
        out[k] = np.arange(bucket, dtype=np.int32)
      elif k in ("q_len", "ctx_len"):
        out[k] = pad(v, 1)
      elif k == "seq_slot":
        out[k] = pad(v, self.cache.pad_slot)
      elif k.startswith("work:"):
        out[k] = v                                  # replaced below, once the padded numbers are known
      elif k.startswith("extra:"):
        width = len(v) // B if B else None          # words per row
        row = (sampling_pad or {}).get(k[len("extra:"):])
        if row is None:
          row = np.zeros(width if width is not None else 1, dtype=np.int32)
        out[k] = np.concatenate([v, np.tile(np.asarray(row, dtype=np.int32), n)])
      else:
        raise KeyError(k)
    host = HostStep(out["q_len"], out["ctx_len"] - out["q_len"], self.cache.max_model_len)
    for name, w in self.work.items():
      out[f"work:{name}"] = np.asarray(w.build(host), dtype=np.int32).reshape(-1)
    return out

  def _graph_step(self, items, sampling, sample_fn, tokens_out, bucket: int, ids_on_device=None, sampling_pad=None) -> torch.Tensor:
    starts = self._check_and_reserve(items)
    self._shape_steps += 1
    B = len(items)
    try:
      # what the captured launches depend on (for attention: the split-KV grid, sized from the class of the
      # longest context) is part of the graph's identity: one graph per (bucket, keys of the work lists)
      q_len = np.ones(bucket, dtype=np.int32)
      start_np = np.zeros(bucket, dtype=np.int32)
      start_np[:B] = starts
      work_keys = self._work_keys(q_len, start_np)
      key = (bucket,) + tuple(work_keys.values())
      g = self._graphs.get(key)
      if g is None:
        g = self._graphs[key] = _DecodeGraph(bucket, self.device)
        g.work_keys = work_keys
        while len(self._graphs) > DECODE_GRAPHS_KEPT:
          self._graphs.popitem(last=False)          # the least recently used graph goes, with its buffers
      else:
        self._graphs.move_to_end(key)
      if g.graph is None:
        described = self._describe(items, starts, sampling)
        arrays = self._decode_layout(g, described, sampling_pad)
        self.cache.sync()
        self._capture(g, arrays, g.offsets, sample_fn)
        g.meta.upload(arrays, fixed_capacity=True)
      else:
        self._fill_decode(g, items, starts, sampling, q_len, start_np)
        self.cache.sync()
      self.last_h2d_bytes = g.meta.bytes_copied
      if ids_on_device is not None:
        # after the upload, before the replay, in stream order: the tokens go from where the step
        # before left them (possibly this graph's own token buffer) into this step's description
        o, _ = g.offsets["ids"]
        g.meta.dev[o:o + B].copy_(ids_on_device[:B], non_blocking=True)
      g.graph.replay()
      self.last_launches = g.launches
    except BaseException:
      self._finish(items, False)
      raise
    self._finish(items, True)
    return g.tokens[:B]

  def _decode_layout(self, g: _DecodeGraph, described: "OrderedDict[str, np.ndarray]", sampling_pad=None
                     ) -> "OrderedDict[str, np.ndarray]":
    """Fixes where each array of a decode-only step lies in the graph's buffers and keeps the
    description of a step without live entries; returns ``described`` padded to the bucket."""
    arrays = self._padded(described, g.bucket, sampling_pad)
    B = len(described["q_len"])
    widths = {k: len(v) // B for k, v in described.items() if k.startswith("extra:")}
    empty_in = OrderedDict((k, v[:0]) for k, v in described.items())
    pad_rows = {k[len("extra:"):]: np.asarray((sampling_pad or {}).get(k[len("extra:"):], np.zeros(w, dtype=np.int32)), dtype=np.int32)
                for k, w in widths.items()}
    empty = self._padded(empty_in, g.bucket, pad_rows)
    g.offsets, g.total = g.meta.layout(arrays)
    g.template = np.zeros(g.total, dtype=np.int32)
    for k, v in empty.items():
      o, n = g.offsets[k]
      g.template[o:o + n] = v
    return arrays

  def _fill_decode(self, g: _DecodeGraph, items, starts, sampling, q_len: np.ndarray, start_np: np.ndarray) -> None:
    """A decode-only step written straight into the graph's staging array: the entries that differ
    from step to step (token, position, cache slot, length, request slot, sampling options) over the
    all-padding description.  Gives the same words as ``_padded(_describe(...))``."""
    cache = self.cache
    B = len(items)
    h = g.meta.begin()
    h[:g.total] = g.template
    off = g.offsets

    def put(name, values):
      o, n = off[name]
      if len(values) > n:
        raise RuntimeError("step description is larger than the captured buffers")
      h[o:o + len(values)] = values

    put("ids", [it.tokens[0] for it in items])
    put("positions", starts)
    put("ctx_len", [s + 1 for s in starts])
    put("seq_slot", [cache.slot_of(it.req_id) for it in items])
    for gi in range(len(cache.paged_groups)):
      put(f"slot_mapping{gi}", [cache.slot_at(it.req_id, gi, s) for it, s in zip(items, starts)])
    for k, v in sampling.items():
      put(f"extra:{k}", v if v.dtype == np.int32 else v.view(np.int32))
    for name, w in self.work.items():
      if w.per_step:          # a list that depends on more than the bucket is made anew from the padded step's numbers
        put(f"work:{name}", np.asarray(w.build(HostStep(q_len, start_np, cache.max_model_len)), dtype=np.int32).reshape(-1))
    g.meta.send(g.total)

  def _neutral(self, arrays: "OrderedDict[str, np.ndarray]") -> "OrderedDict[str, np.ndarray]":
    """A step of the same shape that belongs to nobody: every item sits in the padding slot (whose
    block table points at the dummy page and whose state rows are scratch), every token is token 0
    and is stored in the dummy page.  Lengths, positions and work lists stay, so the same kernels
    run with the same grids."""
    out: "OrderedDict[str, np.ndarray]" = OrderedDict()
    for k, v in arrays.items():
      if k == "ids" or k.startswith("slot_mapping"):
        out[k] = np.zeros_like(v)
      elif k == "seq_slot":
        out[k] = np.full_like(v, self.cache.pad_slot)
      else:
        out[k] = v
    return out

  def _capture(self, g: _DecodeGraph, arrays, offsets, sample_fn, rows: Optional[int] = None) -> None:
    """Records forward pass (and sampler, if given) over the graph's own buffers.  ``rows``: sampled
    rows (default: one per entry of the bucket).

    Nothing of the live requests is touched: the run that sizes the workspace, configures the kernels
    and makes the libraries load what they will launch (nothing may be loaded while a graph is
    recorded) works on a step of the same shape in the padding slot and the dummy page.  The caller
    uploads the real description afterwards and replays the graph once, so the step's tokens pass
    through the model exactly once - which a mixer that updates per-request state in place needs."""
    g.meta.upload(self._neutral(arrays))
    g.ctx = self._context(arrays, offsets, g.meta.dev, g.ws, work_keys=g.work_keys, captured=True)
    g.tokens = torch.zeros(max(g.bucket if rows is None else rows, 1), dtype=torch.int32, device=self.device)

    def run():
      g.ctx.shared.clear()
      g.logits = self.forward(g.ctx)
      if sample_fn is not None and g.logits.shape[0] > 0:
        sample_fn(g.logits, g.ctx.extra, g.tokens[:g.logits.shape[0]], g.ws)

    with ops.recording_graph():
      run()                                  # takes the same paths as the recording
      torch.cuda.current_stream().synchronize()
      g.ws.frozen = True
      before = ops.launch_count()
      graph = torch.cuda.CUDAGraph()
      with torch.cuda.graph(graph):
        run()
    g.launches = ops.launch_count() - before
    g.graph = graph

  def check_status(self) -> None:
    """Raises if a bounded wait inside a kernel ran out since the buffers were made (the step's
    results are then not to be trusted).  Reads a few words from the device."""
    for ws in [self.ws] + [g.ws for g in self._graphs.values()] + [g.ws for g in self._step_graphs.values()]:
      code = ops.device_status(ws)
      if code:
        raise ops.KernelError(f"a bounded wait inside a kernel ran out (status bits {code}: 1 decode attention, "
                              f"2 prefill attention, 4 the tcgen05 matrix product)")

  def num_graphs(self) -> int:
    return sum(1 for g in list(self._graphs.values()) + list(self._step_graphs.values()) if g.graph is not None)
