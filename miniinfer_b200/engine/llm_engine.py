"""The Python entry point: ``LLMEngine(model, **options).generate(prompts, sampling_params)``.

Names follow the reference (miniinfer/engine/llm_engine.py): ``LLMEngine(model, **kwargs)`` :87,
``generate(prompts, sampling_params, use_tqdm)`` :898 returning a list of
``{"text", "token_ids", "request_id"}`` ordered by request :966-1015, ``add_request`` :1309,
``step`` :465, ``is_finished`` :1271, ``start``/``stop`` and use as a context manager :1301-1306.
Prompts are lists of token ids, or strings when the model folder has a ``tokenizer.json``.
One process, one GPU; no server, no worker processes.
"""

from __future__ import annotations

import os
import queue
import threading
import time
from dataclasses import dataclass
from typing import Any, Dict, Hashable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.manager import KVCacheManager
from ..cache.specs import PagedKVSpec
from ..config import EngineConfig, build_model_spec, load_model_config
from ..sampling import Sampler, SamplingParams, derive_seed
from ..utils.crash_dump import dump_step_failure
from ..utils.logging import get_logger
from ..utils.stages import stage
from ..weights import init_random_on_device, load_weights
from .runner import ModelRunner, StepItem
from .scheduler import Request, Scheduler, SchedulerOutput

logger = get_logger(__name__)


def size_cache_pages(layer_specs, page_size: int, dtype: torch.dtype, device: torch.device,
                     utilization: float, max_num_seqs: int, max_model_len: int, max_step_tokens: Optional[int] = None) -> int:
  """Pages of a group that keeps every key, from the memory that is free now (the reference: a share of the free
  memory divided by the bytes of one token, miniinfer/utils/memory_utils.py:85-144), capped at what ``max_num_seqs``
  requests of ``max_model_len`` tokens could ever hold.  Groups that keep a window have a size of their own
  (``KVCacheManager.group_pages``), which is taken off the memory first."""
  cap = max_num_seqs * (-(-max_model_len // page_size))
  if KVCacheManager.bytes_per_page(layer_specs, page_size, dtype) == 0:
    return 1
  if device.type != "cuda":
    return cap
  free, total = torch.cuda.mem_get_info(device)
  usable = int((free - (1.0 - utilization) * total) * 0.9)
  per_page = KVCacheManager.bytes_per_page(layer_specs, page_size, dtype, windowed=False)
  if max_step_tokens is None:
    per_page = KVCacheManager.bytes_per_page(layer_specs, page_size, dtype)
  else:
    size = torch.empty((), dtype=dtype).element_size()
    for spec in layer_specs:
      if isinstance(spec, PagedKVSpec) and spec.window is not None:
        pages = KVCacheManager.group_pages(spec, page_size, cap, max_num_seqs, max_step_tokens) + 1
        usable -= pages * 2 * spec.num_kv_heads * spec.head_dim * page_size * size
  if per_page == 0:
    return cap
  pages = usable // per_page
  if pages < 2:
    raise RuntimeError(f"not enough free device memory for the cache: {free >> 20} MiB free, "
                       f"one page of the groups that keep every key costs {per_page >> 10} KiB")
  return min(pages, cap)


@dataclass
class RequestOutput:
  """What ``stream_generate`` yields for a request and a generated token (the reference's fields,
  miniinfer/engine/llm_engine.py:50-59)."""

  request_id: Hashable
  delta_text: str
  full_text: str
  token_id: int
  output_token_ids: List[int]
  finished: bool
  finish_reason: Optional[str] = None


class LLMEngine:
  def __init__(self, model: str, **kwargs: Any):
    self.config = EngineConfig.from_kwargs(model, **kwargs)
    cfg = self.config
    self.device = torch.device(cfg.device)
    if self.device.type == "cuda":
      torch.cuda.set_device(self.device)
    self.model_config = load_model_config(cfg.model_path)
    self.spec = build_model_spec(self.model_config)
    t0 = time.time()
    if cfg.load_format == "random":
      init_random_on_device(self.spec, cfg.dtype, self.device, cfg.seed)
    else:
      load_weights(self.spec, cfg.model_path, cfg.dtype, self.device)
    logger.info("weights ready in %.1f s", time.time() - t0)
    cfg.max_context_len = min(cfg.max_context_len, self.model_config.max_position_embeddings)
    layer_specs = self.spec.cache_layer_specs()
    max_step_tokens = max(1, min(cfg.max_num_batched_tokens, cfg.chunked_prefill_size))   # the most a request gets in one step
    num_pages = cfg.num_pages
    if num_pages is None:
      num_pages = size_cache_pages(layer_specs, cfg.page_size, cfg.dtype, self.device, cfg.gpu_memory_utilization,
                                   cfg.max_num_seqs, cfg.max_context_len, max_step_tokens)
    self.cache = KVCacheManager(layer_specs, cfg.page_size, num_pages, cfg.max_num_seqs, cfg.max_context_len,
                                cfg.dtype, self.device, max_step_tokens=max_step_tokens)
    self.runner = ModelRunner(self.spec, self.cache, cfg.dtype, self.device)
    self.scheduler = Scheduler(self.cache, cfg.max_num_seqs, cfg.max_num_batched_tokens, cfg.chunked_prefill_size,
                               cfg.max_context_len, self.model_config.eos_ids())
    self.tokenizer = self._load_tokenizer(cfg.model_path)
    self._requests: Dict[Hashable, Request] = {}
    self._next_id = 0
    self._submit_lock = threading.Lock()
    self._tokens_host: Optional[torch.Tensor] = None
    self._tokens_dev: Optional[torch.Tensor] = None
    self._host_tokens: List[Optional[torch.Tensor]] = [None, None]   # two pinned arrays: a step's tokens may still be on their way when the next is launched
    self._flip = 0
    self._inflight: Optional["LLMEngine._InFlight"] = None
    self._new_tokens: List[tuple] = []          # (request, token) of the step whose tokens were read last
    self._submitted: "queue.Queue" = queue.Queue()   # requests handed in from other threads (submit_request)
    self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "h2d_bytes": 0, "d2h_bytes": 0, "launches": 0,
                  "host_schedule_s": 0.0, "host_launch_s": 0.0, "host_wait_s": 0.0, "host_update_s": 0.0}

  # ------------------------------------------------------------------ life cycle (API parity)

  def start(self) -> "LLMEngine":
    return self

  def stop(self) -> None:
    """Lets go of what the kernel wrappers keep per weight and cache tensor, so that this engine's memory
    is free once the engine itself is dropped (the reference's stop ends its worker processes,
    miniinfer/engine/llm_engine.py:1284-1299; this engine has none)."""
    from ..kernels import ops
    ops.forget_tensors()

  def __enter__(self) -> "LLMEngine":
    return self.start()

  def __exit__(self, *exc) -> None:
    self.stop()

  # ------------------------------------------------------------------ text

  @staticmethod
  def _load_tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
      return None
    try:
      from tokenizers import Tokenizer
    except ImportError:
      return None
    return Tokenizer.from_file(path)

  def _encode(self, prompt: Union[str, Sequence[int]]) -> List[int]:
    if isinstance(prompt, str):
      if self.tokenizer is None:
        raise ValueError("a text prompt needs tokenizer.json in the model folder; pass token ids instead")
      return list(self.tokenizer.encode(prompt).ids)
    return [int(t) for t in prompt]

  def _decode(self, ids: Sequence[int]) -> Optional[str]:
    return self.tokenizer.decode(list(ids)) if self.tokenizer is not None else None

  # ------------------------------------------------------------------ requests

  def add_request(self, prompt: Union[str, Sequence[int]], sampling_params: Optional[SamplingParams] = None,
                  request_id: Optional[Hashable] = None) -> Hashable:
    params = sampling_params or SamplingParams()
    with self._submit_lock:
      rid = request_id if request_id is not None else self._next_id
      if rid in self._requests:
        raise ValueError(f"request id {rid!r} is in use")
      self._next_id += 1
    req = Request(req_id=rid, prompt_ids=self._encode(prompt), params=params)
    self.scheduler.add(req)
    req.seed = params.seed if params.seed is not None else derive_seed(self.config.seed, req.number)
    self._requests[rid] = req
    return rid

  def add_requests(self, prompts: Sequence[Union[str, Sequence[int]]],
                   sampling_params: Sequence[SamplingParams]) -> List[Hashable]:
    """Several requests at once (miniinfer/engine/llm_engine.py:325); returns their ids."""
    if len(prompts) != len(sampling_params):
      raise ValueError(f"prompts and sampling_params length mismatch: {len(prompts)} vs {len(sampling_params)}")
    return [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]

  def submit_request(self, prompt: Union[str, Sequence[int]], sampling_params: Optional[SamplingParams] = None) -> Hashable:
    """Hands a request in from any thread (miniinfer/engine/llm_engine.py:362); it joins the
    waiting queue at the next ``step``.  Returns its id."""
    with self._submit_lock:
      rid = self._next_id
      self._next_id += 1
    self._submitted.put((rid, self._encode(prompt), sampling_params or SamplingParams()))
    return rid

  def _take_submitted(self) -> None:
    while True:
      try:
        rid, ids, params = self._submitted.get_nowait()
      except queue.Empty:
        return
      req = Request(req_id=rid, prompt_ids=ids, params=params)
      self.scheduler.add(req)
      req.seed = params.seed if params.seed is not None else derive_seed(self.config.seed, req.number)
      self._requests[rid] = req

  def is_finished(self) -> bool:
    return not self.has_unfinished()

  def has_unfinished(self) -> bool:
    return self._inflight is not None or self.scheduler.has_unfinished() or not self._submitted.empty()

  # ------------------------------------------------------------------ one step

  def _token_buffers(self, n: int):
    if self._tokens_dev is None or self._tokens_dev.numel() < n:
      cap = max(n, 256)
      self._tokens_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
      self._tokens_host = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
    return self._tokens_dev, self._tokens_host

  # A launched step whose tokens the host has not read yet: its scheduler output, the requests it
  # samples for (row order), the pinned array the tokens are copied to, the event after that copy,
  # and the device view of the tokens (the next step may take its input there).
  class _InFlight:
    __slots__ = ("out", "reqs", "host", "done", "tokens_dev", "graph_decode")

  def _launch(self, out: SchedulerOutput, ids_on_device: Optional[torch.Tensor] = None) -> "LLMEngine._InFlight":
    """Describes and launches the scheduled step and starts the copy of its tokens to the host."""
    items, sampling_reqs = [], []
    for it in out.items:
      n = len(it.tokens)
      items.append(StepItem(it.request.req_id, it.tokens, (n - 1,) if it.samples else ()))
      if it.samples:
        sampling_reqs.append(it.request)
    counters = [len(r.output_ids) + (1 if ids_on_device is not None else 0) for r in sampling_reqs]   # the token in flight counts
    extras = Sampler.pack([r.params for r in sampling_reqs], [r.seed for r in sampling_reqs], counters) if sampling_reqs else {}
    R = len(sampling_reqs)
    dev, _ = self._token_buffers(max(R, 1))
    toks_dev = self.runner.step_and_sample(items, extras, Sampler.sample, dev, use_graphs=not self.config.enforce_eager,
                                           ids_on_device=ids_on_device, sampling_pad=Sampler.PAD_ROWS)
    self.stats["h2d_bytes"] += self.runner.last_h2d_bytes
    self.stats["launches"] += self.runner.last_launches
    self.stats["steps"] += 1
    self.stats["prefill_tokens"] += out.num_prefill_tokens
    self.stats["decode_tokens"] += out.num_decode_tokens
    fl = LLMEngine._InFlight()
    fl.out, fl.reqs, fl.tokens_dev = out, sampling_reqs, toks_dev
    fl.graph_decode = not self.config.enforce_eager and self.runner.graph_decode_bucket(items) is not None
    self._flip ^= 1
    fl.host = self._host_tokens[self._flip]
    if fl.host is None or fl.host.numel() < max(R, 1):
      fl.host = self._host_tokens[self._flip] = torch.empty(max(R, 256), dtype=torch.int32, pin_memory=self.device.type == "cuda")
    fl.done = None
    if R:
      fl.host[:R].copy_(toks_dev, non_blocking=True)
      self.stats["d2h_bytes"] += 4 * R
      if self.device.type == "cuda":
        fl.done = torch.cuda.Event()
        fl.done.record()
    return fl

  def _finish(self, fl: "LLMEngine._InFlight") -> List[Dict[str, Any]]:
    """Waits for the step's tokens and hands them to the scheduler; returns the outputs of the requests that finished."""
    if fl.done is not None:
      fl.done.synchronize()
    toks = fl.host[:len(fl.reqs)].tolist() if fl.reqs else []
    # a request that ended one step ago (a stop token the host had not seen yet) was run once more: that token is dropped
    sampled = {r.req_id: t for r, t in zip(fl.reqs, toks)}
    live = [it for it in fl.out.items if it.request.status != "finished"]
    if len(live) != len(fl.out.items):
      fl.out.items = live
    self._new_tokens = [(it.request, sampled[it.request.req_id]) for it in fl.out.items if it.samples]
    done = self.scheduler.update(fl.out, sampled)
    if self.stats["steps"] % 256 == 0:
      self.runner.check_status()
    return [self._output_of(r) for r in done]

  def _continuation(self, fl: "LLMEngine._InFlight") -> Optional[SchedulerOutput]:
    """The step after ``fl`` if it can be told without ``fl``'s tokens: ``fl`` was a graph step of
    decode tokens only, nothing waits for admission, no request of it ends by length with the
    token in flight, and every request finds room for one more token.  Its items carry a
    placeholder token; the step takes the tokens from the device."""
    sch = self.scheduler
    if not self.config.enable_overlap or not fl.graph_decode or sch.waiting:
      return None
    if len(fl.reqs) != len(fl.out.items) or len(fl.reqs) != len(sch.running) or fl.out.num_prefill_tokens:
      return None
    for r, running in zip(fl.reqs, sch.running):
      if r is not running or len(r.output_ids) + 2 > r.max_tokens:
        return None
    need = [0] * len(self.cache.paged_groups)
    for r in fl.reqs:
      if self.cache.length_of(r.req_id) + 1 > self.cache.max_model_len:
        return None
      for g, n in enumerate(self.cache.pages_needed(r.req_id, 1)):
        need[g] += n
    if any(n > f for n, f in zip(need, self.cache.free_pages())):
      return None
    from .scheduler import ScheduledItem
    nxt = SchedulerOutput(items=[ScheduledItem(r, [0], True) for r in fl.reqs])
    nxt.num_decode_tokens = len(fl.reqs)
    return nxt

  def step(self) -> List[Dict[str, Any]]:
    """One engine step (see ``_step``).  If it raises, what the engine knew - queues, cache occupancy, the
    running requests, graphs and libraries - is logged as one structured record before the error goes on
    (miniinfer/utils/crash_logger.py:1-239)."""
    try:
      return self._step()
    except BaseException as exc:
      if not isinstance(exc, (KeyboardInterrupt, SystemExit)):
        dump_step_failure(exc, scheduler=self.scheduler, cache=self.cache, runner=self.runner, stage="LLMEngine.step")
      raise

  @torch.no_grad()
  def _step(self) -> List[Dict[str, Any]]:
    """Schedules, runs and samples one step; returns the outputs of the requests that finished.
    With ``enable_overlap`` a decode step that follows a decode step of the same requests is
    launched before the tokens of the step before are read (it takes them on the device), so the
    host's work on a step runs beside the device's; what a request generates does not change.  A
    request that ends with a stop token is then run for one token more, which is dropped."""
    t0 = time.perf_counter()
    outs: List[Dict[str, Any]] = []
    self._new_tokens = []
    if not self._submitted.empty():
      self._take_submitted()
    fl = self._inflight
    if fl is not None:
      with stage("schedule"):
        nxt = self._continuation(fl)
      if nxt is not None:
        t1 = time.perf_counter()
        with stage("describe+launch"):
          self._inflight = self._launch(nxt, ids_on_device=fl.tokens_dev)
        t2 = time.perf_counter()
        with stage("wait+update"):
          outs = self._finish(fl)
        t3 = time.perf_counter()
        self.stats["host_schedule_s"] += t1 - t0
        self.stats["host_launch_s"] += t2 - t1
        self.stats["host_wait_s"] += t3 - t2
        return outs
      with stage("wait+update"):
        outs = self._finish(fl)
      self._inflight = None
    t0b = time.perf_counter()
    with stage("schedule"):
      out = self.scheduler.schedule()
    if not out.items:
      return outs
    t1 = time.perf_counter()
    with stage("describe+launch"):
      fl = self._launch(out)
    t2 = time.perf_counter()
    if self.config.enable_overlap and fl.graph_decode:
      self._inflight = fl              # its tokens are read at the next call
      t3 = t4 = time.perf_counter()
    else:
      t3 = time.perf_counter()
      with stage("wait+update"):
        outs += self._finish(fl)
      t4 = time.perf_counter()
    # Host seconds by phase: deciding the step, describing and launching it, waiting for the tokens, book-keeping.
    self.stats["host_schedule_s"] += t1 - t0b
    self.stats["host_launch_s"] += t2 - t1
    self.stats["host_wait_s"] += (t0b - t0) + (t4 - t3)
    return outs

  def stream_generate(self, prompts: Union[str, Sequence[int], Sequence[Union[str, Sequence[int]]]],
                      sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None):
    """Generator over the tokens as they come (miniinfer/engine/llm_engine.py:1341): one
    ``RequestOutput`` per request and generated token.  Requests added meanwhile are served too."""
    if isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int)):
      prompts = [prompts]  # type: ignore[list-item]
    if sampling_params is None or isinstance(sampling_params, SamplingParams):
      plist = [sampling_params or SamplingParams()] * len(prompts)
    else:
      plist = list(sampling_params)
    self.add_requests(prompts, plist)
    texts: Dict[Hashable, str] = {}
    while self.has_unfinished():
      self.step()
      for req, tok in self._new_tokens:
        full = self._decode(req.output_ids) or ""
        before = texts.get(req.req_id, "")
        texts[req.req_id] = full
        finished = req.status == "finished"
        yield RequestOutput(request_id=req.req_id, delta_text=full[len(before):] if full.startswith(before) else full,
                            full_text=full, token_id=tok, output_token_ids=list(req.output_ids), finished=finished,
                            finish_reason=req.finish_reason if finished else None)
        if finished:
          texts.pop(req.req_id, None)
          self._requests.pop(req.req_id, None)

  def _output_of(self, req: Request) -> Dict[str, Any]:
    return {"text": self._decode(req.output_ids), "token_ids": list(req.output_ids), "request_id": req.req_id,
            "finish_reason": req.finish_reason}

  # ------------------------------------------------------------------ generate

  def generate(self, prompts: Union[str, Sequence[int], Sequence[Union[str, Sequence[int]]]],
               sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
               use_tqdm: bool = False) -> List[Dict[str, Any]]:
    """Runs all prompts to completion; returns one dict per prompt, in the order given."""
    if isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int)):
      prompts = [prompts]  # type: ignore[list-item]
    if sampling_params is None or isinstance(sampling_params, SamplingParams):
      plist = [sampling_params or SamplingParams()] * len(prompts)
    else:
      plist = list(sampling_params)
      if len(plist) != len(prompts):
        raise ValueError("sampling_params and prompts differ in length")
    ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
    bar = None
    if use_tqdm:
      from tqdm import tqdm
      bar = tqdm(total=len(ids), desc="Generating")
    results: Dict[Hashable, Dict[str, Any]] = {}
    while not self.is_finished():
      for o in self.step():
        results[o["request_id"]] = o
        if bar is not None:
          bar.update(1)
    if bar is not None:
      bar.close()
    self.runner.check_status()
    for rid in ids:
      self._requests.pop(rid, None)
    return [results[rid] for rid in ids]
