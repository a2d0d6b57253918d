#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of a Qwen3-0.6B-shaped model (28 layers, hidden 1024, 16 query and
8 kv heads of 128, intermediate 3072, vocabulary 151936, tied head) in bfloat16, 8 requests with a
2048-token context each.  A step is one decode step of the whole batch.

One JSON line is printed:
  value      decoded tokens per second of the step function with sampling (CUDA-graph replay, device
             timing with CUDA events around K steps; every step reads weights + cache, far more than L2)
  e2e        the same through ``LLMEngine.step`` - scheduler, pinned-host token/metadata upload, graph
             replay, sampled tokens back to the host - timed around K engine steps
  prefill    one whole 2048-token prompt in one step: tokens/s, ms, fraction of the bf16 tensor peak
  roofline   bytes the decode step must read (every weight once + the cache of the live requests)
             divided by its time, against the measured HBM copy bandwidth
  points     decode tokens/s at batch 1 and 64
  kernels    the dominant kernels of the decode step (the matrix products that stream the weights, the
             attention kernel that streams the cache) and of the prefill step (the matrix products, the
             attention kernel): microseconds per step from CUPTI kernel records of a few further steps,
             the bytes or FLOPs they account for, and the rate that follows against the measured peak

``--shape 8b`` / ``--shape 32b`` run the same measurement at the layer sizes of Qwen3-8B (36 layers) and
Qwen3-32B (64 layers, 4096-token contexts, max_model_len 8192).
"""
import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=28, hidden_size=1024,
             num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
             rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=True)
# other shapes for --shape: what differs from MODEL
SHAPES = {"0.6b": {},
          "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     intermediate_size=12288, tie_word_embeddings=False),
          "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      intermediate_size=25600, tie_word_embeddings=False)}
SHAPE_CONTEXT = {"32b": 4096}          # tokens each request holds when decoding starts, where it is not 2048
SHAPE_MAX_MODEL_LEN = {"32b": 8192}
CONTEXT = 2048
GENERATED = 256
MAX_MODEL_LEN = 4096
PREFILL_TOKENS = 2048
PAGE = 64


def peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      d = json.load(f)
    return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
  return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

  FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self):
    self.samples = []
    self.proc = None
    self.thread = None

  def start(self):
    try:
      self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      return
    self.thread = threading.Thread(target=self._read, daemon=True)
    self.thread.start()

  def _read(self):
    for line in self.proc.stdout:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) == 6:
        self.samples.append(parts)

  def stop(self) -> dict:
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    mhz, mx, reasons = [], None, set()
    for s in self.samples:
      try:
        mhz.append(float(s[0]))
        mx = float(s[1])
      except ValueError:
        continue
      for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:]):
        if v.lower().startswith("active"):
          reasons.add(name)
    mhz.sort()
    return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def model_bytes(cfg: dict, layers: int) -> dict:
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  per_layer = ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * 2 + (2 * H + 2 * hd) * 4
  head = V * H * 2
  return {"weights": layers * per_layer + head + H * 4, "kv_per_token": layers * 2 * nkv * hd * 2}


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  gemm = 2.0 * T * ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * layers + 2.0 * V * H
  attn = layers * 2.0 * 2.0 * nh * hd * (T * (T + 1) / 2)
  return gemm + attn


def build_engine(model_dir: str, batch: int):
  from miniinfer_b200 import LLMEngine
  pages = batch * (-(-(CONTEXT + GENERATED + 128) // PAGE)) + 8          # GENERATED covers warm-up + steps (see main)
  pages = max(pages, -(-PREFILL_TOKENS // PAGE) + 8)
  return LLMEngine(model_dir, dtype="bfloat16", device="cuda:0", load_format="random", page_size=PAGE, num_pages=pages,
                   max_num_seqs=max(batch, 1), max_model_len=MAX_MODEL_LEN, max_num_batched_tokens=PREFILL_TOKENS, seed=0)


def fill_context(engine, batch: int, tokens: int, seed: int):
  """Admits `batch` requests and runs their prompts through the step function in portions."""
  import torch
  from miniinfer_b200.engine import StepItem
  g = torch.Generator().manual_seed(seed)
  V = engine.model_config.vocab_size
  ids = []
  for b in range(batch):
    rid = f"bench{b}"
    engine.cache.admit(rid)
    prompt = torch.randint(0, V, (tokens,), generator=g).tolist()
    for s in range(0, tokens, PREFILL_TOKENS):
      engine.runner.step([StepItem(rid, prompt[s:s + PREFILL_TOKENS], ())])
    ids.append(rid)
  torch.cuda.synchronize()
  return ids


def time_decode(engine, batch: int, steps: int, warmup: int) -> dict:
  """K decode steps of the step function with sampling, through the decode CUDA graph."""
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  rids = fill_context(engine, batch, CONTEXT, seed=batch)
  params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
  tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")
  last = [1] * batch
  n = [0]

  def one():
    extras = Sampler.pack(params, list(range(batch)), [n[0]] * batch)
    items = [StepItem(r, [t], (0,)) for r, t in zip(rids, last)]
    engine.runner.step_and_sample(items, extras, Sampler.sample, tokens_dev, sampling_pad=Sampler.PAD_ROWS)
    n[0] += 1

  for _ in range(max(warmup, 3)):
    one()
  torch.cuda.synchronize()
  start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  start.record()
  for _ in range(steps):
    one()
  end.record()
  torch.cuda.synchronize()
  ms = start.elapsed_time(end) / steps
  launches = engine.runner.last_launches
  mean_ctx = CONTEXT + max(warmup, 3) + steps / 2.0
  for r in rids:
    engine.cache.release_request(r)
  return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches_per_step": launches, "mean_ctx": mean_ctx}


def time_e2e(engine, batch: int, steps: int, warmup: int) -> dict:
  """The same decode steps through the Python entry point: host tokens in, host tokens out."""
  import torch
  from miniinfer_b200 import SamplingParams
  g = torch.Generator().manual_seed(100 + batch)
  V = engine.model_config.vocab_size
  # the first requests decode while the later ones' prompts still run, portion by portion
  early = batch * -(-CONTEXT // PREFILL_TOKENS)
  sp = SamplingParams(temperature=0.6, max_tokens=max(warmup, 3) + steps + early + 16, ignore_eos=True)
  for b in range(batch):
    engine.add_request(torch.randint(0, V, (CONTEXT,), generator=g).tolist(), sp)
  while any(r.total_len - r.num_computed != 1 for r in engine.scheduler.running) or engine.scheduler.waiting:
    engine.step()                      # prompts, in portions under the token budget
  for _ in range(max(warmup, 3)):
    engine.step()
  torch.cuda.synchronize()
  s0 = dict(engine.stats)
  t0 = time.perf_counter()
  for _ in range(steps):
    engine.step()
  torch.cuda.synchronize()
  dt = time.perf_counter() - t0
  s1 = dict(engine.stats)
  host = {k[5:-2]: round(1e6 * (s1[k] - s0[k]) / steps, 1) for k in s1 if k.startswith("host_")}
  print(f"e2e host microseconds per step by phase: {host}", file=sys.stderr)
  assert s1["decode_tokens"] - s0["decode_tokens"] == batch * steps, "the timed steps were not pure decode steps"
  while engine.has_unfinished():
    engine.step()
  return {"tok_s": batch * steps / dt, "ms": 1000.0 * dt / steps,
          "h2d": (s1["h2d_bytes"] - s0["h2d_bytes"]) / steps, "d2h": (s1["d2h_bytes"] - s0["d2h_bytes"]) / steps,
          "launches": (s1["launches"] - s0["launches"]) / steps}


def time_prefill(engine, reps: int = 5) -> dict:
  import torch
  from miniinfer_b200.engine import StepItem
  g = torch.Generator().manual_seed(7)
  V = engine.model_config.vocab_size
  times = []
  for i in range(reps + 2):
    rid = f"prefill{i}"
    engine.cache.admit(rid)
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    engine.runner.step([StepItem(rid, prompt, (PREFILL_TOKENS - 1,))])
    end.record()
    torch.cuda.synchronize()
    if i >= 2:
      times.append(start.elapsed_time(end))
    engine.cache.release_request(rid)
  times.sort()
  return {"ms": times[len(times) // 2]}


def kernel_table(engine, batch: int, steps: int = 6, mode: str = "decode") -> str:
  """Device time of every kernel of a decode step (a few graph replays) or of a prefill step, from CUPTI records."""
  import torch
  from torch.profiler import ProfilerActivity, profile
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  if mode == "prefill":
    g = torch.Generator().manual_seed(7)
    V = engine.model_config.vocab_size

    def whole(i):
      rid = f"prefill{i}"
      engine.cache.admit(rid)
      engine.runner.step([StepItem(rid, torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist(), (PREFILL_TOKENS - 1,))])
      engine.cache.release_request(rid)

    for i in range(2):
      whole(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
      for i in range(steps):
        whole(10 + i)
      torch.cuda.synchronize()
    return _table_of(prof, steps, f"prefill step, {PREFILL_TOKENS} tokens")
  rids = fill_context(engine, batch, CONTEXT, seed=batch)
  params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
  tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

  def one(i):
    extras = Sampler.pack(params, list(range(batch)), [i] * batch)
    engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev)

  for i in range(4):
    one(i)
  torch.cuda.synchronize()
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for i in range(steps):
      one(10 + i)
    torch.cuda.synchronize()
  for r in rids:
    engine.cache.release_request(r)
  return _table_of(prof, steps, f"decode step, batch {batch}")


def _table_of(prof, steps: int, title: str) -> str:
  rows = []
  total = 0.0
  for ev in prof.key_averages():
    t = getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0)
    if t <= 0:
      continue
    rows.append((t / steps, ev.count / steps, ev.key))
    total += t / steps
  rows.sort(reverse=True)
  lines = [f"{title}: {total:.1f} us of kernels per step"]
  for t, c, name in rows[:24]:
    lines.append(f"{t:9.1f} us/step  {c:6.1f} launches/step  {t / max(c, 1e-9):7.2f} us each  {name[:110]}")
  return "\n".join(lines)


def _kernel_times(fn, steps: int) -> dict:
  """Kernel name -> microseconds per step, from CUPTI records of `steps` calls of fn."""
  import torch
  from torch.profiler import ProfilerActivity, profile
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for i in range(steps):
      fn(i)
    torch.cuda.synchronize()
  out = {}
  for ev in prof.key_averages():
    t = getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0)
    if t > 0:
      out[ev.key] = t / steps
  return out


def _group(times: dict) -> dict:
  """Sums the kernels of a step by what they do."""
  import re
  g = {"own_products": 0.0, "library_products": 0.0, "attention": 0.0, "other": 0.0}
  for name, us in times.items():
    if "gemm_skinny" in name or "gemm_tc_kernel" in name or "gemm_stream_tc" in name:
      g["own_products"] += us
    elif re.search(r"decode_tma_kernel|decode_cluster_kernel|decode_split_kernel|decode_merge|attention_prefill", name):
      g["attention"] += us
    elif "anonymous namespace" not in name and re.search(r"nvjet|cutlass|cublas|gemm|gemv|xmma", name, re.I):
      g["library_products"] += us
    elif not name.startswith("Memcpy") and not name.startswith("Memset"):
      g["other"] += us
  return g


def kernel_rates(engine, batch: int, cfg: dict, layers: int, pk: dict, steps: int = 4) -> dict:
  """The dominant kernels of a decode step and of a prefill step with the rates they reach: the products
  stream every weight once (decode) or do the step's matrix FLOPs (prefill); the attention kernel streams
  the cache of the live requests (decode) or does the causal attention FLOPs (prefill)."""
  import torch
  from miniinfer_b200.engine import StepItem
  from miniinfer_b200.sampling import Sampler, SamplingParams
  mb = model_bytes(cfg, layers)
  rids = fill_context(engine, batch, CONTEXT, seed=1000 + batch)
  params = [SamplingParams(temperature=0.6, max_tokens=GENERATED, ignore_eos=True)] * batch
  tokens_dev = torch.zeros(max(batch, 1), dtype=torch.int32, device="cuda:0")

  def decode(i):
    extras = Sampler.pack(params, list(range(batch)), [i] * batch)
    engine.runner.step_and_sample([StepItem(r, [1], (0,)) for r in rids], extras, Sampler.sample, tokens_dev,
                                  sampling_pad=Sampler.PAD_ROWS)

  for i in range(4):
    decode(i)
  torch.cuda.synchronize()
  d = _group(_kernel_times(lambda i: decode(10 + i), steps))
  for r in rids:
    engine.cache.release_request(r)
  prod_us = d["own_products"] + d["library_products"]
  kv_bytes = batch * (CONTEXT + 4 + steps / 2.0) * mb["kv_per_token"]
  out = {"source": f"CUPTI kernel records of {steps} further steps in a process of its own, dependent launch off", "decode": {
    "products": {"us": round(prod_us, 1), "bytes": int(mb["weights"]), "GB/s": round(mb["weights"] / prod_us / 1e3, 1),
                 "frac": round(mb["weights"] / prod_us / 1e3 / pk["hbm_gbs"], 4), "own_share": round(d["own_products"] / max(prod_us, 1e-9), 3)},
    "attention": {"us": round(d["attention"], 1), "bytes": int(kv_bytes), "GB/s": round(kv_bytes / d["attention"] / 1e3, 1),
                  "frac": round(kv_bytes / d["attention"] / 1e3 / pk["hbm_gbs"], 4)},
    "other_us": round(d["other"], 1)}}

  g = torch.Generator().manual_seed(7)
  V = engine.model_config.vocab_size

  def whole(i):
    rid = f"rates{i}"
    engine.cache.admit(rid)
    engine.runner.step([StepItem(rid, torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist(), (PREFILL_TOKENS - 1,))])
    engine.cache.release_request(rid)

  for i in range(2):
    whole(i)
  torch.cuda.synchronize()
  p = _group(_kernel_times(lambda i: whole(10 + i), 2))
  H, I, Vv = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  T = PREFILL_TOKENS
  gemm_flops = 2.0 * T * ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * layers + 2.0 * Vv * H
  attn_flops = layers * 2.0 * 2.0 * nh * hd * (T * (T + 1) / 2)
  prod_us = p["own_products"] + p["library_products"]
  out["prefill"] = {
    "products": {"us": round(prod_us, 1), "TFLOP": round(gemm_flops / 1e12, 4), "TFLOP/s": round(gemm_flops / prod_us / 1e6, 1),
                 "frac": round(gemm_flops / prod_us / 1e6 / pk["bf16_tflops"], 4), "own_share": round(p["own_products"] / max(prod_us, 1e-9), 3)},
    "attention": {"us": round(p["attention"], 1), "TFLOP": round(attn_flops / 1e12, 4), "TFLOP/s": round(attn_flops / p["attention"] / 1e6, 1),
                  "frac": round(attn_flops / p["attention"] / 1e6 / pk["bf16_tflops"], 4)},
    "other_us": round(p["other"], 1)}
  return out


def kernel_case(name: str, reps: int = 3) -> str:
  """One kernel alone on an input larger than L2, a few launches: the workload of the ncu summaries under
  profiles/ for the kernels that a benchmark step does not reach (or reaches only at small sizes)."""
  import torch
  from miniinfer_b200.engine.context import Workspace
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.kernels.ops import AttentionBatch
  dev = torch.device("cuda:0")
  g = torch.Generator(device=dev).manual_seed(1)
  rnd = lambda *shape, dtype=torch.bfloat16, scale=1.0: (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)
  ws = Workspace(dev)

  def attention_case(dtype, page, items):
    """items: (context length, new tokens) per request; the cache holds random keys and values."""
    nh, nkv, hd = 16, 8, 128
    pages_per = [-(-c // page) for c, _ in items]
    kv = rnd(sum(pages_per) + 1, 2, nkv, page, hd, dtype=dtype)
    bt = torch.zeros(len(items) + 1, max(pages_per) + 1, dtype=torch.int32)
    nxt = 1
    for b, n in enumerate(pages_per):
      bt[b, :n] = torch.arange(nxt, nxt + n)
      nxt += n
    T = sum(n for _, n in items)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    q_start, pos, tok_item, row = [], [], [], 0
    for b, (c, n) in enumerate(items):
      q_start.append(row)
      pos += list(range(c - n, c))
      tok_item += [b] * n
      row += n
    tiles = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, ops.PREFILL_TILE)]
    wide = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, ops.PREFILL_WIDE_TILE)]
    dec = [b for b, (c, n) in enumerate(items) if n == 1]
    batch = AttentionBatch(token_item=i32(tok_item), positions=i32(pos), seq_slot=i32(list(range(len(items)))), q_start=i32(q_start),
                           q_len=i32([n for _, n in items]), ctx_len=i32([c for c, _ in items]), num_tokens=T, num_items=len(items),
                           prefill_tiles=i32(tiles).view(-1, 2) if tiles else torch.zeros((0, 2), dtype=torch.int32, device=dev),
                           num_prefill_tiles=len(tiles), prefill_wide_tiles=i32(wide).view(-1, 2) if wide else None,
                           num_prefill_wide_tiles=len(wide), decode_items=i32(dec) if dec else torch.zeros(0, dtype=torch.int32, device=dev),
                           num_decode=len(dec), max_ctx_len=max(c for c, _ in items), scratch=ws)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype)
    out = torch.empty(T, nh * hd, dtype=dtype, device=dev)
    return lambda: ops.attention(out, qkv, kv, bt.to(dev), batch, nh, nkv, hd, hd ** -0.5, None), f"{len(items)} requests {items[:2]}.., page {page}, {dtype}"

  if name == "sample":
    R, V = 256, 151936
    logits = rnd(R, V, dtype=torch.float32, scale=2.0)
    f = lambda v, dt: torch.tensor(v, dtype=dt, device=dev)
    args = (f([(0.8, 1.0, 0.6, 0.0)[i % 4] for i in range(R)], torch.float32), f([(0, 50, 0, 0)[i % 4] for i in range(R)], torch.int32),
            f([(1.0, 1.0, 0.9, 1.0)[i % 4] for i in range(R)], torch.float32), f(list(range(R)), torch.int64), f([3] * R, torch.int64))
    out = torch.empty(R, dtype=torch.int32, device=dev)
    fn, what = (lambda: ops.sample(out, logits, *args, ws)), f"{R} rows x {V} float32 logits (155 MB), a quarter each: plain temperature, top-k 50, top-p 0.9, greedy"
  elif name == "silu_mul":
    gu, out = rnd(8192, 2 * 12288), torch.empty(8192, 12288, dtype=torch.bfloat16, device=dev)
    fn, what = (lambda: ops.silu_mul(out, gu)), "8192 x (2 x 12288) bf16: 403 MB in, 201 MB out"
  elif name == "gemm_f32":
    x, w = rnd(256, 4096, dtype=torch.float32), rnd(8192, 4096, dtype=torch.float32, scale=0.02)
    out = torch.empty(256, 8192, device=dev)
    fn, what = (lambda: ops.linear(out, x, w)), "float32, M = 256, N = 8192, K = 4096 (134 MB of weights, 17.2 GFLOP)"
  elif name == "gemm_tc_plain":
    x, w = rnd(2048, 4096), rnd(4096, 4096, scale=0.02)
    out = torch.empty(2048, 4096, dtype=torch.bfloat16, device=dev)
    fn, what = (lambda: ops.linear_tc(out, x, w, ws)), "bf16 plain product on tcgen05, M = 2048, N = 4096, K = 4096 (68.7 GFLOP)"
  elif name == "gemm_stream":
    x, w = rnd(8, 25600), rnd(5120, 25600, scale=0.02)
    out = torch.empty(8, 5120, dtype=torch.bfloat16, device=dev)
    fn, what = (lambda: ops.linear(out, x, w)), "bf16 few-row product on tcgen05, M = 8, N = 5120, K = 25600 (262 MB of weights: the down product of the Qwen3-32B shape)"
  elif name == "attention_generic":
    fn, what = attention_case(torch.float32, 64, [(2048, 1)] * 8 + [(2048, 512)])
  elif name == "attention_prefill_tc":
    fn, what = attention_case(torch.bfloat16, 64, [(2048, 2048)])           # the tcgen05 kernel, blocks alone
  elif name == "attention_prefill_tc_pairs":
    fn, what = attention_case(torch.bfloat16, 64, [(8192, 8192)])           # enough tiles of 128 tokens for blocks in pairs
  elif name == "attention_prefill_mma":
    fn, what = attention_case(torch.bfloat16, 16, [(2048, 2048)])           # pages of 16 tokens: not the tcgen05 kernel's
  elif name == "attention_decode_cpasync":
    fn, what = attention_case(torch.bfloat16, 16, [(2048 + 8 * i, 1) for i in range(64)])
  else:
    raise SystemExit(f"unknown kernel case {name!r}")
  fn()
  torch.cuda.synchronize()
  start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  start.record()
  for _ in range(reps):
    fn()
  end.record()
  torch.cuda.synchronize()
  return f"{name}: {what}: {1000 * start.elapsed_time(end) / reps:.1f} us per call (warm, {reps} calls back to back)"


KERNEL_CASES = ("sample", "silu_mul", "gemm_f32", "gemm_tc_plain", "gemm_stream", "attention_generic", "attention_prefill_tc",
                "attention_prefill_tc_pairs", "attention_prefill_mma", "attention_decode_cpasync")


def mixed_workload(model_dir: str, requests: int = 64, outputs: int = 256) -> dict:
  """A continuous batch through `LLMEngine.generate`: prompts of 128 .. 2048 uniform random tokens, `outputs`
  generated tokens each, prompts cut under a budget of 2048 tokens a step.  Run twice; the second run
  (graphs recorded, kernels loaded) is reported."""
  import torch
  from miniinfer_b200 import LLMEngine, SamplingParams
  pages = requests * (-(-(2048 + outputs) // PAGE) + 1) + 8
  engine = LLMEngine(model_dir, dtype="bfloat16", device="cuda:0", load_format="random", page_size=PAGE, num_pages=pages,
                     max_num_seqs=requests, max_model_len=MAX_MODEL_LEN, max_num_batched_tokens=PREFILL_TOKENS, seed=0)
  g = torch.Generator().manual_seed(0)
  lens = torch.randint(128, 2049, (requests,), generator=g).tolist()
  V = engine.model_config.vocab_size
  prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
  sp = SamplingParams(temperature=0.6, max_tokens=outputs, ignore_eos=True)
  res = {}
  for _ in range(2):
    s0 = dict(engine.stats)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate(prompts, sp)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    steps = engine.stats["steps"] - s0["steps"]
    res = {"workload": f"{requests} requests, prompts 128..2048, {outputs} outputs each, 2048 tokens a step",
           "seconds": round(dt, 3), "prompt_tokens": sum(lens), "output_tokens": requests * outputs,
           "total_tok_s": round((sum(lens) + requests * outputs) / dt, 1), "output_tok_s": round(requests * outputs / dt, 1),
           "steps": steps, "ms_per_step": round(1000 * dt / steps, 3)}
  return res


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _write_reference_model(cfg: dict, out_dir: str, seed: int = 0) -> None:
  """A model folder the reference can load, made without this repository's package: config.json,
  model.safetensors with the tensor names of the Qwen3 checkpoints (random N(0, 0.02) matrices, norm
  weights near one) and a word-level tokenizer of the configuration's vocabulary size."""
  import torch
  from safetensors.torch import save_file
  from tokenizers import Tokenizer, models, pre_tokenizers
  os.makedirs(out_dir, exist_ok=True)
  with open(os.path.join(out_dir, "config.json"), "w") as f:
    json.dump(dict(cfg, torch_dtype="bfloat16", hidden_act="silu", attention_bias=False, use_sliding_window=False,
                   bos_token_id=0, eos_token_id=1), f)
  g = torch.Generator().manual_seed(seed)
  H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
  nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  mat = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(torch.bfloat16)
  vec = lambda n: (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
  sd = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H)}
  for i in range(cfg["num_hidden_layers"]):
    p = f"model.layers.{i}"
    sd.update({f"{p}.input_layernorm.weight": vec(H), f"{p}.post_attention_layernorm.weight": vec(H),
               f"{p}.self_attn.q_proj.weight": mat(nh * hd, H), f"{p}.self_attn.k_proj.weight": mat(nkv * hd, H),
               f"{p}.self_attn.v_proj.weight": mat(nkv * hd, H), f"{p}.self_attn.o_proj.weight": mat(H, nh * hd),
               f"{p}.self_attn.q_norm.weight": vec(hd), f"{p}.self_attn.k_norm.weight": vec(hd),
               f"{p}.mlp.gate_proj.weight": mat(I, H), f"{p}.mlp.up_proj.weight": mat(I, H), f"{p}.mlp.down_proj.weight": mat(H, I)})
  if not cfg.get("tie_word_embeddings"):
    sd["lm_head.weight"] = mat(V, H)
  save_file(sd, os.path.join(out_dir, "model.safetensors"))
  vocab = {"<bos>": 0, "<eos>": 1, "<unk>": 2}
  for i in range(3, V):
    vocab[f"t{i}"] = i
  tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
  tok.pre_tokenizer = pre_tokenizers.Whitespace()
  tok.save(os.path.join(out_dir, "tokenizer.json"))
  with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
    json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "bos_token": "<bos>", "eos_token": "<eos>", "unk_token": "<unk>",
               "pad_token": "<eos>", "model_max_length": cfg["max_position_embeddings"]}, f)


def reference_child(args) -> int:
  """Runs in a process of its own, with nothing of this repository's package imported: the reference as
  installed under baseline/_ref (its sub-packages lie there at top level, so the name ``miniinfer`` is
  bound to that folder), its own ``LLMEngine.generate`` with token-id prompts, as its benchmark does
  (benchmark/bench_miniinfer.py:28-58).  Decode tokens a second: two runs that differ only in the number
  of generated tokens, (tokens of the longer - tokens of the shorter) / (time of the longer - the shorter)."""
  import types
  pkg = types.ModuleType("miniinfer")
  pkg.__path__ = [REF_DIR]
  sys.modules["miniinfer"] = pkg
  sys.path.insert(0, REF_DIR)
  os.environ.update(HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1")
  import torch
  from miniinfer.engine.llm_engine import LLMEngine
  from miniinfer.utils.sampling_params import SamplingParams
  cfg = dict(MODEL, **SHAPES[args.shape])
  if args.layers:
    cfg["num_hidden_layers"] = args.layers
  context = args.context if args.context is not None else SHAPE_CONTEXT.get(args.shape, CONTEXT)
  steps, warmup, batch = args.steps, max(args.warmup, 3), args.batch
  with tempfile.TemporaryDirectory() as d:
    _write_reference_model(cfg, d)
    # no dtype is passed: the reference's engine builds its model in float16 whatever it is asked for
    # (miniinfer/engine/model_runner.py:66-68, models/fused_qwen3.py:272), and its cache must match
    engine = LLMEngine(model=d, use_multiprocess=False, max_num_seqs=max(batch, 8),
                       max_context_len=max(MAX_MODEL_LEN, SHAPE_MAX_MODEL_LEN.get(args.shape, 0)), page_size=PAGE * 4,
                       enable_prefix_cache=False, debug=False)
    engine.start()
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def run(n_tokens: int) -> float:
      prompts = [torch.randint(3, V, (context,), generator=g).tolist() for _ in range(batch)]
      sp = SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=n_tokens)
      torch.cuda.synchronize()
      t0 = time.perf_counter()
      outs = engine.generate(prompts=prompts, sampling_params=sp, use_tqdm=False)
      torch.cuda.synchronize()
      dt = time.perf_counter() - t0
      assert all(len(o["token_ids"]) == n_tokens for o in outs), "the reference generated another number of tokens"
      return dt

    run(warmup + 4)                      # loads kernels, records its CUDA graphs
    clocks = ClockSampler()
    clocks.start()
    short = min(run(4) for _ in range(2))
    long_ = min(run(4 + steps) for _ in range(2))
    clock_info = clocks.stop()
    engine.stop()
  ms = 1000.0 * (long_ - short) / steps
  value = batch * 1000.0 / ms
  print(json.dumps({
    "metric": f"decode tok/s at batch {batch} (Qwen3-{args.shape.upper()} shape, {context}-token contexts)",
    "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (the reference's own; same width as bf16)", "impl": "reference",
    "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
    "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": cfg["num_hidden_layers"], "global_batch": batch, "seq_len": context,
               "page_size": PAGE * 4, "attention_backend": "the reference's default", "parallelism": "single GPU",
               "timing": "LLMEngine.generate end to end, host tokens in and out; (time of 4+K tokens - time of 4 tokens) / K"},
    "e2e": {"value": round(value, 1), "unit": "tok/s", "ms_per_step": round(ms, 4)},
    "clocks": clock_info}))
  return 0


def reference_arm(args) -> int:
  """The reference's own engine on the same shape, batch, context and step count, in a child process.
  If it cannot be imported or run, one line says which import or call failed."""
  if not os.path.isdir(REF_DIR):
    print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not exist: the reference was not installed here"}))
    return 0
  cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-child", "--steps", str(args.steps), "--warmup", str(args.warmup),
         "--batch", str(args.batch), "--shape", args.shape]
  if args.layers:
    cmd += ["--layers", str(args.layers)]
  if args.context is not None:
    cmd += ["--context", str(args.context)]
  try:
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
  except subprocess.TimeoutExpired:
    print(json.dumps({"impl": "reference", "unavailable": "the reference's engine did not finish within 25 minutes"}))
    return 0
  lines = [l for l in proc.stdout.splitlines() if l.startswith("{") and '"impl": "reference"' in l]
  if proc.returncode == 0 and lines:
    print(lines[-1])
    return 0
  err = [l.strip() for l in (proc.stderr or "").splitlines() if l.strip()]
  why = err[-1] if err else f"exit code {proc.returncode} without a message"
  where = next((l for l in reversed(err) if l.startswith("File ") and "_ref" in l), "")
  print(json.dumps({"impl": "reference", "unavailable": f"the reference's own code failed: {why[:300]} {where[:200]}".strip()}))
  return 0


def main() -> int:
  global CONTEXT
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=128)
  ap.add_argument("--warmup", type=int, default=8)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-child", "kernels-child"])
  ap.add_argument("--batch", type=int, default=8)
  ap.add_argument("--shape", default="0.6b", choices=sorted(SHAPES), help="layer sizes: the default, or another Qwen3 model's")
  ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
  ap.add_argument("--context", type=int, default=None, help="tokens each request holds when decoding starts (default 2048; 32b: 4096)")
  ap.add_argument("--skip-kernels", action="store_true", help="leave out the per-kernel rates")
  ap.add_argument("--skip-points", action="store_true")
  ap.add_argument("--mixed", action="store_true",
                  help="run a continuous batch of 64 requests through LLMEngine.generate, print its throughput and exit")
  ap.add_argument("--kernel-case", default=None, choices=KERNEL_CASES,
                  help="run one kernel alone on an input larger than L2 (the workload of the ncu summaries) and exit")
  ap.add_argument("--kernel-table", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                  help="print the device time of each kernel of a decode step (default) or a prefill step and exit")
  args = ap.parse_args()
  if args.kernel_case:
    print(kernel_case(args.kernel_case))
    return 0
  if args.impl == "reference":
    return reference_arm(args)
  if args.impl == "reference-child":
    return reference_child(args)
  MODEL.update(SHAPES[args.shape])
  shape_name = f"Qwen3-{args.shape.upper()} shape"
  if args.layers is None:
    args.layers = MODEL["num_hidden_layers"]
  if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
    print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
    return 2

  import torch
  pk = peaks()
  cfg = dict(MODEL, num_hidden_layers=args.layers)
  warmup = max(args.warmup, 3)
  # room for the tokens that the timed steps generate, whatever --steps says
  global GENERATED, MAX_MODEL_LEN
  CONTEXT = args.context if args.context is not None else SHAPE_CONTEXT.get(args.shape, CONTEXT)
  MAX_MODEL_LEN = max(MAX_MODEL_LEN, SHAPE_MAX_MODEL_LEN.get(args.shape, 0))
  GENERATED = max(GENERATED, warmup + args.steps + args.batch * -(-CONTEXT // PREFILL_TOKENS) + 64)
  MAX_MODEL_LEN = max(MAX_MODEL_LEN, -(-(CONTEXT + GENERATED + 128) // 1024) * 1024)
  cfg["max_position_embeddings"] = max(cfg.get("max_position_embeddings", 0), MAX_MODEL_LEN)
  with tempfile.TemporaryDirectory() as d:
    with open(os.path.join(d, "config.json"), "w") as f:
      json.dump(cfg, f)
    if args.mixed:
      print(json.dumps(dict(mixed_workload(d), layers=args.layers, model=shape_name)))
      return 0
    if args.kernel_table:
      print(kernel_table(build_engine(d, args.batch), args.batch, mode=args.kernel_table))
      return 0
    if args.impl == "kernels-child":
      print(json.dumps({"kernels": kernel_rates(build_engine(d, args.batch), args.batch, cfg, args.layers, pk)}))
      return 0
    clocks = ClockSampler()
    engine = build_engine(d, args.batch)
    clocks.start()
    dec = time_decode(engine, args.batch, args.steps, warmup)
    e2e = time_e2e(engine, args.batch, args.steps, warmup)
    pre = time_prefill(engine)
    clock_info = clocks.stop()
    points = {}
    if not args.skip_points:
      for b in (1, 64):
        engine.stop()
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        engine = build_engine(d, b)
        points[f"decode_b{b}"] = round(time_decode(engine, b, args.steps, warmup)["tok_s"], 1)

    # Per-kernel times come from a process of its own with dependent launch off: with it on, a kernel is placed
    # while its predecessor runs and the time it spends waiting there would count as its own.
    rates = None
    if not args.skip_kernels:
      engine.stop()
      del engine
      gc.collect()
      torch.cuda.empty_cache()
      cmd = [sys.executable, os.path.abspath(__file__), "--impl", "kernels-child", "--shape", args.shape, "--batch", str(args.batch),
             "--layers", str(args.layers), "--context", str(CONTEXT)]
      proc = subprocess.run(cmd, capture_output=True, text=True, env=dict(os.environ, MINIINFER_B200_PDL="0"))
      found = [l for l in proc.stdout.splitlines() if l.startswith('{"kernels"')]
      rates = json.loads(found[-1])["kernels"] if found else {"unavailable": (proc.stderr or "no output").strip().splitlines()[-1][:200]}

  mb = model_bytes(cfg, args.layers)
  step_bytes = mb["weights"] + args.batch * dec["mean_ctx"] * mb["kv_per_token"]
  achieved = step_bytes / (dec["ms"] * 1e-3) / 1e9
  flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
  line = {
    "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.shape.upper()} shape, {CONTEXT}-token contexts)",
    "value": round(dec["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
    "ms_per_step": round(dec["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
    "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform random token ids", "impl": "ours",
    "config": {"model": shape_name, "layers": args.layers, "layers_of_model": MODEL["num_hidden_layers"],
               "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
               "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
               "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": CONTEXT, "generated": GENERATED,
               "max_model_len": MAX_MODEL_LEN, "page_size": PAGE, "parallelism": "single GPU",
               "l2": "each step reads weights+cache (>1 GB), larger than L2", "sampling": "temperature 0.6",
               "decode_path": "CUDA graph replay; e2e: a step is launched before the tokens of the step before are read (enable_overlap)"},
    "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "ms_per_step": round(e2e["ms"], 4),
            "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])},
    "gpu_launches": int(dec["launches_per_step"] * args.steps),
    "launches_per_step": int(dec["launches_per_step"]),
    "prefill": {"value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre["ms"], 3),
                "frac": round(flops / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
    "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                 "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
    "points": points,
    "kernels": rates,
    "clocks": clock_info,
  }
  print(json.dumps(line))
  return 0


if __name__ == "__main__":
  sys.exit(main())
