"""The engine's device operations: thin checked wrappers over the sm_100a kernel libraries.

Every function writes into tensors the caller passes, runs on the current CUDA stream and
allocates nothing, so that a step can be captured in a CUDA graph.  There is no other
implementation behind these names: if the libraries cannot be built or loaded, or a tensor is not
on a CUDA device, the call raises.

Large-M bf16 matrix products go to cuBLAS through ``torch.matmul`` - the reference uses the same
library for all of its products (miniinfer/layers/linear.py:30-32); everything else is this
package's own CUDA.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from . import build

F32, BF16 = 0, 1
PREFILL_TILE = 64     # query rows of one tile of the prefill attention kernels
PREFILL_WIDE_TILE = 128   # tokens of a work of the tcgen05 prefill kernel when a block (or each block of a pair) takes one head
PREFILL_PAIRS_MIN_WIDE_TILES = 48   # steps with at least this many such tiles (6144 new tokens) let two blocks share a work
SKINNY_MAX_M = 64     # the most rows the skinny kernel takes
SKINNY_BEST_M = 16    # up to here it is the faster one; above, cuBLAS is (measured on B200, M = 32 and 64)
# Rows from which the tcgen05 gate-up product with SwiGLU in its epilogue beats the library product followed by the
# activation kernel.  Device times on B200 with a cold L2 (each call recorded into a CUDA graph behind a 256 MB flush),
# library + activation against the fused kernel, at 64 / 512 / 1024 / 1280 / 2048 rows:
#   K = 1024, I = 3072:    7.1 / 11.9 / 17.1 / 19.9 / 28.9 us   against   13.7 / 14.9 / 20.5 / 21.0 / 27.0 us
#   K = 2048, I = 6144:   15.4 / 25.6 / 44.2 / 54.0 / 81.7 us   against   21.4 / 34.0 / 45.4 / 56.3 / 77.4 us
#   K = 4096, I = 12288:  49.6 / 76.1 / 142 / 190 / 284 us      against   63.6 / 84.4 / 149 / 173 / 270 us
# The fused kernel saves the pass over [M, 2I] but needs about 13 us to fill and drain its pipeline of 256-row tiles,
# so for prompt portions and mixed steps of fewer rows the library stays (blocks that work alone on 128-row tiles,
# MINIINFER_B200_GEMM_TC=1, are slower still).
GEMM_TC_MIN_M = 1280        # for K >= 4096
GEMM_TC_MIN_M_NARROW = 1792  # for narrower models
_MM_F32_OUT: Optional[bool] = None   # whether torch.mm writes float32 from bf16 operands into a given tensor


class KernelError(RuntimeError):
  """A kernel refused its arguments or failed to launch."""


_libs: Dict[str, ctypes.CDLL] = {}


def _load(name: str, path: str) -> ctypes.CDLL:
  lib = ctypes.CDLL(path)
  lib.mi_last_error.restype = ctypes.c_char_p
  _libs[name] = lib
  return lib


def common_lib() -> ctypes.CDLL:
  lib = _libs.get("common")
  if lib is None:
    lib = _load("common", build.build_common())
  return lib


def attention_lib(head_dim: int) -> ctypes.CDLL:
  name = f"attn_hd{head_dim}"
  lib = _libs.get(name)
  if lib is None:
    lib = _load(name, build.build_attention(head_dim))
  return lib


def loaded_libraries() -> Dict[str, str]:
  return {k: v._name for k, v in _libs.items()}


_launches = 0


def launch_count() -> int:
  """Kernels of this package launched so far by this process (launches recorded into a CUDA graph
  are counted once, when they are recorded)."""
  return _launches


def _check(lib: ctypes.CDLL, code: int, kernels: int = 1) -> None:
  global _launches
  if code != 0:
    raise KernelError(lib.mi_last_error().decode())
  _launches += kernels


def _dt(t: torch.Tensor) -> int:
  if t.dtype == torch.float32:
    return F32
  if t.dtype == torch.bfloat16:
    return BF16
  raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor], dtype: Optional[torch.dtype] = None) -> ctypes.c_void_p:
  if t is None:
    return ctypes.c_void_p(0)
  if not t.is_cuda:
    raise KernelError("the engine's kernels run on CUDA tensors only (got a CPU tensor)")
  if not t.is_contiguous():
    raise KernelError("kernel arguments must be contiguous")
  if dtype is not None and t.dtype != dtype:
    raise KernelError(f"expected {dtype}, got {t.dtype}")
  return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
  """The current CUDA stream of the current device (also the capture stream while a graph is recorded)."""
  if _raw_stream is not None:
    return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# --------------------------------------------------------------------------------------------


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
  """out[t] = table[ids[t]] as float32.  ids: int32, already checked to lie in the vocabulary."""
  lib = common_lib()
  T, H = out.shape
  if table.shape[1] != H or ids.shape[0] != T:
    raise KernelError("embedding: shapes do not match")
  _check(lib, lib.mi_embedding(_ptr(out, torch.float32), _ptr(table), _dt(table), _ptr(ids, torch.int32),
                               T, H, _stream()))


def add_rmsnorm(out: torch.Tensor, resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
  """out[r] = weight * norm(resid[row] + delta[row]); the sum goes back to resid if write_back."""
  lib = common_lib()
  R, H = out.shape
  if resid.shape[1] != H or weight.shape[0] != H or (delta is not None and delta.shape != resid.shape):
    raise KernelError("add_rmsnorm: shapes do not match")
  if rows is None and resid.shape[0] != R:
    raise KernelError("add_rmsnorm: out and resid differ in rows")
  if rows is not None and rows.shape[0] != R:
    raise KernelError("add_rmsnorm: rows and out differ in length")
  _check(lib, lib.mi_add_rmsnorm(_ptr(out), _dt(out), _ptr(resid, torch.float32), _ptr(delta),
                                 _dt(delta) if delta is not None else F32, _ptr(weight, torch.float32),
                                 _ptr(rows, torch.int32) if rows is not None else _ptr(None), R, H,
                                 ctypes.c_float(eps), int(bool(write_back)), _stream()))


_transposed_views: Dict[int, tuple] = {}
_capturing = False


class recording_graph:
  """``with ops.recording_graph():`` around a stream capture: library products then go through
  PyTorch, whose cuBLAS handle has a workspace that is safe to use while a graph is recorded."""

  def __enter__(self):
    global _capturing
    self._before = _capturing
    _capturing = True
    return self

  def __exit__(self, *exc):
    global _capturing
    _capturing = self._before
    return False



def _transposed(w: torch.Tensor) -> torch.Tensor:
  """``w.t()``, kept per weight tensor: making the view costs more host time than a small product."""
  hit = _transposed_views.get(id(w))
  if hit is not None and hit[0] is w:
    return hit[1]
  if len(_transposed_views) > 4096:
    _transposed_views.clear()
  v = w.t()
  _transposed_views[id(w)] = (w, v)
  return v


def _mm_f32_out_works(device) -> bool:
  """Tried once: bf16 x bf16 -> float32 through cuBLAS, written into a tensor the caller owns."""
  global _MM_F32_OUT
  if _MM_F32_OUT is None:
    try:
      a = torch.ones(32, 16, dtype=torch.bfloat16, device=device)
      o = torch.empty(32, 32, dtype=torch.float32, device=device)
      torch.mm(a, a.t(), out_dtype=torch.float32, out=o)
      _MM_F32_OUT = bool((o == 16).all().item())
    except (TypeError, RuntimeError, NotImplementedError):
      _MM_F32_OUT = False
  return _MM_F32_OUT


def linear(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, force_skinny: bool = False, force_stream: bool = False) -> None:
  """out[M, N] = x[M, K] @ w[N, K]^T.  float32 operands: this package's fp32 FMA kernel (out float32).
  bfloat16 operands: for M <= 16 the weight-streaming kernels (out bf16 or fp32; a row's value does not depend
  on the other rows) - the tcgen05 one from ``STREAM_TC_MIN_BYTES`` of weights on, the mma.sync one below -,
  cuBLAS above 16 rows (where the reference uses it for every product).
  ``force_skinny``: the mma.sync kernel for any M (in slices of 64 rows); ``force_stream``: the tcgen05 one at any size."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N):
    raise KernelError(f"linear: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  lib = common_lib()
  if x.dtype == torch.float32:
    _check(lib, lib.mi_gemm_f32(_ptr(out, torch.float32), _ptr(x), _ptr(w, torch.float32), M, N, K, N, _stream()))
    return
  if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
    raise KernelError(f"linear: operands must both be float32 or both bfloat16, got {x.dtype} and {w.dtype}")
  if _streams(M, N, K, force_skinny, force_stream) and out.dtype in (torch.bfloat16, torch.float32):
    parts, counters, status = _stream_workspace(lib, x.device)
    _check(lib, lib.mi_gemm_stream_tc_bf16(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, N, _ptr(parts, torch.float32),
                                           _ptr(counters, torch.int32), counters.numel(), parts.shape[0],
                                           _ptr(status, torch.int32), _stream()))
    return
  if M <= SKINNY_BEST_M or (force_skinny and M <= SKINNY_MAX_M):
    _check(lib, lib.mi_gemm_skinny_bf16(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, N, _stream()))
    return
  if not force_skinny:
    if not (out.is_cuda and out.is_contiguous() and x.is_contiguous() and w.is_contiguous()):
      raise KernelError("linear: operands and out must be contiguous CUDA tensors")
    if K % 8 != 0:
      raise KernelError(f"linear: K={K} must be a multiple of 8 (16-byte loads of bf16 rows)")
    if not _capturing and out.dtype in (torch.bfloat16, torch.float32):
      # more than 16 rows: straight to cuBLAS (a third of the host time of torch.mm); not while a graph is recorded
      _check(lib, lib.mi_gemm_cublas_bf16(_ptr(out), _dt(out), _ptr(x), _ptr(w), M, N, K, _stream()), kernels=0)
      return
    if out.dtype == torch.bfloat16:
      torch.mm(x, _transposed(w), out=out)
      return
    if out.dtype == torch.float32 and _mm_f32_out_works(out.device):
      torch.mm(x, _transposed(w), out_dtype=torch.float32, out=out)
      return
  for m0 in range(0, M, SKINNY_MAX_M):
    m1 = min(M, m0 + SKINNY_MAX_M)
    _check(lib, lib.mi_gemm_skinny_bf16(_ptr(out[m0:m1]), _dt(out), _ptr(x[m0:m1]), _ptr(w), m1 - m0, N, K, N,
                                        _stream()))


# Few rows times a large weight matrix: the tcgen05 kernel that deals the matrix out to the SMs in equal stretches
# (gemm_stream_tc.cu) from 160 MiB of weights on, and from 80 MiB where the matrix has more than 4096 rows; else the
# mma.sync kernel (gemm_skinny.cu), whose launches start and end faster and whose 16-warp blocks fill the SMs in one
# round for up to 4096 rows.  Measured on B200, 8 rows, cold weights, microseconds (tcgen05 / mma.sync):
#   10240 x 5120 (105 MB) 23.6 / 26.1    5120 x 8192 (84 MB) 19.9 / 21.1    5120 x 25600 (262 MB) 49.2 / 64.1
#   SwiGLU 2 x 25600 x 5120 (524 MB) 84.3 / 93.4    SwiGLU 2 x 12288 x 4096 (201 MB) 38.8 / 41.7
#   151936 x 1024 (311 MB) 55.1 / 56.2    4096 x 12288 (101 MB) 23.1 / 19.7    6144 x 4096 (50 MB) 14.2 / 11.7
STREAM_TC_MIN_BYTES = 160 << 20
STREAM_TC_MIN_BYTES_MANY_ROWS = 80 << 20
STREAM_TC_MAX_TILES = 1 << 14
_stream_ws: Dict[int, tuple] = {}


def _streams(M: int, weight_rows: int, K: int, force_skinny: bool, force_stream: bool) -> bool:
  if M > SKINNY_BEST_M or force_skinny or K < 64 or K % 8 != 0:
    return False
  mode = os.environ.get("MINIINFER_B200_GEMM_STREAM", "")
  if mode == "0":
    return False
  size = 2 * weight_rows * K
  return (force_stream or mode == "1" or size >= STREAM_TC_MIN_BYTES
          or (size >= STREAM_TC_MIN_BYTES_MANY_ROWS and weight_rows > 4096))


def _stream_workspace(lib, device):
  """Partial sums, tile counters and the status word of the tcgen05 streaming product, made once per device."""
  idx = device.index if device.index is not None else torch.cuda.current_device()
  ws = _stream_ws.get(idx)
  if ws is None:
    if torch.cuda.is_current_stream_capturing():
      raise KernelError("gemm_stream_tc: its workspace must exist before a graph is recorded (run the step once before)")
    floats, blocks = ctypes.c_longlong(0), ctypes.c_int(0)
    _check(lib, lib.mi_gemm_stream_tc_workspace(ctypes.byref(floats), ctypes.byref(blocks)), kernels=0)
    parts = torch.zeros((blocks.value, floats.value // blocks.value), dtype=torch.float32, device=device)
    counters = torch.zeros(STREAM_TC_MAX_TILES, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ws = _stream_ws[idx] = (parts, counters, status)
  return ws


def fuses_few_rows(x_rows: int, dtype: torch.dtype) -> bool:
  """Whether a step of ``x_rows`` rows takes the few-row products with the norm and the residual add fused to them
  (six launches per layer instead of eight).  Off unless MINIINFER_B200_FUSE_FEW_ROWS=1: measured on B200 (Qwen3-0.6B
  shape) the fused decode step takes 1.05 ms against 0.99 ms at batch 8 and 0.78 against 0.74 ms at batch 1.  The
  norm kernels between the products are where, under dependent launch, the next product's blocks get onto the SMs
  and fetch their weights - a step from which the norm launches are simply left out is slower, not faster - while a
  product that follows a product directly finds the SMs' registers taken until its predecessor has ended."""
  return dtype == torch.bfloat16 and 0 < x_rows <= SKINNY_BEST_M and os.environ.get("MINIINFER_B200_FUSE_FEW_ROWS", "0") == "1"


def linear_normed(out: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor) -> None:
  """out[M, N] = rmsnorm(resid)[M, K] @ w[N, K]^T for up to 16 rows: the norm in the product's prologue.
  resid float32, w and out bfloat16; the normalised rows are rounded to bfloat16 once, as ``add_rmsnorm`` rounds them."""
  M, K = resid.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N) or norm_weight.shape != (K,):
    raise KernelError(f"linear_normed: shapes do not match: resid {tuple(resid.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  lib = common_lib()
  _check(lib, lib.mi_gemm_skinny_norm_bf16(_ptr(out, torch.bfloat16), _ptr(resid, torch.float32), _ptr(norm_weight, torch.float32),
                                           ctypes.c_float(eps), _ptr(w, torch.bfloat16), M, N, K, N, _stream()))


def linear_swiglu_normed(out: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor) -> None:
  """out[M, I] = silu(n @ w[:I]^T) * (n @ w[I:]^T) with n = rmsnorm(resid), for up to 16 rows, in one kernel."""
  M, K = resid.shape
  I = out.shape[1]
  if w.shape != (2 * I, K) or out.shape[0] != M or norm_weight.shape != (K,):
    raise KernelError(f"linear_swiglu_normed: shapes do not match: resid {tuple(resid.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  lib = common_lib()
  _check(lib, lib.mi_gemm_skinny_norm_swiglu_bf16(_ptr(out, torch.bfloat16), _ptr(resid, torch.float32), _ptr(norm_weight, torch.float32),
                                                  ctypes.c_float(eps), _ptr(w, torch.bfloat16), M, I, K, I, _stream()))


def linear_add(resid: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> None:
  """resid[M, N] += bfloat16(x[M, K] @ w[N, K]^T) for up to 16 rows: the residual add in the product's epilogue.
  The product is rounded to bfloat16 before it is added, as it is when a bfloat16 product is handed to ``add_rmsnorm``."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or resid.shape != (M, N):
    raise KernelError(f"linear_add: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, resid {tuple(resid.shape)}")
  lib = common_lib()
  _check(lib, lib.mi_gemm_skinny_add_f32(_ptr(resid, torch.float32), _ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), M, N, K, N, _stream()))


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                       cos_sin: Optional[torch.Tensor], positions: torch.Tensor,
                       slot_mapping: Optional[torch.Tensor], kv_layer: Optional[torch.Tensor],
                       num_heads: int, num_kv_heads: int, head_dim: int, eps: float) -> None:
  """In place on the fused QKV rows: per-head RMSNorm of q and k, rotary encoding from the table,
  and the store of k and v into the layer's pages at ``slot_mapping`` (page * page_size + offset)."""
  lib = common_lib()
  T = qkv.shape[0]
  if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
    raise KernelError("qk_norm_rope_store: qkv width does not match the head counts")
  rotary_dim = 0
  if cos_sin is not None:
    rotary_dim = cos_sin.shape[1]
  page_size = 0
  if kv_layer is not None:
    if kv_layer.dtype != qkv.dtype:
      raise KernelError("qk_norm_rope_store: cache and activations differ in dtype")
    if kv_layer.shape[1:] != (2, num_kv_heads, kv_layer.shape[3], head_dim):
      raise KernelError(f"qk_norm_rope_store: cache layer has shape {tuple(kv_layer.shape)}")
    page_size = kv_layer.shape[3]
  _check(lib, lib.mi_qk_norm_rope_store(
    _ptr(qkv), _dt(qkv), _ptr(q_weight, torch.float32) if q_weight is not None else _ptr(None),
    _ptr(k_weight, torch.float32) if k_weight is not None else _ptr(None),
    _ptr(cos_sin, torch.float32) if cos_sin is not None else _ptr(None), rotary_dim,
    _ptr(positions, torch.int32), _ptr(slot_mapping, torch.int32) if slot_mapping is not None else _ptr(None),
    _ptr(kv_layer), T, num_heads, num_kv_heads, head_dim, page_size, ctypes.c_float(eps), _stream()))


def linear_swiglu(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, workspace, force_skinny: bool = False,
                  force_tc: bool = False, force_stream: bool = False) -> None:
  """out[M, I] = silu(x @ w[:I]^T) * (x @ w[I:]^T): the gate-and-up product of a SwiGLU feed-forward.
  bfloat16 with M <= 16 or from 1280 rows on (1792 for K < 4096): one kernel, the activation in the product's
  epilogue (few rows: the weight-streaming kernel; many: the tcgen05 kernel).  Otherwise the product into a buffer of
  ``workspace``, then the activation kernel (the same up to the order of the sums over K)."""
  M, K = x.shape
  I = out.shape[1]
  if w.shape != (2 * I, K) or out.shape[0] != M or out.dtype != x.dtype:
    raise KernelError(f"linear_swiglu: shapes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if M == 0:
    return
  if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and _streams(M, 2 * I, K, force_skinny, force_stream):
    lib = common_lib()
    parts, counters, status = _stream_workspace(lib, x.device)
    _check(lib, lib.mi_gemm_stream_tc_swiglu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _ptr(parts, torch.float32),
                                                  _ptr(counters, torch.int32), counters.numel(), parts.shape[0],
                                                  _ptr(status, torch.int32), _stream()))
    return
  if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (M <= SKINNY_BEST_M or (force_skinny and M <= SKINNY_MAX_M)):
    lib = common_lib()
    _check(lib, lib.mi_gemm_skinny_swiglu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _stream()))
    return
  many = force_tc or M >= (GEMM_TC_MIN_M if K >= 4096 else GEMM_TC_MIN_M_NARROW)
  if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and many and K >= 64 and K % 8 == 0 and I % 8 == 0
      and x.is_contiguous() and w.is_contiguous() and out.is_contiguous() and os.environ.get("MINIINFER_B200_GEMM_TC", "1") != "0"):
    # many rows: the product on tcgen05 with the activation in its epilogue; [M, 2I] is never written
    lib = common_lib()
    status = workspace.zeros("gemm_tc_status", 1, torch.int32)
    _check(lib, lib.mi_gemm_tc_swiglu_bf16(_ptr(out), _ptr(x), _ptr(w), M, I, K, I, _ptr(status, torch.int32), _tc_pairs(), _stream()))
    return
  gu = workspace.buffer("gate_up", (M, 2 * I), x.dtype)
  linear(gu, x, w)
  silu_mul(out, gu)


def _tc_pairs() -> int:
  """Whether the tcgen05 product lets two blocks share a tile (MINIINFER_B200_GEMM_TC=1: blocks work alone)."""
  return 0 if os.environ.get("MINIINFER_B200_GEMM_TC", "2") == "1" else 1


def linear_tc(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, workspace) -> None:
  """out = x @ w^T in bfloat16 through the tcgen05 kernel that `linear_swiglu` uses for many rows,
  without the activation (the engine's plain products with many rows go to the library)."""
  M, K = x.shape
  N = w.shape[0]
  if w.shape[1] != K or out.shape != (M, N) or not (x.dtype == w.dtype == out.dtype == torch.bfloat16):
    raise KernelError(f"linear_tc: shapes or dtypes do not match: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
  if not (x.is_contiguous() and w.is_contiguous() and out.is_contiguous()):
    raise KernelError("linear_tc: operands must be contiguous")
  if M == 0:
    return
  lib = common_lib()
  status = workspace.zeros("gemm_tc_status", 1, torch.int32)
  _check(lib, lib.mi_gemm_tc_bf16(_ptr(out), _ptr(x), _ptr(w), M, N, K, N, _ptr(status, torch.int32), _tc_pairs(), _stream()))


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
  lib = common_lib()
  T, I = out.shape
  if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
    raise KernelError("silu_mul: shapes or dtypes do not match")
  _check(lib, lib.mi_silu_mul(_ptr(out), _ptr(gate_up), _dt(out), T, I, _stream()))


def sample(out: torch.Tensor, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seed: torch.Tensor, counter: torch.Tensor, workspace=None) -> None:
  """One token per row of float32 logits; see ``sampling/sampler.py`` for the rule.  ``workspace``
  (a ``Workspace``) lends the scratch for the per-slice results; without it scratch is allocated."""
  lib = common_lib()
  R, V = logits.shape
  for t in (out, temperature, top_k, top_p, seed, counter):
    if t.shape[0] != R:
      raise KernelError("sample: per-row arguments differ in length")
  if R == 0:
    return
  slices = max(1, min(64, 640 // R, -(-V // 1024)))   # about four blocks of the pick kernel per SM
  words = R + 2 * R * slices
  if workspace is not None:
    scratch = workspace.buffer("sample_partials", (words,), torch.int32)
    arrivals = workspace.zeros("sample_arrivals", R, torch.int32)
  else:
    scratch = torch.empty(words, dtype=torch.int32, device=logits.device)
    arrivals = torch.zeros(R, dtype=torch.int32, device=logits.device)
  _check(lib, lib.mi_sample(_ptr(out, torch.int32), _ptr(logits, torch.float32), _ptr(temperature, torch.float32),
                            _ptr(top_k, torch.int32), _ptr(top_p, torch.float32), _ptr(seed, torch.int64),
                            _ptr(counter, torch.int64), _ptr(scratch), _ptr(arrivals, torch.int32), R, V, slices,
                            _stream()), kernels=2)


class AttentionBatch:
  """Device-side description of a step for the attention kernels (all int32).

  ``token_item[t]``: the batch item of token t; ``positions[t]``: its position in its request;
  ``seq_slot[b]``: the block-table row of item b; ``q_start[b]``, ``q_len[b]``, ``ctx_len[b]``:
  the item's first row, its number of new tokens and its length including them.
  Lists the launchers need: ``prefill_tiles`` ((item, first row) of every ``PREFILL_TILE`` rows of the items
  with several new tokens), ``prefill_wide_tiles`` (the same in steps of ``PREFILL_WIDE_TILE``; optional: without it
  the tcgen05 prefill kernel never pairs blocks), ``decode_items`` (the items with exactly one new token), their
  lengths and the largest context."""

  __slots__ = ("token_item", "positions", "seq_slot", "q_start", "q_len", "ctx_len", "num_tokens", "num_items",
               "prefill_tiles", "num_prefill_tiles", "prefill_wide_tiles", "num_prefill_wide_tiles", "decode_items", "num_decode",
               "max_ctx_len", "decode_chunk", "scratch")

  def __init__(self, **kw):
    for k in self.__slots__:
      setattr(self, k, kw.get(k))


def attention(out: torch.Tensor, qkv: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor,
              batch: AttentionBatch, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: Optional[int], force_generic: bool = False) -> None:
  """out[t, h*hd:(h+1)*hd] = softmax(scale * q . K^T over the keys the token may see) V, reading
  K and V through the block table.  ``qkv`` holds the step's fused rows; q is its first part."""
  T = qkv.shape[0]
  if out.shape != (T, num_heads * head_dim) or out.dtype != qkv.dtype or kv_layer.dtype != qkv.dtype:
    raise KernelError("attention: shapes or dtypes do not match")
  page_size = kv_layer.shape[3]
  if kv_layer.shape[1:] != (2, num_kv_heads, page_size, head_dim):
    raise KernelError(f"attention: cache layer has shape {tuple(kv_layer.shape)}")
  win = int(window) if window else 0
  if qkv.dtype == torch.bfloat16 and not force_generic and head_dim % 16 == 0 and 16 <= head_dim <= 256:
    _attention_bf16(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale, win, page_size)
    return
  lib = common_lib()
  _check(lib, lib.mi_attention_generic(
    _ptr(out), _ptr(qkv), qkv.shape[1], _dt(qkv), _ptr(kv_layer), _ptr(block_table, torch.int32),
    block_table.shape[1], _ptr(batch.token_item, torch.int32), _ptr(batch.positions, torch.int32),
    _ptr(batch.seq_slot, torch.int32), T, num_heads, num_kv_heads, head_dim, page_size,
    ctypes.c_float(scale), win, _stream()))


def _rope_in_attention(qkv, cos_sin, kv_layer, batch, nh, nkv, hd, win, page_size) -> int:
  """The cluster size with which a step takes the decode kernel that norms, rotates and stores itself, or 0: a step
  of decode tokens only, bfloat16, head size 128 with the whole head rotated, and few enough (request, kv head)
  pairs for the cluster-scheduled kernel."""
  if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and hd == 128 and page_size % 64 == 0 and nh // nkv <= 8):
    return 0
  if batch.num_prefill_tiles or batch.num_decode != qkv.shape[0] or batch.num_decode == 0:
    return 0
  if cos_sin is not None and (cos_sin.shape[1] != hd or cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous()):
    return 0
  if os.environ.get("MINIINFER_B200_ROPE_IN_ATTENTION", "1") == "0" or os.environ.get("MINIINFER_B200_DECODE_TMA", "1") == "0":
    return 0
  lib = attention_lib(hd)
  span = min(batch.max_ctx_len, win) if win else batch.max_ctx_len
  return decode_cluster_size(lib, hd, batch.num_decode, nkv, span)


def rope_store_attention(out: torch.Tensor, qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                         cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                         kv_layer: torch.Tensor, writes: bool, block_table: torch.Tensor, batch: AttentionBatch,
                         num_heads: int, num_kv_heads: int, head_dim: int, eps: float, scale: float, window: Optional[int]) -> None:
  """From the fused QKV rows of a step to its attention output: ``qk_norm_rope_store`` (which also puts the new
  keys and values into the layer's pages, if ``writes``) followed by ``attention``.  A step of a few decode tokens
  takes one kernel for both (attention_decode_cluster.cu), which does the first step's arithmetic operation for
  operation: the results are the same bit for bit, except that ``qkv`` is then left as the product wrote it."""
  win = int(window) if window else 0
  page_size = kv_layer.shape[3] if kv_layer is not None and kv_layer.dim() == 5 else 0
  cluster = _rope_in_attention(qkv, cos_sin, kv_layer, batch, num_heads, num_kv_heads, head_dim, win, page_size) if page_size else 0
  if not cluster:
    qk_norm_rope_store(qkv, q_weight, k_weight, cos_sin, positions, slot_mapping if writes else None,
                       kv_layer if writes else None, num_heads, num_kv_heads, head_dim, eps)
    attention(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale, window)
    return
  T = qkv.shape[0]
  if out.shape != (T, num_heads * head_dim) or out.dtype != qkv.dtype or kv_layer.dtype != qkv.dtype:
    raise KernelError("rope_store_attention: shapes or dtypes do not match")
  if kv_layer.shape[1:] != (2, num_kv_heads, page_size, head_dim) or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
    raise KernelError(f"rope_store_attention: cache layer {tuple(kv_layer.shape)} or qkv {tuple(qkv.shape)} do not match the head counts")
  lib = attention_lib(head_dim)
  if batch.scratch is not None:
    status = batch.scratch.zeros("attention_decode_counters", batch.num_decode * num_kv_heads + 1, torch.int32)[:1]
  else:
    status = torch.zeros(1, dtype=torch.int32, device=qkv.device)
  none = _ptr(None)
  _check(lib, lib.mi_attention_decode_cluster_rope(
    _ptr(out), _ptr(qkv), qkv.shape[1], _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
    none, _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),     # no list of decode items: all items are, in order (one dependent load less before the first copy: 0.4 % of a step)
    _ptr(batch.seq_slot, torch.int32), _ptr(status, torch.int32), batch.num_decode, num_heads, num_kv_heads, page_size,
    ctypes.c_float(scale), win, cluster, batch.max_ctx_len,
    _ptr(q_weight, torch.float32) if q_weight is not None else none, _ptr(k_weight, torch.float32) if k_weight is not None else none,
    _ptr(cos_sin, torch.float32) if cos_sin is not None else none,
    _ptr(slot_mapping, torch.int32) if (writes and slot_mapping is not None) else none,
    _ptr(kv_layer) if writes else none, ctypes.c_float(eps), _stream()))
  if batch.scratch is None and int(status[0]) != 0:
    raise KernelError("attention_decode_cluster: a bounded wait on a copy barrier ran out")


DECODE_CHUNKS = (512, 256, 128, 64)
def decode_chunk(num_decode: int, num_kv_heads: int, max_ctx_len: int, head_dim: int) -> int:
  """Keys per block of the cp.async split-KV decode kernel: the longest chunk that still gives every
  SM about two blocks, so that a small batch is spread over the whole GPU."""
  forced = os.environ.get("MINIINFER_B200_DECODE_CHUNK")
  if forced:
    return int(forced)
  two_per_sm = 2 * _num_sms(torch.device("cuda", torch.cuda.current_device()))
  for c in DECODE_CHUNKS:
    if num_decode * num_kv_heads * -(-max_ctx_len // c) >= two_per_sm:
      return c
  return DECODE_CHUNKS[-1]


_cluster_fit: Dict[tuple, int] = {}


def decode_cluster_size(lib, head_dim: int, num_decode: int, num_kv_heads: int, span: int) -> int:
  """Blocks per (request, kv head) for the cluster-scheduled decode kernel (attention_decode_cluster.cu), or 0 if
  the step should take the persistent kernel instead.  The largest cluster (16, 8, 4, 2, 1 blocks) that leaves a
  block at least one 64-key tile (6 is tried as well: two requests are a little faster with it) and whose clusters - one per (request, kv head) - can all be on the GPU at once:
  a second round of clusters would double the kernel's time.  (Measured on B200, 8 kv heads of 128, 2048-token
  contexts: 1 / 2 / 4 / 8 / 16 requests are fastest with clusters of 8 / 4 / 4 / 2 / 1, which is what this rule
  picks; decode steps took 0.74 / 0.79 / 0.83 / 0.99 / 1.34 ms against 0.92 / 0.92 / 0.99 / 1.12 / 1.55 ms with
  the persistent kernel, and the sizes were measured again after the cluster's merge had lost a barrier.)  Blocks with more than 64 tiles each, or more (request, kv head) pairs than fit at once,
  stream better from the persistent kernel, which deals the tiles out evenly over the SMs."""
  tiles = -(-span // 64) + 1

  def fit(c: int) -> int:
    key = (head_dim, c, -(-tiles // c))
    n = _cluster_fit.get(key)
    if n is None:
      n = _cluster_fit[key] = int(lib.mi_attention_decode_cluster_fit(c, -(-tiles // c)))
    return n

  forced = os.environ.get("MINIINFER_B200_DECODE_CLUSTER")
  if forced is not None:
    c = int(forced)
    return c if c and fit(c) > 0 else 0
  pairs = num_decode * num_kv_heads
  for c in (16, 8, 6, 4, 2, 1):
    if c <= tiles and -(-tiles // c) <= DECODE_CLUSTER_MAX_TILES_PER_BLOCK and pairs <= fit(c):
      return c
  return 0


DECODE_CLUSTER_MAX_TILES_PER_BLOCK = 64


def _attention_bf16(out, qkv, kv_layer, block_table, batch, nh, nkv, hd, scale, win, page_size) -> None:
  """Tensor-core kernel for the items with several new tokens, split-KV kernel for the decode items;
  the two write disjoint rows of ``out``."""
  lib = attention_lib(hd)
  if batch.num_prefill_tiles:
    use_tc = (page_size % 64 == 0 and lib.mi_attention_prefill_tc_supported() == 1
              and os.environ.get("MINIINFER_B200_PREFILL_TC", "1") != "0")
    if use_tc:
      if batch.scratch is not None:
        status = batch.scratch.zeros("attention_prefill_status", 1, torch.int32)
      else:
        status = torch.zeros(1, dtype=torch.int32, device=qkv.device)
      wide, n_wide = batch.prefill_wide_tiles, int(batch.num_prefill_wide_tiles or 0)
      # two blocks on one work (tcgen05 cta_group::2: half the K / V bytes per SM, twice the stages): measured on B200
      # at 16 heads of 128, 291 against 303 us for 8192 new tokens, 31.4 against 31.2 us for 2048 - so only large steps
      force = os.environ.get("MINIINFER_B200_PREFILL_PAIRS")
      pairs = int(force == "1") if force in ("0", "1") else int(n_wide >= PREFILL_PAIRS_MIN_WIDE_TILES)
      _check(lib, lib.mi_attention_prefill_tc(
        _ptr(out), _qkv_tensor_map(lib, qkv), _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.prefill_tiles, torch.int32), batch.num_prefill_tiles, _ptr(batch.q_start, torch.int32),
        _ptr(batch.q_len, torch.int32), _ptr(batch.ctx_len, torch.int32), _ptr(batch.seq_slot, torch.int32),
        _ptr(status, torch.int32), nh, nkv, page_size, ctypes.c_float(scale), win, _num_sms(qkv.device), _stream(),
        _ptr(wide, torch.int32) if wide is not None else _ptr(None), n_wide, pairs))
      if batch.scratch is None and int(status[0]) != 0:
        raise KernelError("attention_prefill_tc: a bounded wait on a barrier ran out")
    else:
      _check(lib, lib.mi_attention_prefill_bf16(
        _ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.prefill_tiles, torch.int32), batch.num_prefill_tiles, _ptr(batch.q_start, torch.int32),
        _ptr(batch.q_len, torch.int32), _ptr(batch.ctx_len, torch.int32), _ptr(batch.seq_slot, torch.int32),
        nh, nkv, page_size, ctypes.c_float(scale), win, _stream()))
  if batch.num_decode:
    span = min(batch.max_ctx_len, win) if win else batch.max_ctx_len
    G = nh // nkv
    tma_shapes = hd % 64 == 0 and page_size % 64 == 0 and os.environ.get("MINIINFER_B200_DECODE_TMA", "1") != "0"
    cluster = decode_cluster_size(lib, hd, batch.num_decode, nkv, span) if (tma_shapes and G <= 8) else 0
    if cluster:
      if batch.scratch is not None:
        status = batch.scratch.zeros("attention_decode_counters", batch.num_decode * nkv + 1, torch.int32)[:1]
      else:
        status = torch.zeros(1, dtype=torch.int32, device=qkv.device)
      _check(lib, lib.mi_attention_decode_cluster(
        _ptr(out), _ptr(qkv), qkv.shape[1], _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.decode_items, torch.int32), _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),
        _ptr(batch.seq_slot, torch.int32), _ptr(status, torch.int32), batch.num_decode, nh, nkv, page_size, ctypes.c_float(scale), win,
        cluster, batch.max_ctx_len, _stream()))
      if batch.scratch is None and int(status[0]) != 0:
        raise KernelError("attention_decode_cluster: a bounded wait on a copy barrier ran out")
      return
    # more than 8 query heads per kv head: the TMA kernel would walk an item's tiles twice and hand a stage back only
    # in the second pass, which cannot work once an item has more tiles than there are stages - the cp.async kernel takes those
    use_tma = (hd % 64 == 0 and page_size % 64 == 0 and G <= 8 and os.environ.get("MINIINFER_B200_DECODE_TMA", "1") != "0")
    if use_tma:
      # the TMA kernel deals 64-key tiles out evenly; a (request, kv head) is cut into at most as many
      # pieces as it has tiles, and no more than there are blocks
      chunk = 64
      max_splits = min(-(-span // 64) + 2, _num_sms(qkv.device))
    else:
      chunk = batch.decode_chunk or decode_chunk(batch.num_decode, nkv, span, hd)
      max_splits = -(-span // chunk) + 1
    n = batch.num_decode * nh * max_splits * (hd + 2)
    if batch.scratch is not None:
      scratch = batch.scratch.buffer("attention_decode_partials", (n,), torch.float32)
      counters = batch.scratch.zeros("attention_decode_counters", batch.num_decode * nkv + 1, torch.int32)
    else:
      scratch = torch.empty(n, dtype=torch.float32, device=qkv.device)
      counters = torch.zeros(batch.num_decode * nkv + 1, dtype=torch.int32, device=qkv.device)
    if use_tma:
      _check(lib, lib.mi_attention_decode_tma(
        _ptr(out), _ptr(qkv), qkv.shape[1], _kv_tensor_map(lib, kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.decode_items, torch.int32), _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),
        _ptr(batch.seq_slot, torch.int32), _ptr(scratch, torch.float32), _ptr(counters[1:], torch.int32), _ptr(counters[:1], torch.int32),
        batch.num_decode, nh, nkv, page_size, ctypes.c_float(scale), win, chunk, max_splits, _num_sms(qkv.device), _stream()))
      if batch.scratch is None and int(counters[0]) != 0:
        raise KernelError("attention_decode_tma: a bounded wait on a copy barrier ran out")
    else:
      _check(lib, lib.mi_attention_decode_bf16(
        _ptr(out), _ptr(qkv), qkv.shape[1], _ptr(kv_layer), _ptr(block_table, torch.int32), block_table.shape[1],
        _ptr(batch.decode_items, torch.int32), _ptr(batch.q_start, torch.int32), _ptr(batch.ctx_len, torch.int32),
        _ptr(batch.seq_slot, torch.int32), _ptr(scratch, torch.float32), _ptr(counters[1:], torch.int32),
        batch.num_decode, nh, nkv, page_size, ctypes.c_float(scale), win, chunk, max_splits, _stream()))


_tensor_maps: Dict[tuple, ctypes.Array] = {}
_sm_counts: Dict[int, int] = {}


def _num_sms(device) -> int:
  idx = device.index if device.index is not None else torch.cuda.current_device()
  if idx not in _sm_counts:
    _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
  return _sm_counts[idx]


def _kv_tensor_map(lib, kv_layer: torch.Tensor):
  """The TMA descriptor of a cache layer (made once per layer: it holds the layer's address)."""
  key = (kv_layer.data_ptr(), tuple(kv_layer.shape))
  m = _tensor_maps.get(key)
  if m is None:
    m = ctypes.create_string_buffer(128)
    rows = kv_layer.shape[0] * kv_layer.shape[1] * kv_layer.shape[2] * kv_layer.shape[3]
    code = lib.mi_kv_tensor_map(m, _ptr(kv_layer), ctypes.c_longlong(rows))
    if code != 0:
      raise KernelError(lib.mi_last_error().decode())
    _tensor_maps[key] = m
  return m


def _qkv_tensor_map(lib, qkv: torch.Tensor):
  """The TMA descriptor of a step's fused QKV rows (kept per address and shape: the workspace hands
  out the same buffer step after step)."""
  key = ("qkv", qkv.data_ptr(), tuple(qkv.shape))
  m = _tensor_maps.get(key)
  if m is None:
    if not qkv.is_contiguous():
      raise KernelError("attention: the QKV rows must be contiguous")
    if len(_tensor_maps) > 4096:
      _tensor_maps.clear()
    m = ctypes.create_string_buffer(128)
    code = lib.mi_qkv_tensor_map(m, _ptr(qkv), ctypes.c_longlong(qkv.shape[0]), ctypes.c_longlong(qkv.shape[1]))
    if code != 0:
      raise KernelError(lib.mi_last_error().decode())
    _tensor_maps[key] = m
  return m


def forget_tensors() -> None:
  """Drops what this module keeps per tensor address (transposed views of weights, TMA descriptors of cache
  layers and QKV buffers).  The views keep the weights' memory alive: an engine that is done calls this so
  that its memory can go back to the device."""
  _transposed_views.clear()
  _tensor_maps.clear()


def device_status(ws) -> int:
  """The status words that kernels with bounded waits set when a wait ran out (0: all well)."""
  code = 0
  for name in ("attention_decode_counters", "attention_prefill_status", "gemm_tc_status"):
    buf = ws._bufs.get((name, torch.int32))
    if buf is not None:
      code |= int(buf[0])
  for _, _, status in _stream_ws.values():
    code |= int(status[0])
  return code
