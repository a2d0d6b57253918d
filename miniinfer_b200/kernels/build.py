"""Compiles the CUDA sources under ``csrc/`` for sm_100a into shared libraries beside them.

A library is a set of ``.cu`` files plus preprocessor definitions (the attention kernels are
compiled once for each head size a model needs).  Its file name carries a hash of the sources,
headers and flags, so a stale build is never loaded.  Everything is built with plain ``nvcc``; no
Python headers are involved, the libraries export C functions and are loaded with ``ctypes``.

Only what is asked for is compiled: the first use of a model compiles the common library and the
attention library of that model's head size, printing a line for every file meanwhile.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# No fast-math: softmax, norms and rotations are compared with a float32 reference.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xptxas", "-v"]

COMMON_SOURCES = ["common.cu", "embedding.cu", "norm.cu", "gemm_f32.cu", "gemm_skinny.cu", "gemm_skinny_fused.cu",
                  "qk_norm_rope.cu", "attention_generic.cu", "activation.cu", "sampling.cu", "gemm_cublas.cu", "gemm_tc.cu",
                  "gemm_stream_tc.cu"]
COMMON_LIBS = ["cublas"]
ATTENTION_SOURCES = ["attention_prefill.cu", "attention_decode.cu", "attention_decode_tma.cu", "attention_prefill_tc.cu",
                     "attention_decode_cluster.cu"]

_lock = threading.Lock()


class BuildError(RuntimeError):
  pass


def _say(msg: str) -> None:
  print(f"[miniinfer_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
  for cand in (os.environ.get("MINIINFER_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise BuildError("nvcc was not found (set MINIINFER_B200_NVCC); the CUDA kernels cannot be built")


def build_dir() -> str:
  """``csrc/_build`` if it can be written, else a per-user folder under the temporary directory."""
  want = os.environ.get("MINIINFER_B200_BUILD_DIR") or os.path.join(CSRC, "_build")
  try:
    os.makedirs(want, exist_ok=True)
    probe = os.path.join(want, f".w{os.getpid()}")
    with open(probe, "w"):
      pass
    os.remove(probe)
    return want
  except OSError:
    alt = os.path.join(tempfile.gettempdir(), f"miniinfer_b200_build_{os.getuid()}")
    os.makedirs(alt, exist_ok=True)
    return alt


def _with_headers(sources: Sequence[str]) -> List[str]:
  """The sources and the headers of this folder that they include, directly or through one another."""
  seen: List[str] = []
  todo = list(sources)
  while todo:
    name = todo.pop()
    if name in seen or not os.path.exists(os.path.join(CSRC, name)):
      continue
    seen.append(name)
    with open(os.path.join(CSRC, name), "r", encoding="utf-8") as f:
      for line in f:
        line = line.strip()
        if line.startswith("#include \""):
          todo.append(line.split("\"")[1])
  return sorted(seen)


def _digest(sources: Sequence[str], defines: Dict[str, str]) -> str:
  h = hashlib.sha256()
  names = _with_headers(sources)
  for name in names:
    h.update(name.encode())
    with open(os.path.join(CSRC, name), "rb") as f:
      h.update(f.read())
  h.update(repr(sorted(defines.items())).encode())
  h.update(repr(ARCH_FLAGS + NVCC_FLAGS).encode())
  return h.hexdigest()[:12]


def library_path(name: str, sources: Sequence[str], defines: Dict[str, str]) -> str:
  return os.path.join(build_dir(), f"libmi_{name}_{_digest(sources, defines)}.so")


def _run(cmd: List[str], what: str, log_path: Optional[str] = None) -> str:
  t0 = time.time()
  proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
  if log_path:
    with open(log_path, "w") as f:
      f.write(" ".join(cmd) + "\n" + proc.stdout)
  if proc.returncode != 0:
    raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout[-6000:]}")
  _say(f"{what}: {time.time() - t0:.1f} s")
  return proc.stdout


def build_library(name: str, sources: Sequence[str], defines: Optional[Dict[str, str]] = None,
                  libs: Sequence[str] = ()) -> str:
  """Returns the path of the built library, compiling it first if it is not there."""
  defines = dict(defines or {})
  with _lock:
    out = library_path(name, sources, defines)
    if os.path.exists(out):
      return out
    nvcc = find_nvcc()
    bdir = os.path.dirname(out)
    tag = os.path.basename(out)[:-3]
    _say(f"compiling {name} ({len(sources)} files) for sm_100a into {bdir}")
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]

    def compile_one(src: str) -> str:
      obj = os.path.join(bdir, f"{tag}_{src[:-3]}.o")
      _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *dflags, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj],
           f"nvcc {src}" + (f" {dflags}" if dflags else ""), obj[:-2] + ".log")
      return obj

    with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 2, 8)) as pool:
      objs = list(pool.map(compile_one, sources))
    tmp = out + f".tmp{os.getpid()}"
    _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, *[f"-l{l}" for l in libs]], f"link {os.path.basename(out)}")
    os.replace(tmp, out)
    for obj in objs:
      try:
        os.remove(obj)
      except OSError:
        pass
    return out


def build_common() -> str:
  return build_library("common", COMMON_SOURCES, libs=COMMON_LIBS)


def build_attention(head_dim: int) -> str:
  if head_dim % 16 or head_dim < 16 or head_dim > 256:
    raise BuildError(f"attention kernels take head sizes 16..256 in steps of 16, got {head_dim}")
  return build_library(f"attn_hd{head_dim}", ATTENTION_SOURCES, {"MI_HEAD_DIM": str(head_dim)})


def build_all(head_dims: Sequence[int] = (16, 32, 48, 64, 80, 128, 256), remove_stale: bool = True) -> List[str]:
  """Builds the common library and the attention library of every head size in ``head_dims``.  Libraries
  of other source versions (another hash in the name) and their compiler logs are then removed from the
  build folder, so that it holds one build."""
  paths = [build_common()]
  for hd in head_dims:
    paths.append(build_attention(hd))
  if remove_stale:
    keep = {os.path.basename(p)[:-3] for p in paths}
    bdir = os.path.dirname(paths[0])
    for name in os.listdir(bdir):
      if name.startswith("libmi_") and not any(name.startswith(k) for k in keep):
        try:
          os.remove(os.path.join(bdir, name))
        except OSError:
          pass
  return paths
