"""The sampling entry point that allocates nothing (csrc/no_alloc_api.h), called through its exported
C symbol and compared with the regular entry point.

Some users of the kernel library may not allocate device memory when they sample - the whole device
belongs to their own pool, or their serving loop bans cudaMalloc because it synchronises the device -
so this variant keeps its scratch in a fixed array inside the library.  The test checks that it
gives the tokens the regular kernel gives, twice in a row (the second call finds the scratch as the
first left it), that it refuses more rows than it has scratch for, and that it really left the
allocator alone.  It sits in a file of its own that is collected last, so a failure here cannot
hide the result of any other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, out, logits, temperature, top_k, top_p, seed, counter):
  R, V = logits.shape
  p = lambda t: ctypes.c_void_p(t.data_ptr())
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  return lib.mi_sample_static(p(out), p(logits), p(temperature), p(top_k), p(top_p), p(seed), p(counter), R, V, stream)


@pytest.mark.parametrize("R,V", [(6, 1000), (1, 151936), (256, 520)])
def test_no_alloc_sampler_matches_the_regular_one(R, V):
  from miniinfer_b200.kernels import ops
  lib = ops.common_lib()
  dev = "cuda:0"
  g = torch.Generator().manual_seed(R * 7 + V)
  f = lambda v, dt: torch.tensor(v, dtype=dt, device=dev)
  temperature = f([(0.8, 1.0, 0.5, 1.3, 0.0, 0.7)[i % 6] for i in range(R)], torch.float32)
  top_k = f([(0, 20, 0, 50, 0, 1)[i % 6] for i in range(R)], torch.int32)
  top_p = f([(1.0, 1.0, 0.9, 0.6, 1.0, 1.0)[i % 6] for i in range(R)], torch.float32)
  seed = f([100 + i for i in range(R)], torch.int64)
  for call in range(2):                         # two calls in a row share the library's scratch
    logits = (torch.randn(R, V, generator=g) * 2.0).to(dev)
    counter = f([call * 3 + i for i in range(R)], torch.int64)
    want = torch.full((R,), -1, dtype=torch.int32, device=dev)
    ops.sample(want, logits, temperature, top_k, top_p, seed, counter)
    got = torch.full((R,), -2, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    # free bytes as the driver counts them: a cudaMalloc inside the library would take them from here,
    # whereas PyTorch's own allocator statistics never see what a C library allocates
    free_before, _ = torch.cuda.mem_get_info(dev)
    code = _call_static(lib, got, logits, temperature, top_k, top_p, seed, counter)
    torch.cuda.synchronize()
    assert code == 0, lib.mi_last_error().decode()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after >= free_before, f"the call took {free_before - free_after} bytes of device memory"
    assert torch.equal(got, want), f"call {call}: {got.tolist()[:8]} vs {want.tolist()[:8]}"
    assert int(got.min()) >= 0 and int(got.max()) < V


def test_no_alloc_sampler_refuses_what_it_has_no_scratch_for():
  from miniinfer_b200.kernels import ops
  lib = ops.common_lib()
  dev = "cuda:0"
  R, V = 257, 64
  z = lambda dt: torch.zeros(R, dtype=dt, device=dev)
  out = torch.full((R,), -5, dtype=torch.int32, device=dev)
  code = _call_static(lib, out, torch.zeros(R, V, device=dev), z(torch.float32), z(torch.int32), z(torch.float32) + 1,
                      z(torch.int64), z(torch.int64))
  torch.cuda.synchronize()
  assert code != 0
  assert "257" in lib.mi_last_error().decode() and "256" in lib.mi_last_error().decode()
  assert int(out.max()) == -5                     # nothing ran
