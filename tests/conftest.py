import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
  if p not in sys.path:
    sys.path.insert(0, p)


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200)")


ON_CPU = os.environ.get("MINIINFER_TEST_DEVICE") == "cpu"


@pytest.fixture(autouse=True)
def _statements_in_place_of_kernels(request, monkeypatch):
  """With MINIINFER_TEST_DEVICE=cpu the gpu tests run on the CPU against the kernels' PyTorch
  statements: a check of the tests' own logic where no GPU is at hand, not of the kernels."""
  if ON_CPU and "gpu" in request.keywords:
    import torch_ops
    torch_ops.install(monkeypatch)
  yield


def pytest_collection_modifyitems(config, items):
  if torch.cuda.is_available() or ON_CPU:
    return
  skip = pytest.mark.skip(reason="no CUDA device")
  for item in items:
    if "gpu" in item.keywords:
      item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
  """Model folders with random weights for the tiny configurations, made once per session in a
  temporary folder.  ``model_dirs(tag, dtype="bfloat16")`` -> path."""
  from miniinfer_b200.weights import write_random_model
  from tiny_configs import ALL

  made = {}

  def get(tag: str, dtype: str = "bfloat16", seed: int = None) -> str:
    key = (tag, dtype, seed)
    if key not in made:
      d = tmp_path_factory.mktemp(f"tiny_{tag}_{dtype}")
      s = seed if seed is not None else {"A": 1, "B": 2, "C": 3, "D": 4, "E": 5, "F": 6, "R": 7}[tag]
      write_random_model(dict(ALL[tag]), str(d), seed=s, dtype=getattr(torch, dtype))
      made[key] = str(d)
    return made[key]

  return get


@pytest.fixture
def cpu_kernels(monkeypatch):
  """Replaces the CUDA kernels by their PyTorch statements so host-side logic runs on the CPU."""
  import torch_ops
  torch_ops.install(monkeypatch)
