"""Helpers of the GPU tests: random paged caches and attention batches."""
from __future__ import annotations

import random
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from miniinfer_b200.kernels.ops import AttentionBatch

import os

# MINIINFER_TEST_DEVICE=cpu runs the gpu tests' own logic on the CPU with the kernels' PyTorch statements
# (see conftest.py); it checks the tests, not the kernels.
DEV = os.environ.get("MINIINFER_TEST_DEVICE", "cuda:0")


def make_attention_case(items: Sequence[Tuple[int, int]], nh: int, nkv: int, hd: int, page_size: int,
                        dtype: torch.dtype, seed: int = 0, num_slots: int = 8, scale_q: float = 1.0):
  """``items``: (context length including the new tokens, number of new tokens) for each request.
  Returns (qkv rows, cache layer, block table, batch) with pages handed out in shuffled order and the
  cache already holding every key and value, also those of the new tokens."""
  rng = random.Random(seed)
  g = torch.Generator().manual_seed(seed)
  max_ctx = max(c for c, _ in items)
  pages_per_seq = -(-max_ctx // page_size)
  total_pages = sum(-(-c // page_size) for c, _ in items)
  ids = list(range(1, total_pages + 4))
  rng.shuffle(ids)
  bt = np.zeros((num_slots + 1, pages_per_seq + 2), dtype=np.int32)
  slots = rng.sample(range(num_slots), len(items))
  kv = (torch.randn((total_pages + 4, 2, nkv, page_size, hd), generator=g) * 1.0).to(dtype)
  q_len = [n for _, n in items]
  T = sum(q_len)
  qkv = (torch.randn((T, (nh + 2 * nkv) * hd), generator=g) * scale_q).to(dtype)
  positions, token_item, q_start, ctx_len = [], [], [], []
  row = 0
  for b, (c, n) in enumerate(items):
    npages = -(-c // page_size)
    for i in range(npages):
      bt[slots[b], i] = ids.pop()
    q_start.append(row)
    ctx_len.append(c)
    for i in range(n):
      positions.append(c - n + i)
      token_item.append(b)
    row += n

  def dev(x, dt=torch.int32):
    return torch.tensor(x, dtype=dt, device=DEV)

  tiles = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, 64)]
  wide = [(b, o) for b, (c, n) in enumerate(items) if n > 1 for o in range(0, n, 128)]
  dec = [b for b, (c, n) in enumerate(items) if n == 1]
  batch = AttentionBatch(
    token_item=dev(token_item), positions=dev(positions), seq_slot=dev(slots), q_start=dev(q_start), q_len=dev(q_len),
    ctx_len=dev(ctx_len), num_tokens=T, num_items=len(items),
    prefill_tiles=dev(tiles).view(-1, 2) if tiles else torch.zeros((0, 2), dtype=torch.int32, device=DEV),
    num_prefill_tiles=len(tiles), prefill_wide_tiles=dev(wide).view(-1, 2) if wide else None, num_prefill_wide_tiles=len(wide),
    decode_items=dev(dec) if dec else torch.zeros(0, dtype=torch.int32, device=DEV),
    num_decode=len(dec), max_ctx_len=max_ctx, scratch=None)
  return qkv.to(DEV), kv.to(DEV), torch.from_numpy(bt).to(DEV), batch


def tol(dtype: torch.dtype) -> float:
  return 2e-5 if dtype == torch.float32 else 2e-2
