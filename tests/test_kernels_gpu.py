"""Each CUDA kernel alone against its PyTorch statement (tests/torch_ops.py), at sizes other than the
tiny models': widths and vocabularies that are no power of two, head sizes in steps of 16, odd head
counts and groups, small and large pages."""
import math

import numpy as np
import pytest
import torch

import torch_ops as ref
from gpu_helpers import DEV, make_attention_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
  from miniinfer_b200.kernels import ops as o
  o.common_lib()
  return o


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
  g = torch.Generator().manual_seed(seed)
  return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def test_fails_loudly_on_cpu_tensors(ops):
  with pytest.raises(ops.KernelError, match="CUDA"):
    ops.silu_mul(torch.zeros(2, 4), torch.zeros(2, 8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,T", [(1000, 136, 37), (17, 1024, 3)])
def test_embedding(ops, dtype, V, H, T):
  table = rnd(V, H, dtype=dtype)
  ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
  out = torch.empty(T, H, device=DEV)
  ops.embedding(out, table, ids)
  assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,eps", [(5, 200, 1e-5), (3, 1024, 1e-6), (2, 5120, 1e-6), (1, 7, 1e-3),
                                     (300, 1024, 1e-6), (257, 200, 1e-5), (260, 520, 1e-6), (256, 4096, 1e-6)])   # many rows
def test_add_rmsnorm(ops, dtype, T, H, eps):
  w = 1 + 0.1 * rnd(H, seed=1)
  for delta_on, rows_on, wb in ((True, False, True), (False, False, True), (True, True, False), (False, True, False)):
    resid = rnd(T, H, seed=2)
    delta = rnd(T, H, dtype=dtype, seed=3) if delta_on else None
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV) if rows_on else None
    R = 2 if rows_on else T
    out, out_ref = torch.empty(R, H, dtype=dtype, device=DEV), torch.empty(R, H, dtype=dtype, device=DEV)
    r1, r2 = resid.clone(), resid.clone()
    ops.add_rmsnorm(out, r1, delta, w, eps, rows, wb)
    ref.add_rmsnorm(out_ref, r2, delta, w, eps, rows, wb)
    assert torch.allclose(r1, r2, atol=1e-6), "residual"
    assert torch.allclose(out.float(), out_ref.float(), atol=2e-5 if dtype == torch.float32 else 2e-2, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    if not wb:
      assert torch.equal(r1, resid)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (33, 130, 70), (257, 100, 333), (64, 1000, 96)])
def test_linear_float32_is_true_float32_and_row_invariant(ops, M, N, K):
  x, w = rnd(M, K, seed=1), rnd(N, K, seed=2)
  out = torch.empty(M, N, device=DEV)
  ops.linear(out, x, w)
  exact = (x.double() @ w.double().t())
  # TF32 would err by ~1e-3 here; true fp32 stays within a few ulp of the exact sum
  assert (out.double() - exact).abs().max() < 1e-5 * math.sqrt(K) * 4
  one = torch.empty(1, N, device=DEV)
  ops.linear(one, x[M // 2:M // 2 + 1].contiguous(), w)
  assert torch.equal(one[0], out[M // 2]), "a row's value must not depend on the other rows"


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("N,K", [(24, 64), (1000, 136), (4096, 1024), (333, 2048), (8, 8),
                                 (6144, 512), (5000, 520)])     # a little more than 296 blocks of 16 rows: 24 rows per warp
def test_linear_bf16_few_rows(ops, out_dtype, N, K):
  w = rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.05)
  xs = rnd(64, K, dtype=torch.bfloat16, seed=1)
  full = {}
  for M in (64, 16, 1, 3, 8, 9, 17, 33):
    x = xs[:M].contiguous()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear(out, x, w, force_skinny=True)
    exact = x.float() @ w.float().t()
    err = (out.float() - exact).abs().max().item()
    bound = (1e-4 if out_dtype == torch.float32 else 1e-2) * max(1.0, exact.abs().max().item())
    assert err <= bound, (M, err, bound)
    # up to 16 rows (the sizes the engine gives this kernel) the sums over K are split one way,
    # above another; inside each class a row's value must not depend on the other rows
    cls = M <= 16
    if cls not in full:
      full[cls] = out
    else:
      assert torch.equal(out, full[cls][:M]), "a row's value must not depend on the other rows"
    routed = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear(routed, x, w)                      # above 16 rows: the library product
    if M <= 16:
      assert torch.equal(routed, out)
    else:
      assert (routed.float() - exact).abs().max().item() <= bound, M


def test_linear_bf16_many_rows_and_float32_logits(ops):
  x = rnd(200, 136, dtype=torch.bfloat16, seed=1)
  w = rnd(1000, 136, dtype=torch.bfloat16, seed=2, scale=0.05)
  exact = x.float() @ w.float().t()
  out = torch.empty(200, 1000, dtype=torch.bfloat16, device=DEV)
  ops.linear(out, x, w)
  assert (out.float() - exact).abs().max() < 2e-2 * exact.abs().max()
  out32 = torch.empty(200, 1000, dtype=torch.float32, device=DEV)
  ops.linear(out32, x, w)
  assert (out32 - exact).abs().max() < 1e-4 * max(1.0, exact.abs().max().item())
  for M in (2, 20):
    with pytest.raises(ops.KernelError, match="multiple of 8"):
      ops.linear(torch.empty(M, 5, dtype=torch.bfloat16, device=DEV), rnd(M, 12, dtype=torch.bfloat16), rnd(5, 12, dtype=torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,P,T", [(6, 2, 48, 8, 23), (4, 4, 16, 16, 23), (16, 8, 128, 64, 23), (3, 1, 256, 32, 23),
                                             (16, 8, 128, 64, 200), (5, 3, 128, 16, 77), (3, 1, 256, 32, 100),    # many tokens: the wide kernels
                                             (5, 3, 128, 16, 1300), (40, 4, 128, 64, 700)])   # several tokens per block; more than 32 heads
def test_qk_norm_rope_store(ops, dtype, nh, nkv, hd, P, T):
  pages, max_pos = max(9, -(-T // P) + 2), 300
  g = torch.Generator().manual_seed(4)
  for norm_on, rope_on, store_on in ((True, True, True), (False, True, True), (True, False, False), (True, True, False)):
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=5)
    qw, kw = (1 + 0.1 * rnd(hd, seed=6), 1 + 0.1 * rnd(hd, seed=7)) if norm_on else (None, None)
    rot = hd if hd != 48 else 32                              # a partial rotation for one case
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))
    fr = torch.outer(torch.arange(max_pos).float(), inv)
    table = torch.cat((fr.cos(), fr.sin()), -1).to(DEV) if rope_on else None
    pos = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32).to(DEV)
    slot = torch.randperm(pages * P, generator=g)[:T].to(torch.int32).to(DEV)
    slot[3] = -1                                              # a padded token stores nothing
    kv1 = torch.zeros(pages, 2, nkv, P, hd, dtype=dtype, device=DEV)
    kv2 = kv1.clone()
    a, b = qkv.clone(), qkv.clone()
    ops.qk_norm_rope_store(a, qw, kw, table, pos, slot if store_on else None, kv1 if store_on else None, nh, nkv, hd, 1e-5)
    ref.qk_norm_rope_store(b, qw, kw, table, pos, slot if store_on else None, kv2 if store_on else None, nh, nkv, hd, 1e-5)
    t = 3e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(a.float(), b.float(), atol=t, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    assert torch.allclose(kv1.float(), kv2.float(), atol=t, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    if store_on:
      assert kv1.abs().sum() > 0


CASES = [
  # (items (ctx, new), nh, nkv, hd, page, window)
  ([(37, 37), (9, 1), (70, 5), (130, 1)], 6, 2, 48, 8, None),
  ([(64, 64), (65, 1), (128, 2), (1, 1)], 4, 4, 16, 16, None),
  ([(300, 77), (257, 1), (64, 1)], 16, 8, 128, 64, None),
  ([(200, 150), (90, 1), (41, 2), (333, 1)], 6, 2, 32, 8, 40),
  ([(129, 129), (100, 1)], 5, 1, 64, 64, 64),
  ([(50, 3)], 2, 1, 256, 32, None),


  # more query heads per kv head than one pass of the decode kernel takes; long contexts; many splits
  ([(2100, 1), (1000, 1), (257, 1), (2048, 1), (1, 1), (640, 1), (300, 300), (511, 2)], 24, 2, 64, 64, None),
  ([(900, 1), (1500, 1), (77, 1)], 7, 7, 128, 16, 300),
  ([(700, 500), (64, 64), (1200, 130)], 4, 2, 128, 64, None),
  ([(333, 333), (100, 1)], 3, 1, 80, 8, 50),
  ([(150, 1), (150, 150)], 2, 2, 256, 64, None),
  ([(260, 1), (150, 150)], 8, 1, 16, 32, None),
  # exactly 8 and 16 query heads per kv head in the TMA decode kernel (one full pass, two full passes)
  ([(500, 1), (70, 1), (64, 1)], 16, 2, 128, 64, None),
  ([(300, 1), (129, 1)], 16, 1, 64, 64, 100),
  # the tcgen05 prefill kernel: one head per kv head (128 tokens of one head per block), head size 128;
  # a long portion that starts inside the prompt, with a window that cuts its first key tiles; one key tile only
  ([(700, 300), (130, 129), (2, 2)], 3, 3, 128, 64, None),
  ([(2500, 1100), (200, 1)], 4, 2, 128, 128, 700),
  ([(100, 100)], 6, 1, 64, 64, None),
  # long prompts: ten and more key tiles per block of the tcgen05 prefill kernel, 64-token and 128-token blocks
  ([(1500, 700), (1100, 1100)], 4, 2, 128, 64, None),
  ([(1300, 1300), (40, 1)], 3, 1, 64, 64, None),
]


@pytest.mark.parametrize("mode", ["float32", "bfloat16", "bfloat16-generic"])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_attention_over_pages(ops, mode, case):
  dtype = torch.float32 if mode == "float32" else torch.bfloat16
  items, nh, nkv, hd, P, window = CASES[case]
  qkv, kv, bt, batch = make_attention_case(items, nh, nkv, hd, P, dtype, seed=case)
  T = qkv.shape[0]
  out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
  want = torch.empty_like(out)
  ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, window, force_generic=mode.endswith("generic"))
  ref.attention(want, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, window)
  assert torch.isfinite(out.float()).all()
  assert (out.float() - want.float()).abs().max() < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("nh,nkv", [(16, 1), (32, 4), (24, 2)])
def test_decode_attention_many_requests_long_contexts_wide_groups(ops, nh, nkv):
  """Sixteen, eight and twelve query heads per kv head, 40 requests of 2048 and more tokens: every block of
  the decode kernels gets many key tiles.  No bounded wait may run out (the call raises if one does)."""
  items = [(2048 + 37 * i, 1) for i in range(40)]
  qkv, kv, bt, batch = make_attention_case(items, nh, nkv, 128, 64, torch.bfloat16, seed=3, num_slots=48)
  out = torch.full((len(items), nh * 128), float("nan"), dtype=torch.bfloat16, device=DEV)
  want = torch.empty_like(out)
  ops.attention(out, qkv, kv, bt, batch, nh, nkv, 128, 128 ** -0.5, None)
  ref.attention(want, qkv, kv, bt, batch, nh, nkv, 128, 128 ** -0.5, None)
  assert torch.isfinite(out.float()).all()
  assert (out.float() - want.float()).abs().max() < 2e-2


@pytest.mark.parametrize("cluster", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(16, 8, 128, None), (8, 1, 64, None), (3, 3, 128, 700), (4, 2, 256, None)])
def test_decode_attention_in_clusters(ops, monkeypatch, cluster, nh, nkv, hd, window):
  """The cluster-scheduled decode kernel at every cluster size, on requests from one token to several
  thousand: with one block per (request, kv head) a block has far more tiles than its ring has stages, so
  every stage is used many times; with sixteen most blocks of the short requests have no tile at all."""
  monkeypatch.setenv("MINIINFER_B200_DECODE_CLUSTER", str(cluster))
  items = [(3000, 1), (1, 1), (64, 1), (65, 1), (1500, 1), (700, 1), (2049, 1)]
  qkv, kv, bt, batch = make_attention_case(items, nh, nkv, hd, 64, torch.bfloat16, seed=cluster, num_slots=8)
  out = torch.full((len(items), nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
  want = torch.empty_like(out)
  for _ in range(3):                                   # the same launch again: nothing is left behind between launches
    out.fill_(float("nan"))
    ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, window)
  ref.attention(want, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, window)
  assert torch.isfinite(out.float()).all()
  assert (out.float() - want.float()).abs().max() < 2e-2


@pytest.mark.parametrize("cluster", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("nh,nkv,window,with_norm,with_table,writes,P", [(16, 8, None, True, True, True, 64), (6, 2, 700, True, True, True, 64),
                                                                         (8, 8, None, False, True, True, 128), (4, 2, None, True, False, True, 64),
                                                                         (16, 8, None, True, True, False, 64), (16, 2, 100, True, True, True, 256)])
def test_decode_attention_that_norms_rotates_and_stores_itself(ops, monkeypatch, cluster, nh, nkv, window, with_norm, with_table, writes, P):
  """A step of decode tokens through the one kernel that norms and rotates q and k, stores the new token's k and v
  and attends, against the two kernels it stands for: the same output rows and the same cache, bit for bit, at every
  cluster size, with and without norm weights, rotation table, window and cache store, pages of 64 to 256 tokens,
  one to eight query heads per kv head."""
  hd = 128
  monkeypatch.setenv("MINIINFER_B200_DECODE_CLUSTER", str(cluster))
  items = [(3000, 1), (1, 1), (64, 1), (65, 1), (1500, 1), (700, 1), (2049, 1), (128, 1)]
  qkv0, kv0, bt, batch = make_attention_case(items, nh, nkv, hd, P, torch.bfloat16, seed=cluster, num_slots=9)
  qw = (1 + 0.1 * rnd(hd, seed=3)) if with_norm else None
  kw = (1 + 0.1 * rnd(hd, seed=4)) if with_norm else None
  table = None
  if with_table:
    ang = torch.arange(3100, device=DEV)[:, None].float() * (10000.0 ** (-torch.arange(hd // 2, device=DEV).float() / (hd // 2)))[None, :]
    table = torch.cat((ang.cos(), ang.sin()), dim=1).contiguous()
  slots = torch.tensor([int(bt[int(batch.seq_slot[b]), (c - 1) // P]) * P + (c - 1) % P for b, (c, _) in enumerate(items)],
                       dtype=torch.int32, device=DEV)
  eps, scale = 1e-6, hd ** -0.5
  results = []
  for fused in ("1", "0"):
    monkeypatch.setenv("MINIINFER_B200_ROPE_IN_ATTENTION", fused)
    qkv, kv = qkv0.clone(), kv0.clone()
    out = torch.full((len(items), nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.rope_store_attention(out, qkv, qw, kw, table, batch.positions, slots, kv, writes, bt, batch, nh, nkv, hd, eps, scale, window)
    assert torch.isfinite(out.float()).all()
    results.append((out, kv, qkv))
  (out1, kv1, qkv1), (out0, kv0_, qkv0_) = results
  assert torch.equal(qkv1, qkv0), "the one kernel leaves the rows as the product wrote them"
  assert not torch.equal(qkv0_, qkv0) or not (with_norm or with_table)
  assert torch.equal(kv1, kv0_), "the cache"
  assert torch.equal(out1, out0), "the output rows"
  if not writes:
    assert torch.equal(kv1, kv0)
  # and both against the statements
  qkv, kv = qkv0.clone(), kv0.clone()
  ref.qk_norm_rope_store(qkv, qw, kw, table, batch.positions, slots if writes else None, kv if writes else None, nh, nkv, hd, eps)
  want = torch.empty_like(out1)
  ref.attention(want, qkv, kv, bt, batch, nh, nkv, hd, scale, window)
  assert (out1.float() - want.float()).abs().max() < 3e-2


@pytest.mark.parametrize("nh,nkv,P,window", [(16, 8, 64, None), (8, 2, 128, None), (16, 2, 64, 900), (6, 2, 64, None), (4, 4, 64, None)])
def test_prefill_attention_on_tcgen05_alone_and_in_pairs(ops, monkeypatch, nh, nkv, P, window):
  """The tcgen05 prefill kernel in its three forms - two blocks sharing 128 tokens of two heads (an even number of
  query heads per kv head), a block alone on the list of 128-token tiles, and a block alone without that list - on
  prompts and portions of many lengths, several launches in a row (the barriers' phases run on within a launch
  only): every form against the statement, and the forms that cut the keys the same way bit for bit."""
  hd = 128
  items = [(3000, 1700), (129, 129), (700, 2), (64, 64), (1, 1), (1300, 1153), (500, 1)]
  qkv, kv, bt, batch = make_attention_case(items, nh, nkv, hd, P, torch.bfloat16, seed=nh, num_slots=9)
  T = qkv.shape[0]
  want = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
  ref.attention(want, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, window)
  wide, n_wide = batch.prefill_wide_tiles, batch.num_prefill_wide_tiles
  outs = {}
  for form in ("pairs", "alone", "alone without the wide tiles"):
    monkeypatch.setenv("MINIINFER_B200_PREFILL_PAIRS", "1" if form == "pairs" else "0")
    batch.prefill_wide_tiles, batch.num_prefill_wide_tiles = (None, 0) if form.endswith("tiles") else (wide, n_wide)
    out = torch.empty_like(want)
    for _ in range(3):
      out.fill_(float("nan"))
      ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, window)
    assert torch.isfinite(out.float()).all(), form
    assert (out.float() - want.float()).abs().max() < 2e-2, form
    outs[form] = out
  if window is None:      # without a window every form walks the same key tiles from the first key on
    assert torch.equal(outs["pairs"], outs["alone"])
    assert torch.equal(outs["alone"], outs["alone without the wide tiles"])


def test_prefill_attention_pairs_blocks_on_a_large_step(ops, monkeypatch):
  """A step with more new tokens than ``ops.PREFILL_PAIRS_MIN_WIDE_TILES`` tiles of 128: nothing is forced, the
  blocks work in pairs; the same rows as from blocks that work alone, and as the statement's."""
  nh, nkv, hd, P = 4, 2, 128, 64
  items = [(6500, 6300), (300, 1)]
  qkv, kv, bt, batch = make_attention_case(items, nh, nkv, hd, P, torch.bfloat16, seed=11, num_slots=3)
  assert batch.num_prefill_wide_tiles >= ops.PREFILL_PAIRS_MIN_WIDE_TILES
  monkeypatch.delenv("MINIINFER_B200_PREFILL_PAIRS", raising=False)
  out = torch.full((qkv.shape[0], nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
  ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, None)
  monkeypatch.setenv("MINIINFER_B200_PREFILL_PAIRS", "0")
  alone = torch.empty_like(out)
  ops.attention(alone, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, None)
  want = torch.empty_like(out)
  ref.attention(want, qkv, kv, bt, batch, nh, nkv, hd, hd ** -0.5, None)
  assert torch.equal(out, alone)
  assert (out.float() - want.float()).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_and_respects_the_window_edge(ops, dtype):
  """Random data would hide a key that is skipped: make one key's score stand out."""
  nh, nkv, hd, P = 4, 2, 64, 16
  for window, far in ((None, 3), (None, 257), (100, 401), (100, 400)):
    ctx = 501
    qkv, kv, bt, batch = make_attention_case([(ctx, 1)], nh, nkv, hd, P, dtype, seed=1)
    slot = int(batch.seq_slot[0])
    page, off = int(bt[slot, far // P]), far % P
    q = qkv.float().view(1, -1, hd)
    kv[page, 0, :, off, :] = (q[0, :nh:nh // nkv] * 4.0).to(dtype)   # aligned with the group's first head
    kv[page, 1, :, off, :] = 7.0
    out = torch.empty((1, nh * hd), dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    ops.attention(out, qkv, kv, bt, batch, nh, nkv, hd, 1.0, window)
    ref.attention(want, qkv, kv, bt, batch, nh, nkv, hd, 1.0, window)
    assert (out.float() - want.float()).abs().max() < (1e-4 if dtype == torch.float32 else 5e-2)
    first_head = out.float()[0, :hd]
    visible = window is None or far > (ctx - 1) - window
    assert (first_head.mean() > 6.0) == visible, (window, far, first_head.mean())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,I", [(7, 176), (3, 3072), (1, 5)])
def test_silu_mul(ops, dtype, T, I):
  gu = rnd(T, 2 * I, dtype=dtype, scale=3.0)
  out, want = torch.empty(T, I, dtype=dtype, device=DEV), torch.empty(T, I, dtype=dtype, device=DEV)
  ops.silu_mul(out, gu)
  ref.silu_mul(want, gu)
  assert torch.allclose(out.float(), want.float(), atol=1e-6 if dtype == torch.float32 else 2e-2, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)


class _Scratch:
  def __init__(self):
    self.made = {}

  def buffer(self, name, shape, dtype):
    return torch.empty(shape, dtype=dtype, device=DEV)

  def zeros(self, name, n, dtype):
    if name not in self.made:
      self.made[name] = torch.zeros(n, dtype=dtype, device=DEV)
    return self.made[name]


@pytest.mark.parametrize("N,K,swiglu", [(6144, 4096, False), (4096, 4096, False), (3080, 4104, False), (3072, 4096, True),
                                          (12288, 2048, True), (2056, 6152, True),
                                          (12288, 4096, True), (10240, 5120, False), (5128, 8200, False)])   # sizes that the engine gives the tcgen05 streaming kernel
def test_few_rows_times_many_megabytes_of_weights(ops, N, K, swiglu):
  """The few-row product at the sizes of larger models (24 MB of weights and more) against the
  statement; a row's value must not depend on the other rows."""
  w = rnd((2 if swiglu else 1) * N, K, dtype=torch.bfloat16, seed=2, scale=0.03)
  xs = rnd(16, K, dtype=torch.bfloat16, seed=1)
  first = {}
  for M in (16, 8, 1, 5, 11):
    x = xs[:M].contiguous()
    want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    if swiglu:
      gu = torch.empty(M, 2 * N, dtype=torch.bfloat16, device=DEV)
      ref.linear(gu, x, w)
      ref.silu_mul(want, gu)
      ops.linear_swiglu(out, x, w, _Scratch())
    else:
      ref.linear(want, x, w)
      ops.linear(out, x, w)
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), (M, err)
    if M in (16, 8):
      first[M] = out
    else:
      assert torch.equal(out, first[16][:M]), "a row's value must not depend on the other rows"
  assert torch.equal(first[8], first[16][:8])


@pytest.mark.parametrize("N,K,swiglu,out_dtype", [(1000, 200, False, torch.bfloat16), (128, 64, False, torch.bfloat16),
                                                    (4096, 4096, False, torch.bfloat16), (18992, 264, False, torch.float32),
                                                    (300, 1032, True, torch.bfloat16), (3072, 1024, True, torch.bfloat16),
                                                    (70, 9000, False, torch.bfloat16), (8, 72, True, torch.bfloat16)])
def test_streaming_product_on_tcgen05(ops, N, K, swiglu, out_dtype):
  """The few-row product that deals the weight matrix out to the SMs in equal stretches (tcgen05, TMA), forced at
  sizes below its threshold too: widths that are no multiple of its tiles and slices, stretches that cut tiles
  (one tile for all SMs; many tiles), both outputs.  Against the statement; a row's value must not depend on the
  other rows nor on the call; the tile counters are left at zero."""
  w = rnd((2 if swiglu else 1) * N, K, dtype=torch.bfloat16, seed=2, scale=0.05)
  xs = rnd(16, K, dtype=torch.bfloat16, seed=1)
  first = None
  for M in (16, 1, 5, 8, 16):
    x = xs[:M].contiguous()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    if swiglu:
      gu = torch.empty(M, 2 * N, dtype=torch.bfloat16, device=DEV)
      want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
      ref.linear(gu, x, w)
      ref.silu_mul(want, gu)
      ops.linear_swiglu(out, x, w, _Scratch(), force_stream=True)
      want = want.float()
    else:
      want = x.float() @ w.float().t()
      ops.linear(out, x, w, force_stream=True)
    err = (out.float() - want).abs().max().item()
    bound = (1e-4 if out_dtype == torch.float32 else 2e-2) * max(1.0, want.abs().max().item())
    assert err <= bound, (M, err, bound)
    if first is None:
      first = out
    else:
      assert torch.equal(out, first[:M]), "a row's value must not depend on the other rows, nor on the call"
  parts, counters, status = ops._stream_ws[torch.cuda.current_device()]
  assert int(counters.abs().sum()) == 0 and int(status[0]) == 0


@pytest.mark.parametrize("I,K", [(24, 64), (3072, 1024), (1000, 136), (7, 8), (333, 2048)])
def test_linear_swiglu(ops, I, K):
  """The fused gate-and-up product against product + activation (which it must match up to the
  order of its K-sums), and a row's value must not depend on the other rows."""
  w = rnd(2 * I, K, dtype=torch.bfloat16, seed=2, scale=0.08)
  xs = rnd(100, K, dtype=torch.bfloat16, seed=1)
  full = {}
  for M in (64, 16, 1, 3, 8, 9, 17, 33, 100):       # 100 rows: the unfused path
    x = xs[:M].contiguous()
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    want = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ref.linear(gu, x, w)
    ref.silu_mul(want, gu)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(out, x, w, _Scratch(), force_skinny=True)
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), (M, err)
    cls = M <= 16
    if M in (64, 16):
      full[cls] = out
    elif M < 64:
      assert torch.equal(out, full[cls][:M]), "a row's value must not depend on the other rows"
    routed = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(routed, x, w, _Scratch())    # above 16 rows: library product, then the activation kernel
    if M <= 16:
      assert torch.equal(routed, out)
    else:
      assert (routed.float() - want.float()).abs().max().item() <= 2e-2 * max(1.0, want.float().abs().max().item()), M
  x32, w32 = xs[:5].float(), w.float()
  out32 = torch.empty(5, I, device=DEV)
  ops.linear_swiglu(out32, x32, w32, _Scratch())
  g = x32 @ w32.t()
  assert torch.allclose(out32, torch.nn.functional.silu(g[:, :I]) * g[:, I:], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("N,K", [(24, 64), (4096, 1024), (1000, 136), (1024, 3072), (6144, 4096), (5000, 520), (8, 8)])
def test_few_row_products_with_the_norm_and_the_residual_add_fused(ops, N, K):
  """The decode step's fused products against their statements (norm kernel, then product; product, then
  add): the values agree to bfloat16 rounding, a row's value does not depend on the other rows, and the
  residual rows beyond M are not touched."""
  w = rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.05)
  wn = 1 + 0.1 * rnd(K, seed=3)
  resid_k = rnd(16, K, seed=4, scale=2.0)
  xs = rnd(16, K, dtype=torch.bfloat16, seed=1)
  first_norm = first_add = None
  for M in (16, 8, 1, 5, 11):
    # norm in the prologue
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    want = torch.empty_like(out)
    ops.linear_normed(out, resid_k[:M].contiguous(), wn, 1e-6, w)
    ref.linear_normed(want, resid_k[:M].contiguous(), wn, 1e-6, w)
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), ("norm", M, err)
    if first_norm is None:
      first_norm = out
    else:
      assert torch.equal(out, first_norm[:M]), "a row's value must not depend on the other rows"
    # against the unfused kernels: the same products of the same rounded activations
    normed = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(normed, resid_k[:M].clone(), None, wn, 1e-6, None, False)
    two = torch.empty_like(out)
    ops.linear(two, normed, w)
    assert (out.float() - two.float()).abs().max().item() <= 1e-2 * max(1.0, want.float().abs().max().item())
    # residual add in the epilogue
    resid = rnd(16, N, seed=6)
    got = resid.clone()
    ops.linear_add(got[:M], xs[:M].contiguous(), w)
    want32 = resid.clone()
    ref.linear_add(want32[:M], xs[:M].contiguous(), w)
    assert torch.equal(got[M:], resid[M:])
    scale = max(1.0, (xs[:M].float() @ w.float().t()).abs().max().item())
    assert (got - want32).abs().max().item() <= 1e-2 * scale, ("add", M)
    if first_add is None:
      first_add = got
    else:
      assert torch.equal(got[:M], first_add[:M])


@pytest.mark.parametrize("I,K", [(24, 64), (3072, 1024), (1000, 136), (12288, 4096), (7, 8)])
def test_few_row_gate_and_up_product_with_the_norm_fused(ops, I, K):
  w = rnd(2 * I, K, dtype=torch.bfloat16, seed=2, scale=0.08)
  wn = 1 + 0.1 * rnd(K, seed=3)
  resid = rnd(16, K, seed=4, scale=2.0)
  first = None
  for M in (16, 8, 3):
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    want = torch.empty_like(out)
    ops.linear_swiglu_normed(out, resid[:M].contiguous(), wn, 1e-5, w)
    ref.linear_swiglu_normed(want, resid[:M].contiguous(), wn, 1e-5, w)
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), (M, err)
    if first is None:
      first = out
    else:
      assert torch.equal(out, first[:M])
  with pytest.raises(ops.KernelError, match="0..16"):
    ops.linear_swiglu_normed(torch.empty(17, I, dtype=torch.bfloat16, device=DEV), rnd(17, K), wn, 1e-5, w)


@pytest.mark.parametrize("mode", ["2", "1"])          # blocks in pairs, blocks alone
@pytest.mark.parametrize("I,K", [(24, 64), (3072, 1024), (1000, 136), (200, 72), (128, 4096)])
def test_linear_swiglu_many_rows(ops, I, K, mode, monkeypatch):
  """The tcgen05 product with the activation in its epilogue: tiles of 128 rows, edges in every
  direction, against product + activation; a row's value must not depend on the other rows."""
  monkeypatch.setenv("MINIINFER_B200_GEMM_TC", mode)
  w = rnd(2 * I, K, dtype=torch.bfloat16, seed=2, scale=0.08)
  xs = rnd(1400, K, dtype=torch.bfloat16, seed=1)
  scratch = _Scratch()
  first = None
  for M in (1400, 65, 128, 129, 384):     # 1400 rows: what the engine itself sends to this kernel
    x = xs[:M].contiguous()
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    want = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ref.linear(gu, x, w)
    ref.silu_mul(want, gu)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(out, x, w, scratch, force_tc=True)
    assert int(scratch.made["gemm_tc_status"][0]) == 0
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), (M, err)
    if first is None:
      first = out
    else:
      assert torch.equal(out, first[:M]), "a row's value must not depend on the other rows"


@pytest.mark.parametrize("mode", ["2", "1"])
@pytest.mark.parametrize("N,K", [(256, 64), (4096, 1024), (1000, 136), (8, 72), (384, 2048)])
def test_linear_tc(ops, N, K, mode, monkeypatch):
  monkeypatch.setenv("MINIINFER_B200_GEMM_TC", mode)
  w = rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.08)
  xs = rnd(300, K, dtype=torch.bfloat16, seed=1)
  scratch = _Scratch()
  for M in (300, 1, 128, 130):
    x = xs[:M].contiguous()
    want = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ref.linear(want, x, w)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(out, x, w, scratch)
    assert int(scratch.made["gemm_tc_status"][0]) == 0
    err = (out.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), (M, err)


def _sample(ops, logits, temp, k, p, seed, counter):
  R = logits.shape[0]
  out = torch.full((R,), -1, dtype=torch.int32, device=DEV)
  f = lambda v, dt: torch.tensor(v, dtype=dt, device=DEV)
  ops.sample(out, logits, f(temp, torch.float32), f(k, torch.int32), f(p, torch.float32), f(seed, torch.int64), f(counter, torch.int64))
  return out.tolist()


def test_sampler_greedy_and_ties(ops):
  logits = rnd(5, 1000, seed=3)
  logits[1, 700] = logits[1, 40] = 50.0                      # equal maxima: the lowest index wins
  logits[2, 999] = 60.0
  got = _sample(ops, logits, [0.0] * 5, [0] * 5, [1.0] * 5, [1] * 5, [0] * 5)
  assert got == logits.argmax(-1).tolist() and got[1] == 40 and got[2] == 999


@pytest.mark.parametrize("scale", [2.0, 12.0])       # 12: most scores lie too far under the best to win, and are passed over
@pytest.mark.parametrize("V", [1000, 151936])
def test_sampler_draws_match_the_statement(ops, V, scale):
  R = 6
  logits = rnd(R, V, seed=5, scale=scale)
  temp = [0.8, 1.0, 0.5, 1.3, 0.7, 0.0]
  k = [0, 20, 0, 50, 1, 0]
  p = [1.0, 1.0, 0.9, 0.6, 1.0, 1.0]
  seed = [11, 12, 13, 14, 15, 16]
  counter = [0, 5, 7, 1, 2, 3]
  got = _sample(ops, logits, temp, k, p, seed, counter)
  again = _sample(ops, logits, temp, k, p, seed, counter)
  assert got == again
  for r in range(R):
    if temp[r] == 0:
      assert got[r] == int(logits[r].argmax())
      continue
    sc = ref.gumbel_scores(logits[r], temp[r], k[r], p[r], seed[r], counter[r])
    assert torch.isfinite(sc[got[r]]), f"row {r}: token {got[r]} is outside the kept set"
    assert sc[got[r]] >= sc.max() - 1e-4, f"row {r}: score {sc[got[r]]} vs best {sc.max()}"
  assert got[4] == int(logits[4].argmax())                    # top_k = 1
  other = _sample(ops, logits, temp, k, p, seed, [c + 1 for c in counter])
  assert other[:4] != got[:4]


def test_sampler_follows_the_distribution(ops):
  logits = torch.tensor([[0.1, 2.0, 1.9, -1.0, 0.5, 0.3, -2.0]], device=DEV).repeat(64, 1)
  counts = torch.zeros(7)
  for c in range(40):
    for t in _sample(ops, logits, [1.0] * 64, [0] * 64, [1.0] * 64, list(range(64)), [c] * 64):
      counts[t] += 1
  pr = torch.softmax(logits[0].cpu(), -1)
  assert (counts / counts.sum() - pr).abs().max() < 0.03
  counts = torch.zeros(7)
  for t in _sample(ops, logits, [1.0] * 64, [3] * 64, [0.7] * 64, list(range(64)), [1] * 64):
    counts[t] += 1
  assert counts[[0, 3, 4, 5, 6]].sum() == 0                   # top-3 then top-p 0.7 keeps tokens 1 and 2
