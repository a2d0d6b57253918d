"""Plain PyTorch statements of the engine's device operations, one for each function of
``miniinfer_b200.kernels.ops`` and with the same arguments.

Two uses: (1) on the GPU, each CUDA kernel is compared with its statement here; (2) on the CPU,
``install(monkeypatch)`` puts these in place of the kernels so that the host-side logic of the
engine (cache manager, step metadata, scheduler, replay) can be tested without a device.  They are
test code only; the package itself has no implementation other than its CUDA kernels.

All arithmetic is float32 (float64 where noted) on whatever device the tensors are on.
"""

from __future__ import annotations

import math
from typing import Optional

import torch


def embedding(out, table, ids):
  out.copy_(table[ids.long()].float())


def add_rmsnorm(out, resid, delta, weight, eps, rows=None, write_back=True):
  idx = rows.long() if rows is not None else None
  x = resid if idx is None else resid[idx]
  if delta is not None:
    x = x + (delta if idx is None else delta[idx]).float()
    if write_back:
      if idx is None:
        resid.copy_(x)
      else:
        resid[idx] = x
  var = x.pow(2).mean(-1, keepdim=True)
  out.copy_((weight * (x * torch.rsqrt(var + eps))).to(out.dtype))


def linear(out, x, w, force_skinny=False):
  out.copy_((x.float() @ w.float().t()).to(out.dtype))


def _rms(resid, weight, eps):
  x = resid.float()
  return (weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))).to(torch.bfloat16)


def linear_normed(out, resid, norm_weight, eps, w):
  linear(out, _rms(resid, norm_weight, eps), w)


def linear_swiglu_normed(out, resid, norm_weight, eps, w):
  linear_swiglu(out, _rms(resid, norm_weight, eps), w, None)


def linear_add(resid, x, w):
  resid.add_((x.float() @ w.float().t()).to(torch.bfloat16).float())


def qk_norm_rope_store(qkv, q_weight, k_weight, cos_sin, positions, slot_mapping, kv_layer,
                       num_heads, num_kv_heads, head_dim, eps):
  T = qkv.shape[0]
  nh, nkv, hd = num_heads, num_kv_heads, head_dim
  x = qkv.float().view(T, nh + 2 * nkv, hd)
  q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]

  def norm(t, w):
    if w is None:
      return t
    return w * (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps))

  def rope(t):
    if cos_sin is None:
      return t
    rot = cos_sin.shape[1]
    cs = cos_sin[positions.long()]
    c, s = cs[:, None, :rot // 2], cs[:, None, rot // 2:]
    t1, t2, rest = t[..., :rot // 2], t[..., rot // 2:rot], t[..., rot:]
    return torch.cat((t1 * c - t2 * s, t2 * c + t1 * s, rest), dim=-1)

  q = rope(norm(q, q_weight))
  k = rope(norm(k, k_weight))
  res = torch.cat((q, k, v), dim=1).reshape(T, -1).to(qkv.dtype)
  qkv.copy_(res)
  if slot_mapping is not None and kv_layer is not None:
    P = kv_layer.shape[3]
    r = res.view(T, nh + 2 * nkv, hd)
    slot = slot_mapping.long()
    ok = slot >= 0
    page, off = (slot // P)[ok], (slot % P)[ok]
    kv_layer[page, 0, :, off, :] = r[ok, nh:nh + nkv]
    kv_layer[page, 1, :, off, :] = r[ok, nh + nkv:]


def attention(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale, window,
              force_generic=False):
  T = qkv.shape[0]
  nh, nkv, hd = num_heads, num_kv_heads, head_dim
  P = kv_layer.shape[3]
  g = nh // nkv
  q = qkv.float().view(T, -1, hd)[:, :nh]
  pos = batch.positions.tolist()
  item = batch.token_item.tolist()
  slots = batch.seq_slot.tolist()
  res = torch.zeros((T, nh, hd), dtype=torch.float32, device=qkv.device)
  for t in range(T):
    p = pos[t]
    lo = max(0, p - window + 1) if window else 0
    js = torch.arange(lo, p + 1, device=qkv.device)
    pages = block_table[slots[item[t]]].long()[js // P]
    k = kv_layer[pages, 0, :, js % P, :].float()          # [n, nkv, hd]
    v = kv_layer[pages, 1, :, js % P, :].float()
    k = k.repeat_interleave(g, dim=1)                     # [n, nh, hd]
    v = v.repeat_interleave(g, dim=1)
    s = torch.einsum("hd,nhd->hn", q[t], k) * scale
    pr = torch.softmax(s, dim=-1)
    res[t] = torch.einsum("hn,nhd->hd", pr, v)
  out.copy_(res.reshape(T, nh * hd).to(out.dtype))


def linear_swiglu(out, x, w, workspace, force_skinny=False, force_tc=False):
  gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype)
  linear(gu, x, w)
  silu_mul(out, gu)


def silu_mul(out, gate_up):
  I = out.shape[1]
  g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
  out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


_M = (1 << 64) - 1


def _mix64(x: int) -> int:
  x &= _M
  x ^= x >> 30
  x = (x * 0xBF58476D1CE4E5B9) & _M
  x ^= x >> 27
  x = (x * 0x94D049BB133111EB) & _M
  x ^= x >> 31
  return x


def gumbel_scores(logits_row, temperature, top_k, top_p, seed, counter):
  """The perturbed scores whose arg-max is the sampled token (float64), -inf where filtered out."""
  V = logits_row.numel()
  z = logits_row.double().cpu() / temperature
  if top_k and 0 < top_k < V:
    kth = torch.topk(z, top_k).values[-1]
    z = torch.where(z >= kth, z, torch.full_like(z, float("-inf")))
  if top_p < 1.0:
    pr = torch.softmax(z, dim=-1)
    sp, _ = torch.sort(pr, descending=True)
    before = torch.cumsum(sp, 0) - sp
    last = int((before < top_p).nonzero().max())
    z = torch.where(pr >= sp[last], z, torch.full_like(z, float("-inf")))
  key = _mix64((seed & _M) ^ _mix64(counter + 0x9E3779B97F4A7C15))
  u = torch.tensor([((_mix64(key ^ ((i * 0xD1342543DE82EF95) & _M)) >> 41) + 0.5) / (1 << 23) for i in range(V)],
                   dtype=torch.float64)
  return z - torch.log(-torch.log(u))


def sample(out, logits, temperature, top_k, top_p, seed, counter, workspace=None):
  R = logits.shape[0]
  for r in range(R):
    t = float(temperature[r])
    if t <= 0:
      out[r] = int(torch.argmax(logits[r].float()))
    else:
      sc = gumbel_scores(logits[r], t, int(top_k[r]), float(top_p[r]), int(seed[r]), int(counter[r]))
      out[r] = int(torch.argmax(sc))


def install(monkeypatch) -> None:
  """Puts the statements above in place of the CUDA kernels (CPU tests of the host-side logic)."""
  from miniinfer_b200.kernels import ops

  for name in ("embedding", "add_rmsnorm", "linear", "linear_swiglu", "qk_norm_rope_store", "attention", "silu_mul", "sample",
               "linear_normed", "linear_swiglu_normed", "linear_add"):
    monkeypatch.setattr(ops, name, globals()[name])
