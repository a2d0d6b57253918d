"""The block table on the device is what the host's table held when `sync()` was called, even if the
upload runs later than changes the host makes afterwards (a step that is launched while the step
before still runs)."""
import pytest
import torch

from gpu_helpers import DEV

pytestmark = pytest.mark.gpu


def test_an_upload_reads_the_table_as_it_was_when_it_was_queued():
  from miniinfer_b200.cache import KVCacheManager, PagedKVSpec
  cache = KVCacheManager([PagedKVSpec(1, 16)], 8, 64, 4, 512, torch.bfloat16, DEV)
  group = cache.paged_groups[0]
  cache.admit("a")
  cache.append("a", 20)                      # three pages
  cache.commit("a", 20)
  slot = cache.slot_of("a")
  want = group.block_table_host[slot].copy()
  # keep the stream busy so that the upload is still waiting when the host goes on
  busy = torch.randn(4096, 4096, device=DEV)
  for _ in range(30):
    busy = busy @ busy * 1e-3
  cache.sync()
  for rounds in range(12):                   # more changes and uploads than there are snapshots
    cache.append("a", 8)
    cache.commit("a", 8)
  torch.cuda.synchronize()
  # nothing was uploaded after the first sync, so the device still holds the table of that moment
  assert group.block_table[slot].cpu().numpy().tolist() == want.tolist()
  cache.sync()
  torch.cuda.synchronize()
  assert group.block_table[slot].cpu().numpy().tolist() == group.block_table_host[slot].tolist()
  assert group.block_table_host[slot].tolist() != want.tolist()
  # many uploads in a row, each followed by a change: every one delivers its own snapshot
  seen = []
  for _ in range(20):
    cache.append("a", 8)
    cache.commit("a", 8)
    cache.sync()
    seen.append((group.block_table_host[slot].copy(), group.block_table[slot].clone()))   # the clone is queued behind the upload
  torch.cuda.synchronize()
  for host_row, dev_row in seen:
    assert dev_row.cpu().numpy().tolist() == host_row.tolist()
