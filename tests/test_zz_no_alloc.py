"""The neighbor count pass that brings its own scratch.

tfgpc_find_neighbors_count_static is for hosts that cannot hand the library a
temporary device buffer (a framework that owns all device memory, a service
with its budget already committed): its scan scratch is a fixed array inside
the library.  This test calls it through the C ABI three times in a row, on
different clouds, and checks ranges and pair count against the regular entry
point, bit for bit.  Every call runs on the leftovers of the one before, which
must not matter: the sequence is a scan over several tiles, one over a single
tile, and again one over several tiles (whose tile sums then sit on stale
ones).  The file sorts last so that a run stopping at the first
failure has already been through every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from tensorflow_graphics_point_clouds_b200 import _lib, pc
from tensorflow_graphics_point_clouds_b200._lib import c_i64, c_int, c_sz, ptr

pytestmark = pytest.mark.gpu


def count_both(grid, samples, sample_bids, radius):
  """Runs the workspace entry point and the static one on the same inputs."""
  lib = _lib.lib()
  dev = samples.device
  ns, d = samples.shape
  inv_r = torch.full((d,), 1.0 / radius, device=dev)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  common = (stream, c_int(d), c_i64(ns), ptr(samples), ptr(sample_bids),
            c_i64(grid._sorted_points.shape[0]), ptr(grid._sorted_points), ptr(grid._sorted_keys),
            ptr(grid.get_DS()), c_i64(grid._batch_size), ptr(grid._num_cells),
            ptr(grid._scaled_aabb_min), ptr(grid._inv_cell_sizes), ptr(inv_r), c_int(0))
  nbytes = lib.tfgpc_find_neighbors_workspace_bytes(c_i64(ns))
  ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
  ref_ranges = torch.empty(ns, dtype=torch.int32, device=dev)
  ref_total = c_i64(0)
  _lib.check(lib.tfgpc_find_neighbors_count(*common, ptr(ref_ranges), ptr(ws), c_sz(nbytes),
                                            ctypes.byref(ref_total)))
  got_ranges = torch.empty(ns, dtype=torch.int32, device=dev)
  got_total = c_i64(0)
  _lib.check(lib.tfgpc_find_neighbors_count_static(*common, ptr(got_ranges),
                                                   ctypes.byref(got_total)))
  return ref_ranges, ref_total.value, got_ranges, got_total.value


def test_static_scratch_count_matches_workspace_count_on_calls_in_a_row():
  rng = np.random.default_rng(77)
  for n_pts, n_smp, radius in ((20000, 9000, 0.05), (3000, 700, 0.2), (15000, 13000, 0.07)):
    pts = torch.from_numpy(rng.uniform(0, 1, (n_pts, 3)).astype(np.float32)).cuda()
    bid = torch.from_numpy(rng.integers(0, 4, n_pts).astype(np.int32)).cuda()
    smp = torch.from_numpy(rng.uniform(0, 1, (n_smp, 3)).astype(np.float32)).cuda()
    sbid = torch.from_numpy(rng.integers(0, 4, n_smp).astype(np.int32)).cuda()
    grid = pc.Grid(pc.PointCloud(pts, bid, 4), radius)
    ref_ranges, ref_total, got_ranges, got_total = count_both(grid, smp, sbid, radius)
    assert got_total == ref_total and ref_total > 0
    assert torch.equal(got_ranges, ref_ranges)     # integer output: bit-exact


def test_static_scratch_count_rejects_oversized_calls():
  lib = _lib.lib()
  limit = lib.tfgpc_find_neighbors_static_max_samples()
  assert limit == 1 << 24
  total = c_i64(0)
  rc = lib.tfgpc_find_neighbors_count_static(
      None, c_int(3), c_i64(limit + 1), None, None, c_i64(0), None, None, None, c_i64(1), None,
      None, None, None, c_int(0), None, ctypes.byref(total))
  assert rc == 1
  assert b"at most" in lib.tfgpc_last_error()
