"""Pins the oracle to the reference's own CUDA kernels, compiled from the
reference checkout into oracle/_ref/ (oracle/build_ref.py) and run on the same
GPU.  The reference orders neighbors, samples and cells with atomics, so those
are compared as sets; keys, tube ranges and counts are compared exactly.
Skipped where the compiled reference kernels are not present."""
import numpy as np
import pytest

import oracle as orc
from oracle import pylib_ref as pr
from oracle import ref_kernels as ref
from tensorflow_graphics_point_clouds_b200 import synthetic

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref.available(), reason="oracle/_ref was not built")]
F32 = np.float32


def close(x, y, rel=1e-4):
  x = np.asarray(x, np.float64); y = np.asarray(y, np.float64)
  scale = np.maximum(np.abs(y), np.sqrt(np.mean(y * y)))
  assert np.all(np.abs(x - y) <= rel * scale + 1e-30), np.abs(x - y).max()


@pytest.fixture(scope="module")
def case():
  pts, bid = synthetic.surface_clouds(4, seed=1, min_points=20000, max_points=40000)
  radius = 0.05
  grid = pr.Grid(pts, bid, 4, radius)
  neigh = pr.Neighborhood(grid, radius)
  return pts, bid, radius, grid, neigh


def test_keys_and_tube_ranges_equal_reference_kernels(case):
  pts, bid, radius, grid, _ = case
  keys, _ = ref.compute_keys(pts, bid, grid.scaled_aabb_min, grid.num_cells, grid.inv_cell_sizes)
  assert np.array_equal(keys, grid.keys)            # oracle with the fused multiply-add
  ds, _ = ref.build_grid_ds(grid.sorted_keys, grid.num_cells, 4)
  assert np.array_equal(ds, grid.get_ds())


def test_keys_on_many_points_settle_the_rounding_convention():
  """2 million coordinates at three cell sizes: the reference kernel must agree
  with the fused form everywhere (the unfused form differs on a few points)."""
  pts, bid = synthetic.uniform_clouds(8, 65536, seed=2)
  for cell in (0.079, 0.05, 0.025):
    grid = pr.Grid(pts, bid, 8, cell, fused=True)
    keys, _ = ref.compute_keys(pts, bid, grid.scaled_aabb_min, grid.num_cells, grid.inv_cell_sizes)
    assert np.array_equal(keys, grid.keys)


def test_neighbor_sets_equal_reference_kernels(case):
  pts, bid, radius, grid, neigh = case
  inv_r = np.repeat(F32(1) / F32(radius), 3)
  ranges, nb, _ = ref.find_neighbors(grid.sorted_points, grid.sorted_batch_ids, grid.sorted_points,
                                     grid.sorted_keys, grid.get_ds(), grid.num_cells,
                                     grid.scaled_aabb_min, grid.inv_cell_sizes, inv_r,
                                     capacity=len(neigh.neighbors) + 1000)
  assert np.array_equal(ranges, neigh.ranges)        # same count for every sample
  assert len(nb) == len(neigh.neighbors)
  # same pairs: sort the reference's atomically placed lists into canonical order
  order = np.lexsort((nb[:, 0], nb[:, 1]))
  assert np.array_equal(nb[order], neigh.neighbors)


def test_pdf_and_gradients_match_reference_kernels(case):
  pts, bid, radius, grid, neigh = case
  inv_bw = np.repeat(F32(1 / 0.2), 3); inv_r = np.repeat(F32(1) / F32(radius), 3)
  rng = np.random.default_rng(3)
  g = rng.standard_normal(len(pts)).astype(F32)
  pdf, grads, _ = ref.compute_pdf(grid.sorted_points, neigh.neighbors, neigh.ranges, inv_bw, inv_r,
                                  0, g)
  close(orc.compute_pdf(grid.sorted_points, neigh.neighbors, neigh.ranges, inv_bw, inv_r, 0), pdf)
  # (the reference scatters every term with atomicAdd in arbitrary order,
  # compute_pdf_kernels.cu.cc:187-213; measured difference 2.8e-6)
  close(orc.compute_pdf_pt_grads(grid.sorted_points, neigh.neighbors, neigh.ranges, inv_bw, inv_r,
                                 g, 0), grads)


@pytest.mark.parametrize("c,k", [(8, 16), (32, 8), (3, 32)])
def test_basis_proj_matches_reference_kernels(c, k):
  rng = np.random.default_rng(c + k)
  pts, bid = synthetic.uniform_clouds(3, 3000, seed=9)
  grid = pr.Grid(pts, bid, 3, 0.1)
  neigh = pr.Neighborhood(grid, 0.1, pts, bid)
  m = len(neigh.neighbors)
  basis = rng.standard_normal((m, k)).astype(F32)
  feat = rng.standard_normal((len(pts), c)).astype(F32)
  out, _, _, _ = ref.basis_proj(basis, feat, neigh.original_neigh_ids, neigh.ranges)
  mine = orc.basis_proj(basis, feat, neigh.original_neigh_ids, neigh.ranges)
  close(mine, out)
  g = rng.standard_normal(out.shape).astype(F32)
  _, db, df, _ = ref.basis_proj(basis, feat, neigh.original_neigh_ids, neigh.ranges, g)
  mdb, mdf = orc.basis_proj_grads(basis, feat, neigh.original_neigh_ids, neigh.ranges, g)
  close(mdb, db)
  close(mdf, df)


def test_sampling_sets_equal_reference_kernels(case):
  pts, bid, radius, grid, neigh = case
  p, b, idx, _ = ref.sampling(grid.sorted_points, grid.sorted_batch_ids, grid.sorted_keys,
                              grid.num_cells, neigh.neighbors, neigh.ranges, 0)
  mp, mb, midx = orc.sampling(grid.sorted_points, grid.sorted_batch_ids, grid.sorted_keys,
                              grid.num_cells, neigh.neighbors, neigh.ranges, 0)
  assert np.array_equal(np.sort(idx), midx)          # same Poisson-disk sample set
  order = np.argsort(idx)
  assert np.array_equal(p[order], mp) and np.array_equal(b[order], mb)
  p, b, _, _ = ref.sampling(grid.sorted_points, grid.sorted_batch_ids, grid.sorted_keys,
                            grid.num_cells, neigh.neighbors, neigh.ranges, 1)
  mp, mb, _ = orc.sampling(grid.sorted_points, grid.sorted_batch_ids, grid.sorted_keys,
                           grid.num_cells, neigh.neighbors, neigh.ranges, 1)
  assert len(p) == len(mp)
  # the reference's cell order is arbitrary: compare as sorted rows
  order_r = np.lexsort((p[:, 2], p[:, 1], p[:, 0], b))
  order_m = np.lexsort((mp[:, 2], mp[:, 1], mp[:, 0], mb))
  assert np.array_equal(b[order_r], mb[order_m])
  close(p[order_r], mp[order_m])
