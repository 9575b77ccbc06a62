"""Writes tests/golden/hot_path_small.npz: seeded inputs and the CPU oracle's
outputs for every op of the hot path on one small batch.

The reference itself cannot be run in this environment (its Python side needs
TensorFlow), so the vectors come from the oracle after it has been pinned to
the reference tests' known answers (tests/test_oracle_known_answers.py); they
freeze that state: a later change of the oracle or of the CUDA library that
moves any of these outputs is caught by tests/test_golden.py.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle as orc  # noqa: E402
from oracle import pylib_ref as pr  # noqa: E402
from tensorflow_graphics_point_clouds_b200 import synthetic  # noqa: E402

F32 = np.float32


def build():
  b, per, cin, k, cout, radius = 3, 160, 8, 8, 16, 0.2
  pts, bid = synthetic.uniform_clouds(b, per, seed=11)
  rng = np.random.default_rng(12)
  # shuffle so that clouds are interleaved (batch ids need not be sorted)
  order = rng.permutation(b * per)
  pts, bid = pts[order], bid[order]
  feat = rng.standard_normal((b * per, cin), dtype=F32)
  d_out = rng.standard_normal((b * per, cout), dtype=F32)
  w1, b1, wf = synthetic.mcconv_weights(13, 3, cin, cout, 1, k)
  grid = pr.Grid(pts, bid, b, radius)
  neigh = pr.Neighborhood(grid, radius, pts, bid)
  self_neigh = pr.Neighborhood(grid, radius)
  pdf = neigh.get_pdf(bandwidth=0.2, mode=0)
  basis, _, _ = pr.mcconv_basis(pts, pts, neigh, pdf, w1, b1, radius)
  out, x = pr.mcconv_forward(feat, basis, neigh, wf)
  d_wf, d_basis, d_feat, _ = pr.mcconv_backward(feat, basis, neigh, wf, x, d_out)
  pd_pts, pd_bid, pd_idx = pr.sample(self_neigh, 0)
  avg_pts, avg_bid, _ = pr.sample(self_neigh, 1)
  return dict(
      batch_size=b, radius=F32(radius), points=pts, batch_ids=bid, features=feat, d_out=d_out,
      w1=w1, b1=b1, wf=wf, num_cells=grid.num_cells, keys=grid.keys,
      sorted_indices=grid.sorted_indices, sorted_keys=grid.sorted_keys, ds=grid.get_ds(),
      ranges=neigh.ranges, neighbors=neigh.neighbors, self_ranges=self_neigh.ranges,
      self_neighbors=self_neigh.neighbors, point_pdf=neigh.point_pdf, basis=basis,
      projection=x, out=out, d_wf=d_wf, d_basis=d_basis, d_feat=d_feat,
      poisson_indices=pd_idx, poisson_batch_ids=pd_bid, average_points=avg_pts,
      average_batch_ids=avg_bid)


if __name__ == "__main__":
  data = build()
  path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hot_path_small.npz")
  np.savez_compressed(path, **data)
  print("wrote", path, os.path.getsize(path), "bytes")
