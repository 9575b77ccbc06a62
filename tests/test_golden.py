"""Committed golden vectors (tests/golden/hot_path_small.npz, written by
tests/golden/make_golden.py): the oracle must still reproduce them on CPU, and
the CUDA library must match them on the GPU (integers bit-exact, floats within
rel 1e-4)."""
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "hot_path_small.npz")

INT_KEYS = ["num_cells", "keys", "sorted_indices", "sorted_keys", "ds", "ranges", "neighbors",
            "self_ranges", "self_neighbors", "poisson_indices", "poisson_batch_ids",
            "average_batch_ids"]
FLOAT_KEYS = ["point_pdf", "basis", "projection", "out", "d_wf", "d_basis", "d_feat",
              "average_points"]


def close(x, y, rel=1e-4):
  x = np.asarray(x, np.float64); y = np.asarray(y, np.float64)
  scale = np.maximum(np.abs(y), np.sqrt(np.mean(y * y)))
  assert np.all(np.abs(x - y) <= rel * scale + 1e-30)


@pytest.fixture(scope="module")
def golden():
  return dict(np.load(GOLDEN))


def test_oracle_reproduces_golden(golden):
  spec = importlib.util.spec_from_file_location("make_golden",
                                                os.path.join(HERE, "golden", "make_golden.py"))
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  fresh = mod.build()
  for k in INT_KEYS:
    assert np.array_equal(fresh[k], golden[k]), k
  for k in FLOAT_KEYS:
    close(fresh[k], golden[k], rel=1e-6)


@pytest.mark.gpu
def test_cuda_library_matches_golden(golden):
  import torch
  from tensorflow_graphics_point_clouds_b200 import mcconv, pc

  def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()

  b, radius = int(golden["batch_size"]), float(golden["radius"])
  cloud = pc.PointCloud(t(golden["points"]), t(golden["batch_ids"]), b)
  grid = pc.Grid(cloud, radius)
  assert np.array_equal(grid._num_cells.cpu().numpy(), golden["num_cells"])
  assert np.array_equal(grid._cur_keys.cpu().numpy(), golden["keys"])
  assert np.array_equal(grid._sorted_indices.cpu().numpy(), golden["sorted_indices"])
  assert np.array_equal(grid._sorted_keys.cpu().numpy(), golden["sorted_keys"])
  assert np.array_equal(grid.get_DS().cpu().numpy(), golden["ds"])
  neigh = pc.Neighborhood(grid, radius, cloud)
  assert np.array_equal(neigh._samples_neigh_ranges.cpu().numpy(), golden["ranges"])
  assert np.array_equal(neigh._neighbors.cpu().numpy(), golden["neighbors"])
  self_neigh = pc.Neighborhood(grid, radius)
  assert np.array_equal(self_neigh._samples_neigh_ranges.cpu().numpy(), golden["self_ranges"])
  assert np.array_equal(self_neigh._neighbors.cpu().numpy(), golden["self_neighbors"])
  layer = mcconv.MCConv(t(golden["w1"]), t(golden["b1"]), t(golden["wf"]),
                        golden["features"].shape[1])
  out = layer.forward(t(golden["features"]), cloud, cloud, radius, neighborhood=neigh)
  dfeat, dw1, db1, dwf = layer.backward(t(golden["d_out"]))
  layer._op.check_status()
  close(neigh.point_pdf().cpu().numpy(), golden["point_pdf"])
  close(layer.saved_basis().cpu().numpy(), golden["basis"])
  close(out.cpu().numpy(), golden["out"])
  close(dfeat.cpu().numpy(), golden["d_feat"])
  close(dwf.cpu().numpy(), golden["d_wf"])
  pts, idx = pc.sample(self_neigh, "poisson")
  assert np.array_equal(idx.cpu().numpy(), golden["poisson_indices"])
  assert np.array_equal(pts._batch_ids.cpu().numpy(), golden["poisson_batch_ids"])
  avg, _ = pc.sample(self_neigh, "average")
  assert np.array_equal(avg._batch_ids.cpu().numpy(), golden["average_batch_ids"])
  close(avg._points.cpu().numpy(), golden["average_points"])
