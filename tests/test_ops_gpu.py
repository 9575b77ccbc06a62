"""Parity of the CUDA library (through the C ABI) with the CPU oracle, op by op.

Integer outputs (keys, permutation, grid ranges, CSR neighbor lists, sampled
indices) must be bit-exact; float outputs must satisfy
|x - y| <= 1e-4 * max(|y|, rms(y)).
"""
import numpy as np
import pytest
import torch

import oracle as orc
from oracle import pylib_ref as pr
from tensorflow_graphics_point_clouds_b200 import custom_ops as ops
from tensorflow_graphics_point_clouds_b200 import pc, synthetic
from tensorflow_graphics_point_clouds_b200._lib import TfgpcError

pytestmark = pytest.mark.gpu
F32 = np.float32
DEV = "cuda"


def t(a):
  return torch.as_tensor(np.ascontiguousarray(a)).to(DEV)


def close(x, y, rel=1e-4):
  x = np.asarray(x, np.float64); y = np.asarray(y, np.float64)
  if y.size == 0:
    assert x.size == 0
    return
  scale = np.maximum(np.abs(y), np.sqrt(np.mean(y * y)))
  bad = np.abs(x - y) > rel * scale + 1e-30
  assert not bad.any(), "max rel err %g at %d of %d" % (
      (np.abs(x - y) / np.maximum(scale, 1e-30)).max(), bad.sum(), y.size)


def random_cloud(rng, b, n, d):
  pts = rng.uniform(0, 1, (n, d)).astype(F32)
  bid = rng.integers(0, b, n).astype(np.int32)
  bid[:b] = np.arange(b)
  return pts, bid


def grid_pair(pts, bid, b, cell):
  """The oracle grid and the CUDA grid of the same cloud."""
  g_ref = pr.Grid(pts, bid, b, cell)
  g = pc.Grid(pc.PointCloud(t(pts), t(bid), b), cell)
  return g_ref, g


def assert_grid_equal(g_ref, g):
  assert np.array_equal(g._num_cells.cpu().numpy(), g_ref.num_cells)
  assert np.array_equal(g._scaled_aabb_min.cpu().numpy(), g_ref.scaled_aabb_min)
  assert np.array_equal(g._cur_keys.cpu().numpy(), g_ref.keys)
  assert np.array_equal(g._sorted_indices.cpu().numpy(), g_ref.sorted_indices)
  assert np.array_equal(g._sorted_keys.cpu().numpy(), g_ref.sorted_keys)
  assert np.array_equal(g._sorted_points.cpu().numpy(), g_ref.sorted_points)
  assert np.array_equal(g._sorted_batch_ids.cpu().numpy(), g_ref.sorted_batch_ids)
  assert np.array_equal(g.get_DS().cpu().numpy(), g_ref.get_ds())


@pytest.mark.parametrize("d", [2, 3, 4, 5, 6])
@pytest.mark.parametrize("cell", [0.05, 0.3])
def test_grid_build(d, cell):
  rng = np.random.default_rng(100 + d)
  b = 5
  pts, bid = random_cloud(rng, b, 3000, d)
  if d >= 5 and cell < 0.1:
    cell = 0.15
  g_ref, g = grid_pair(pts, bid, b, cell)
  assert_grid_equal(g_ref, g)


def test_grid_build_large_keys_and_ties():
  # many points per cell (ties in the sort) and a cloud with a single point
  rng = np.random.default_rng(7)
  pts = np.concatenate([rng.uniform(0, 1, (5000, 3)), [[0.5, 0.5, 0.5]]]).astype(F32)
  bid = np.concatenate([np.zeros(5000), [1]]).astype(np.int32)
  g_ref, g = grid_pair(pts, bid, 2, 0.5)
  assert_grid_equal(g_ref, g)


def neigh_pair(g_ref, g, radius, smp=None, sbid=None, max_neighbors=0):
  if smp is None:
    nb_ref = pr.Neighborhood(g_ref, radius, max_neighbors=max_neighbors)
    nb = pc.Neighborhood(g, radius, max_neighbors=max_neighbors)
  else:
    nb_ref = pr.Neighborhood(g_ref, radius, smp, sbid, max_neighbors)
    nb = pc.Neighborhood(g, radius, pc.PointCloud(t(smp), t(sbid), g_ref.batch_size),
                         max_neighbors)
  return nb_ref, nb


def assert_neigh_equal(nb_ref, nb):
  assert np.array_equal(nb._samples_neigh_ranges.cpu().numpy(), nb_ref.ranges)
  assert np.array_equal(nb._neighbors.cpu().numpy(), nb_ref.neighbors)
  assert np.array_equal(nb._original_neigh_ids.cpu().numpy(), nb_ref.original_neigh_ids)


@pytest.mark.parametrize("d", [2, 3, 4, 5, 6])
@pytest.mark.parametrize("radius", [0.08, 0.3, 0.9])
def test_find_neighbors_random(d, radius):
  rng = np.random.default_rng(200 + d)
  b = 4
  pts, bid = random_cloud(rng, b, 2500, d)
  smp, sbid = random_cloud(rng, b, 300, d)
  if d >= 5 and radius < 0.1:
    radius = 0.2
  g_ref, g = grid_pair(pts, bid, b, radius)
  nb_ref, nb = neigh_pair(g_ref, g, radius, smp, sbid)
  assert_neigh_equal(nb_ref, nb)
  # self neighborhood
  nb_ref, nb = neigh_pair(g_ref, g, radius)
  assert_neigh_equal(nb_ref, nb)


@pytest.mark.parametrize("radius,expected", [(0.05, 1), (0.11, 7), (0.142, 19), (0.174, 27)])
def test_find_neighbors_lattice_known_answers(radius, expected):
  """neighbors_test.py:113-146."""
  tk = np.linspace(0, 1, num=10, endpoint=False)
  pts = np.array(np.meshgrid(tk, tk, tk)).T.reshape(-1, 3).astype(F32)
  ts = np.linspace(1 / 5, 1, num=4, endpoint=False)
  smp = np.array(np.meshgrid(ts, ts, ts)).T.reshape(-1, 3).astype(F32)
  bid = np.zeros(len(pts), np.int32); sbid = np.zeros(len(smp), np.int32)
  g_ref, g = grid_pair(pts, bid, 1, radius)
  nb_ref, nb = neigh_pair(g_ref, g, radius, smp, sbid)
  assert_neigh_equal(nb_ref, nb)
  counts = np.diff(np.concatenate([[0], nb._samples_neigh_ranges.cpu().numpy()]))
  assert np.all(counts == expected)


def test_find_neighbors_edge_cases():
  rng = np.random.default_rng(3)
  pts, bid = random_cloud(rng, 3, 500, 3)
  g_ref, g = grid_pair(pts, bid, 3, 0.2)
  # samples outside the bounding box are clamped into border cells
  smp = np.array([[-0.5, 0.2, 0.2], [1.5, 1.5, 1.5], [0.5, 0.5, 0.5]], F32)
  sbid = np.array([0, 1, 2], np.int32)
  nb_ref, nb = neigh_pair(g_ref, g, 0.2, smp, sbid)
  assert_neigh_equal(nb_ref, nb)
  # no neighbors at all (M == 0)
  smp = np.array([[9.0, 9.0, 9.0]], F32); sbid = np.array([0], np.int32)
  nb_ref, nb = neigh_pair(g_ref, g, 0.2, smp, sbid)
  assert nb._neighbors.shape == (0, 2)
  assert_neigh_equal(nb_ref, nb)
  # max_neighbors keeps the first ones in canonical order
  nb_ref, nb = neigh_pair(g_ref, g, 0.2, max_neighbors=3)
  assert_neigh_equal(nb_ref, nb)
  # zero samples
  r, nbh = ops.find_neighbors(torch.zeros((0, 3), device=DEV), torch.zeros(0, dtype=torch.int32, device=DEV),
                              g._sorted_points, g._sorted_keys, g.get_DS(), g._num_cells,
                              g._scaled_aabb_min, g._inv_cell_sizes, torch.ones(3, device=DEV))
  assert r.shape[0] == 0 and nbh.shape == (0, 2)


def test_single_point_cloud():
  pts = np.array([[0.3, 0.4, 0.5]], F32); bid = np.zeros(1, np.int32)
  g_ref, g = grid_pair(pts, bid, 1, 0.1)
  assert_grid_equal(g_ref, g)
  nb_ref, nb = neigh_pair(g_ref, g, 0.1)
  assert_neigh_equal(nb_ref, nb)
  assert nb._neighbors.cpu().numpy().tolist() == [[0, 0]]


@pytest.mark.parametrize("d", [2, 3, 4])
@pytest.mark.parametrize("mode", [0, 1])
def test_compute_pdf_and_grads(d, mode):
  rng = np.random.default_rng(300 + d)
  b = 3
  pts, bid = random_cloud(rng, b, 1500, d)
  radius, bw = 0.25, 0.2
  g_ref, g = grid_pair(pts, bid, b, radius)
  nb_ref, nb = neigh_pair(g_ref, g, radius)
  assert_neigh_equal(nb_ref, nb)
  inv_bw = np.repeat(F32(1 / bw), d); inv_r = np.repeat(F32(1 / radius), d)
  ref = orc.compute_pdf(g_ref.sorted_points, nb_ref.neighbors, nb_ref.ranges, inv_bw, inv_r, mode)
  got = ops.compute_pdf_with_pt_grads(g._sorted_points, nb._neighbors, nb._samples_neigh_ranges,
                                      t(inv_bw), t(inv_r), mode)
  close(got.cpu().numpy(), ref)
  gvec = rng.normal(size=len(pts)).astype(F32)
  ref_g = orc.compute_pdf_pt_grads(g_ref.sorted_points, nb_ref.neighbors, nb_ref.ranges, inv_bw,
                                   inv_r, gvec, mode)
  got_g = ops.compute_pdf_pt_grads(g._sorted_points, nb._neighbors, nb._samples_neigh_ranges,
                                   t(inv_bw), t(inv_r), t(gvec), mode)
  close(got_g.cpu().numpy(), ref_g)      # measured: 1.2e-6


def test_pdf_matches_sklearn_kde():
  """compute_pdf_test.py:32-108 with a radius that covers the whole cloud."""
  from sklearn.neighbors import KernelDensity
  rng = np.random.default_rng(11)
  d, b, n_per, bw, cell = 3, 4, 100, 0.1, float(np.sqrt(3))
  pts = rng.uniform(0, 1, (b * n_per, d)).astype(F32)
  bid = np.repeat(np.arange(b), n_per).astype(np.int32)
  g = pc.Grid(pc.PointCloud(t(pts), t(bid), b), cell)
  nb = pc.Neighborhood(g, cell)
  nb.compute_pdf(bandwidth=bw, mode=0)
  pdf = nb._point_pdf.cpu().numpy() / n_per
  sp = g._sorted_points.cpu().numpy(); sb = g._sorted_batch_ids.cpu().numpy()
  ref = np.zeros(len(pts))
  for i in range(b):
    x = sp[sb == i].astype(np.float64) / cell
    ref[sb == i] = np.exp(KernelDensity(bandwidth=bw).fit(x).score_samples(x))
  np.testing.assert_allclose(pdf, ref, rtol=1e-4)


BP_CASES = [(1, 8, 2), (3, 16, 3), (7, 32, 3), (8, 64, 3), (16, 8, 4), (32, 16, 3),
            (64, 32, 3), (128, 16, 3), (136, 16, 3), (256, 16, 3), (64, 64, 3)]


@pytest.mark.parametrize("scratch", [True, False])
@pytest.mark.parametrize("c,k,d", BP_CASES)
def test_basis_proj_and_grads(c, k, d, scratch):
  """scratch=True: tensor-core kernels where the shape has them (K in 16/32/64,
  C % 16 == 0), fp32 kernels elsewhere; scratch=False: fp32 kernels only."""
  rng = np.random.default_rng(400 + c + k)
  b = 3
  pts, bid = random_cloud(rng, b, 1200, d)
  smp, sbid = random_cloud(rng, b, 150, d)
  radius = 0.3
  g_ref, g = grid_pair(pts, bid, b, radius)
  nb_ref, nb = neigh_pair(g_ref, g, radius, smp, sbid)
  m = len(nb_ref.neighbors)
  basis = rng.normal(size=(m, k)).astype(F32)
  feat = rng.normal(size=(len(pts), c)).astype(F32)
  ref = orc.basis_proj(basis, feat, nb_ref.original_neigh_ids, nb_ref.ranges)
  got = ops.basis_proj(t(basis), t(feat), nb._original_neigh_ids, nb._samples_neigh_ranges,
                       scratch=scratch)
  close(got.cpu().numpy(), ref)
  gin = rng.normal(size=ref.shape).astype(F32)
  ref_db, ref_df = orc.basis_proj_grads(basis, feat, nb_ref.original_neigh_ids, nb_ref.ranges, gin)
  got_db, got_df = ops.basis_proj_grads(t(basis), t(feat), nb._original_neigh_ids,
                                        nb._samples_neigh_ranges, t(gin), scratch=scratch)
  close(got_db.cpu().numpy(), ref_db)
  close(got_df.cpu().numpy(), ref_df)


def test_basis_proj_rejects_bad_shapes():
  z = torch.zeros
  with pytest.raises(TfgpcError, match="basis functions"):
    ops.basis_proj(z((4, 12), device=DEV), z((4, 8), device=DEV),
                   z((4, 2), dtype=torch.int32, device=DEV), z(2, dtype=torch.int32, device=DEV))
  with pytest.raises(TfgpcError, match="input features"):
    ops.basis_proj(z((4, 16), device=DEV), z((4, 9), device=DEV),
                   z((4, 2), dtype=torch.int32, device=DEV), z(2, dtype=torch.int32, device=DEV))
  with pytest.raises(TfgpcError, match="same number of basis"):
    ops.basis_proj(z((5, 16), device=DEV), z((4, 8), device=DEV),
                   z((4, 2), dtype=torch.int32, device=DEV), z(2, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("d,cell", [(2, 0.1), (3, 0.1), (3, 0.3), (4, 0.25)])
def test_sampling_poisson_and_average(d, cell):
  rng = np.random.default_rng(500 + d)
  b = 4
  pts, bid = random_cloud(rng, b, 4000, d)
  g_ref, g = grid_pair(pts, bid, b, cell)
  nb_ref, nb = neigh_pair(g_ref, g, cell)
  for mode, name in ((0, 'poisson'), (1, 'average')):
    rp, rb, ri = pr.sample(nb_ref, mode)
    cloud, idx = pc.sample(nb, name)
    assert np.array_equal(cloud._batch_ids.cpu().numpy(), rb)
    if mode == 0:
      assert np.array_equal(idx.cpu().numpy(), ri)
      assert np.array_equal(cloud._points.cpu().numpy(), rp)
    else:
      assert idx is None
      close(cloud._points.cpu().numpy(), rp)
  # pc.sample takes the symmetric-list entry for a self neighborhood; the entry
  # that assumes nothing about the lists must select the same points
  for symmetric in (False, True):
    p2, b2, i2 = ops.sampling(g._sorted_points, g._sorted_batch_ids, g._sorted_keys, g._num_cells,
                              nb._neighbors, nb._samples_neigh_ranges, 0, symmetric=symmetric)
    rp, rb, ri = pr.sample(nb_ref, 0)
    assert np.array_equal(g._sorted_indices[i2.long()].cpu().numpy(), ri)
    assert np.array_equal(p2.cpu().numpy(), rp)
    assert np.array_equal(b2.cpu().numpy(), rb)


def test_sampling_poisson_truncated_lists():
  """Lists cut by a neighbor limit are not symmetric: pc.sample must then select
  like the reference kernel, which looks only at a point's own list
  (count_sampling_pd_kernels.cu.cc:59-106)."""
  rng = np.random.default_rng(77)
  pts, bid = random_cloud(rng, 3, 5000, 3)
  g_ref, g = grid_pair(pts, bid, 3, 0.15)
  nb_ref, nb = neigh_pair(g_ref, g, 0.15, max_neighbors=6)
  rp, rb, ri = pr.sample(nb_ref, 0)
  cloud, idx = pc.sample(nb, 'poisson')
  assert np.array_equal(idx.cpu().numpy(), ri)
  assert np.array_equal(cloud._points.cpu().numpy(), rp)


def test_sampling_poisson_crowded_cells():
  """Cells holding thousands of points with thousands of neighbors each: the
  case where the symmetric-list passes and the general ones differ most in
  the work they do."""
  pts, bid = synthetic.gaussian_mixture_clouds(2, 12000, seed=11)
  g_ref, g = grid_pair(pts, bid, 2, 0.1)
  nb_ref, nb = neigh_pair(g_ref, g, 0.1)
  rp, rb, ri = pr.sample(nb_ref, 0)
  for symmetric in (False, True):
    p2, b2, i2 = ops.sampling(g._sorted_points, g._sorted_batch_ids, g._sorted_keys, g._num_cells,
                              nb._neighbors, nb._samples_neigh_ranges, 0, symmetric=symmetric)
    assert np.array_equal(g._sorted_indices[i2.long()].cpu().numpy(), ri)
    assert np.array_equal(b2.cpu().numpy(), rb)


@pytest.mark.parametrize("n,scale", [(6, 1), (100, 5)])
def test_poisson_lattice_known_answer(n, scale):
  """sample_test.py:61-78: n lines of n points, every second point survives."""
  tk = np.linspace(0, scale, num=n)
  pts = np.array(np.meshgrid(tk, tk)).T.reshape(-1, 2).astype(F32)
  bid = np.repeat(np.arange(n), n).astype(np.int32)
  cs = scale * np.array([2, 2], F32) / n
  g = pc.Grid(pc.PointCloud(t(pts), t(bid), n), cs)
  nb = pc.Neighborhood(g, cs)
  cloud, _ = pc.sample(nb, 'poisson')
  assert cloud._points.shape[0] == n * n // 2


def test_point_hierarchy_matches_oracle():
  pts, bid = synthetic.gaussian_mixture_clouds(3, 4000, seed=3)
  radii = [0.025, 0.05, 0.1, 0.2]
  ref = pr.point_hierarchy(pts, bid, 3, radii, mode=0)
  hier = pc.PointHierarchy(pc.PointCloud(t(pts), t(bid), 3), radii, 'poisson')
  for lvl in range(1, 5):
    assert np.array_equal(hier._point_clouds[lvl]._points.cpu().numpy(), ref[lvl][0])
    assert np.array_equal(hier._sample_indices[lvl - 1].cpu().numpy(), ref[lvl][2])
  ref = pr.point_hierarchy(pts, bid, 3, radii, mode=1)
  hier = pc.PointHierarchy(pc.PointCloud(t(pts), t(bid), 3), radii, 'average')
  for lvl in range(1, 5):
    close(hier._point_clouds[lvl]._points.cpu().numpy(), ref[lvl][0])
    assert np.array_equal(hier._point_clouds[lvl]._batch_ids.cpu().numpy(), ref[lvl][1])


def test_results_are_deterministic():
  pts, bid = synthetic.surface_clouds(2, seed=1, min_points=3000, max_points=5000)
  outs = []
  for _ in range(2):
    g = pc.Grid(pc.PointCloud(t(pts), t(bid), 2), 0.05)
    nb = pc.Neighborhood(g, 0.05)
    cloud, idx = pc.sample(nb, 'poisson')
    outs.append((g._sorted_indices.cpu().numpy().tobytes(), nb._neighbors.cpu().numpy().tobytes(),
                 idx.cpu().numpy().tobytes()))
  assert outs[0] == outs[1]


@pytest.mark.parametrize("d", [2, 3, 6])
def test_compute_aabb(d):
  rng = np.random.default_rng(600 + d)
  b = 7
  pts = (rng.normal(size=(5000, d)) * 3).astype(F32)      # negative and positive values
  bid = rng.integers(0, b - 1, 5000).astype(np.int32)     # cloud b-1 stays empty
  mn, mx = ops.compute_aabb(t(pts), t(bid), b)
  ref_mn = np.full((b, d), np.inf, F32); ref_mx = np.full((b, d), -np.inf, F32)
  np.minimum.at(ref_mn, bid, pts); np.maximum.at(ref_mx, bid, pts)
  assert np.array_equal(mn.cpu().numpy(), ref_mn)
  assert np.array_equal(mx.cpu().numpy(), ref_mx)
  # contiguous clouds (the common layout)
  bid2 = np.sort(bid)
  mn, mx = ops.compute_aabb(t(pts), t(bid2), b)
  ref_mn[:] = np.inf; ref_mx[:] = -np.inf
  np.minimum.at(ref_mn, bid2, pts); np.maximum.at(ref_mx, bid2, pts)
  assert np.array_equal(mn.cpu().numpy(), ref_mn) and np.array_equal(mx.cpu().numpy(), ref_mx)


def test_compute_aabb_negative_zero():
  """-0.0 has the bit pattern of the most negative int: it must neither replace
  a negative minimum nor be lost as the maximum of a cloud of negative values.
  Clouds: 0 all negative with -0.0 as its maximum, 1 mixed signs with -0.0 in
  between, 2 only zeros of both signs; points of a cloud are spread over many
  threads so that the atomics meet in every order."""
  rng = np.random.default_rng(8)
  n = 30000
  pts = np.empty((3 * n, 3), F32)
  pts[:n] = -rng.uniform(0.5, 5.0, (n, 3))
  pts[n:2 * n] = rng.uniform(-5.0, 5.0, (n, 3))
  pts[2 * n:] = 0.0
  zeros = rng.integers(0, 3 * n, 6000)
  pts[zeros] = -0.0
  pts[2 * n + rng.integers(0, n, 500)] = -0.0
  bid = np.repeat(np.arange(3), n).astype(np.int32)
  perm = rng.permutation(3 * n)
  for p, b in ((pts, bid), (pts[perm], bid[perm])):
    ref_mn, ref_mx = pr.aabb(p, b, 3)          # min - 1e-9, max + 1e-9 (PointCloud.py:38-43)
    cloud = pc.PointCloud(t(p), t(b), 3)
    mn, mx = cloud.get_AABB()
    assert np.array_equal(mn.cpu().numpy(), ref_mn) and np.array_equal(mx.cpu().numpy(), ref_mx)
    raw_mn, raw_mx = ops.compute_aabb(t(p), t(b), 3)
    exp_mn = np.full((3, 3), np.inf, F32); exp_mx = np.full((3, 3), -np.inf, F32)
    np.minimum.at(exp_mn, b, p); np.maximum.at(exp_mx, b, p)
    assert np.array_equal(raw_mn.cpu().numpy(), exp_mn)
    assert np.array_equal(raw_mx.cpu().numpy(), exp_mx)


def test_pdf_without_second_neighbor_search_matches_self_neighborhood():
  """A neighborhood whose samples are the grid's own cloud (unsorted) gets its
  densities from one search; pylib's route is the sorted self neighborhood."""
  rng = np.random.default_rng(42)
  b = 3
  pts, bid = random_cloud(rng, b, 3000, 3)
  g_ref = pr.Grid(pts, bid, b, 0.2)
  nb_ref = pr.Neighborhood(g_ref, 0.2, pts, bid)
  ref_pdf = nb_ref.get_pdf(bandwidth=0.2, mode=0)
  cloud = pc.PointCloud(t(pts), t(bid), b)
  nb = pc.Neighborhood(pc.Grid(cloud, 0.2), 0.2, cloud)
  assert nb._samples_are_grid_points() and not nb._equal_samples
  close(nb.get_pdf(bandwidth=0.2, mode=0).cpu().numpy(), ref_pdf)
  close(nb.point_pdf().cpu().numpy(), nb_ref.point_pdf)


@pytest.mark.parametrize("d", [2, 3, 4])
def test_find_neighbors_visiting_order_does_not_change_results(d):
  """The *_ordered entries work on the samples in a given sequence; ranges and
  lists must equal those of the plain entries bit for bit, for the key sort's
  permutation (what pc.Neighborhood passes for a cloud on its own grid) and
  for an arbitrary one."""
  rng = np.random.default_rng(40 + d)
  pts, bid = random_cloud(rng, 3, 6000, d)
  g_ref, g = grid_pair(pts, bid, 3, 0.2)
  cloud = g._point_cloud
  args = (cloud._points, cloud._batch_ids, g._sorted_points, g._sorted_keys, g.get_DS(),
          g._num_cells, g._scaled_aabb_min, g._inv_cell_sizes,
          torch.reciprocal(torch.full((d,), 0.2, device=DEV)))
  r0, n0 = ops.find_neighbors(*args, 0)
  for order in (g._sorted_indices, t(rng.permutation(len(pts)).astype(np.int32))):
    r1, n1 = ops.find_neighbors(*args, 0, sample_order=order)
    assert torch.equal(r0, r1) and torch.equal(n0, n1)
  r2, n2 = ops.find_neighbors(*args, 7, sample_order=g._sorted_indices)
  r3, n3 = ops.find_neighbors(*args, 7)
  assert torch.equal(r2, r3) and torch.equal(n2, n3)
  nb = pc.Neighborhood(g, 0.2, cloud)          # takes the ordered entries
  nb_ref = pr.Neighborhood(g_ref, 0.2, pts, bid)
  assert_neigh_equal(nb_ref, nb)


def test_neighborhood_transpose():
  """Neighborhood.py:318-329: the transposed neighborhood holds the same pairs
  with the roles exchanged; a self neighborhood is its own transpose."""
  rng = np.random.default_rng(9)
  b = 3
  pts, bid = random_cloud(rng, b, 2500, 3)
  smp, sbid = random_cloud(rng, b, 400, 3)
  g_ref, g = grid_pair(pts, bid, b, 0.2)
  nb_ref, nb = neigh_pair(g_ref, g, 0.2, smp, sbid)
  tr = nb.transpose()
  assert tr is nb.transpose()                     # built once
  assert tr._samples_neigh_ranges.shape[0] == len(pts)
  pairs = nb._original_neigh_ids.cpu().numpy()     # (point, sample)
  tpairs = tr._original_neigh_ids.cpu().numpy()    # (sample, point)
  assert len(pairs) == len(tpairs)
  key = lambda a, bb: np.sort(a.astype(np.int64) * 1_000_000 + bb)
  assert np.array_equal(key(pairs[:, 0], pairs[:, 1]), key(tpairs[:, 1], tpairs[:, 0]))
  # the oracle's search with the roles exchanged gives the same lists, bit for bit
  gt_ref = pr.Grid(smp, sbid, b, 0.2)
  nbt_ref = pr.Neighborhood(gt_ref, 0.2, pts, bid)
  assert_neigh_equal(nbt_ref, tr)
  own = pc.Neighborhood(g, 0.2)
  assert own.transpose() is own


@pytest.mark.parametrize("mode", [0, 1])
def test_fused_fill_matches_separate_passes(mode):
  """The fill pass that also writes original ids (and, on request, densities)
  must give what the separate passes give: lists and ids bit for bit, densities
  within 1e-4."""
  rng = np.random.default_rng(21)
  b = 4
  pts, bid = random_cloud(rng, b, 6000, 3)
  cloud = pc.PointCloud(t(pts), t(bid), b)
  g = pc.Grid(cloud, 0.15)
  nb = pc.Neighborhood(g, 0.15, cloud)            # ids come from the fused pass
  plain = ops.find_neighbors_fill(nb._count)
  ids, _ = ops.original_neighbor_ids(plain, g._sorted_indices)
  assert torch.equal(nb._neighbors, plain)
  assert torch.equal(nb._original_neigh_ids, ids)
  inv_bw = torch.full((3,), 1 / 0.2, device=DEV)
  n2, i2, pdf = ops.find_neighbors_fill(nb._count, g._sorted_indices, inv_bw, mode)
  assert torch.equal(n2, plain) and torch.equal(i2, ids)
  nb.compute_pdf(bandwidth=0.2, mode=mode)
  close(pdf.cpu().numpy(), nb.pdf_by_neighbor_id().cpu().numpy())
  g_ref = pr.Grid(pts, bid, b, 0.15)
  nb_ref = pr.Neighborhood(g_ref, 0.15, pts, bid)
  close(nb.get_pdf().cpu().numpy(), nb_ref.get_pdf(bandwidth=0.2, mode=mode))
  close(nb.point_pdf().cpu().numpy(), nb_ref.point_pdf)


@pytest.mark.parametrize("d,radius", [(2, 0.05), (3, 0.12), (4, 0.3)])
@pytest.mark.parametrize("samples", ["self", "points", "other"])
def test_grid_neighborhood_one_call(d, radius, samples):
  """Grid and Neighborhood from the single-call entry equal the oracle's (and so
  the separate constructors'), bit for bit, for the three kinds of samples."""
  rng = np.random.default_rng(31 + d)
  b = 3
  pts, bid = random_cloud(rng, b, 3000, d)
  g_ref = pr.Grid(pts, bid, b, radius)
  cloud = pc.PointCloud(t(pts), t(bid), b)
  if samples == "self":
    nb = pc.grid_neighborhood(cloud, radius)
    nb_ref = pr.Neighborhood(g_ref, radius)
  elif samples == "points":
    nb = pc.grid_neighborhood(cloud, radius, cloud, max_neighbors=7)
    nb_ref = pr.Neighborhood(g_ref, radius, pts, bid, 7)
  else:
    smp, sbid = random_cloud(rng, b, 500, d)
    nb = pc.grid_neighborhood(cloud, radius, pc.PointCloud(t(smp), t(sbid), b))
    nb_ref = pr.Neighborhood(g_ref, radius, smp, sbid)
  assert_grid_equal(g_ref, nb._grid)
  assert np.array_equal(nb._grid._num_cells_host.numpy(), g_ref.num_cells)
  assert_neigh_equal(nb_ref, nb)
  assert nb.num_pairs == len(nb_ref.neighbors)
  # what follows a neighborhood works on it as on one built by the constructors
  two = pc.Neighborhood(pc.Grid(cloud, radius), radius,
                        None if samples == "self" else nb._point_cloud_sampled,
                        7 if samples == "points" else 0)
  assert torch.equal(nb.get_pdf(), two.get_pdf())


def test_grid_neighborhood_repeats_with_larger_bound():
  """A grid with more cells per dimension than the call was sized for is reported
  (status 3 with the counts asked for) and the wrapper repeats the call."""
  rng = np.random.default_rng(5)
  pts, bid = random_cloud(rng, 2, 4000, 2)
  cloud = pc.PointCloud(t(pts), t(bid), 2)
  with pytest.raises(TfgpcError) as e:
    ops.grid_neighborhood_count(cloud._points, cloud._batch_ids, 2, [0.004, 0.004],
                                [0.004, 0.004], 64, samples_are_points=2)
  assert e.value.code == 3 and max(e.value.num_cells) > 64
  pc._MAX_CELLS.pop((2, 2), None)
  nb = pc.grid_neighborhood(cloud, 0.004)
  assert pc._MAX_CELLS[(2, 2)] >= max(e.value.num_cells)
  g_ref = pr.Grid(pts, bid, 2, 0.004)
  assert_grid_equal(g_ref, nb._grid)
  assert_neigh_equal(pr.Neighborhood(g_ref, 0.004), nb)
  pc._MAX_CELLS.pop((2, 2), None)
  # a grid finer than the one-call form sizes for: the separate constructors take over
  pts1, bid1 = random_cloud(rng, 1, 3000, 2)
  cloud1 = pc.PointCloud(t(pts1), t(bid1), 1)
  nb1 = pc.grid_neighborhood(cloud1, 0.0006, cloud1)
  g1_ref = pr.Grid(pts1, bid1, 1, 0.0006)
  assert max(g1_ref.num_cells) > pc._ONE_CALL_CELLS_LIMIT
  assert_grid_equal(g1_ref, nb1._grid)
  assert_neigh_equal(pr.Neighborhood(g1_ref, 0.0006, pts1, bid1), nb1)
  assert (2, 1) not in pc._MAX_CELLS or pc._MAX_CELLS[(2, 1)] <= pc._ONE_CALL_CELLS_LIMIT


def test_grid_neighborhood_one_call_with_reduced_cell_counts():
  """A shard of a distributed batch: the cell counts pass through the caller's
  reduction on the device (here a stand-in that raises them, as a larger cloud on
  another rank would) and the one-call form equals the separate constructors
  given the same reduction."""
  rng = np.random.default_rng(77)
  b = 3
  pts, bid = random_cloud(rng, b, 3000, 3)
  pts *= np.array([0.6, 1.0, 0.8], F32)
  other = torch.tensor([9, 7, 8], dtype=torch.int32, device=DEV)
  calls = []

  def reduce(counts):
    calls.append(1)
    return torch.maximum(counts, other)

  cloud = pc.PointCloud(t(pts), t(bid), b, num_cells_reduce=reduce)
  nb = pc.grid_neighborhood(cloud, 0.15, cloud)
  assert len(calls) == 1
  cloud2 = pc.PointCloud(t(pts), t(bid), b, num_cells_reduce=reduce)
  g2 = pc.Grid(cloud2, 0.15)
  nb2 = pc.Neighborhood(g2, 0.15, cloud2)
  assert nb._grid._num_cells.cpu().tolist() == [9, 7, 8]
  for name in ("_num_cells", "_scaled_aabb_min", "_cur_keys", "_sorted_indices", "_sorted_keys",
               "_sorted_points", "_sorted_batch_ids"):
    assert torch.equal(getattr(nb._grid, name), getattr(g2, name)), name
  assert torch.equal(nb._grid.get_DS(), g2.get_DS())
  assert torch.equal(nb._samples_neigh_ranges, nb2._samples_neigh_ranges)
  assert torch.equal(nb._neighbors, nb2._neighbors)
  assert torch.equal(nb._original_neigh_ids, nb2._original_neigh_ids)
