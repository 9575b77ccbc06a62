"""Pins the CPU oracle to the known answers held by the reference's own tests.

Each test restates one reference test with seeded inputs:
  keys        pylib/pc/tests/grid_test.py:29-71
  grid ds     pylib/pc/tests/grid_test.py:73-130
  neighbors   pylib/pc/tests/neighbors_test.py:30-76, 113-146
  pdf         pylib/pc/tests/compute_pdf_test.py:32-108
  basis proj  pylib/pc/layers/tests/basis_proj_test.py:30-111
  sampling    pylib/pc/tests/sample_test.py:31-125
"""
import numpy as np
import pytest

import oracle as orc
from oracle import pylib_ref as pr

F32 = np.float32


def random_cloud(rng, batch_size, n, d, equal=False):
  """pylib/pc/tests/utils.py:20-44, seeded."""
  pts = rng.uniform(0, 1, (n, d)).astype(F32)
  if equal:
    bid = np.repeat(np.arange(batch_size), n // batch_size)
  else:
    bid = rng.integers(0, batch_size, n)
    bid[:batch_size] = np.arange(batch_size)
  return pts, bid.astype(np.int32)


@pytest.mark.parametrize("d", [2, 3, 4])
def test_keys_match_numpy_formula(d):
  rng = np.random.default_rng(10 + d)
  b = 8
  pts, bid = random_cloud(rng, b, 4000, d)
  cell = F32(0.1)
  g = pr.Grid(pts, bid, b, [cell] * d)
  rel = (pts.astype(np.float64) - g.aabb_min[bid].astype(np.float64)) / float(cell)
  # points far enough from a cell border cannot be moved by float32 rounding
  safe = np.all(np.abs(rel - np.round(rel)) > 1e-4, axis=1)
  cells = np.clip(np.floor(rel).astype(np.int64), 0, g.num_cells - 1)
  mult = np.concatenate([np.cumprod(g.num_cells[::-1])[::-1], [1]]).astype(np.int64)
  keys = bid * mult[0] + (cells * mult[1:]).sum(axis=1)
  assert safe.mean() > 0.99
  assert np.array_equal(g.keys[safe], keys[safe])
  # sorted keys are the flipped ascending sort (grid_test.py:68-71)
  assert np.array_equal(g.sorted_keys, np.flip(np.sort(g.keys)))
  # ties keep the lower original index first (tf top_k contract)
  same = g.sorted_keys[1:] == g.sorted_keys[:-1]
  assert np.all(g.sorted_indices[1:][same] > g.sorted_indices[:-1][same])


@pytest.mark.parametrize("d", [2, 3, 4])
def test_grid_ds_matches_sequential_build(d):
  rng = np.random.default_rng(20 + d)
  b = 4
  pts, bid = random_cloud(rng, b, 2000, d)
  g = pr.Grid(pts, bid, b, [F32(0.2)] * d)
  ds = g.get_ds()
  nc = g.num_cells
  div = int(np.prod(nc[2:])) if d > 2 else 1
  ref = np.zeros((b * nc[0] * nc[1], 2), np.int32)
  idx = (g.sorted_keys // div).astype(np.int64)
  for i, k in enumerate(idx):          # grid_test.py:99-130
    if i == 0 or idx[i - 1] != k:
      ref[k, 0] = i
    ref[k, 1] = i + 1
  assert np.array_equal(ds.reshape(-1, 2), ref)


def lattice3d(n, bb_min=0.0):
  t = np.linspace(bb_min, 1, num=n, endpoint=False)
  return np.array(np.meshgrid(t, t, t)).T.reshape(-1, 3)


@pytest.mark.parametrize("radius,expected", [(0.05, 1), (0.11, 7), (0.142, 19),
                                             (0.174, 27)])
def test_neighbors_on_3d_lattice(radius, expected):
  pts = lattice3d(10)
  smp = lattice3d(4, bb_min=1 / 5)
  r = np.repeat(F32(radius), 3)
  g = pr.Grid(pts, np.zeros(len(pts), np.int32), 1, r)
  nb = pr.Neighborhood(g, r, smp, np.zeros(len(smp), np.int32))
  counts = np.diff(np.concatenate([[0], nb.ranges]))
  assert np.all(counts == expected)


@pytest.mark.parametrize("d", [2, 3, 4])
@pytest.mark.parametrize("radius", [0.05, 0.25, 0.7])
def test_neighbors_match_brute_force(d, radius):
  rng = np.random.default_rng(30 + d)
  b = 4
  pts, bid = random_cloud(rng, b, 600, d)
  smp, sbid = random_cloud(rng, b, 80, d)
  r = np.repeat(F32(radius), d)
  g = pr.Grid(pts, bid, b, r)
  nb = pr.Neighborhood(g, r, smp, sbid)
  bf = pr.brute_force_neighbors(smp, sbid, g.sorted_points, g.sorted_batch_ids, r)
  start = 0
  for s in range(len(smp)):
    got = nb.neighbors[start:nb.ranges[s]]
    start = nb.ranges[s]
    assert np.array_equal(got[:, 0], bf[s])      # canonical: ascending index
    assert np.all(got[:, 1] == s)
  # neighbors_test.py:78-111: neighbor and sample share the batch id
  assert np.array_equal(g.sorted_batch_ids[nb.neighbors[:, 0]],
                        sbid[nb.neighbors[:, 1]])


@pytest.mark.parametrize("d,cell", [(2, 0.2), (2, 0.7), (3, 0.2), (3, 0.7),
                                    (3, np.sqrt(3)), (4, 0.2), (4, 2.0)])
def test_pdf_matches_sklearn_kde(d, cell):
  from sklearn.neighbors import KernelDensity
  rng = np.random.default_rng(40 + d)
  b, n_per, bw = 4, 100, 0.1
  pts, bid = random_cloud(rng, b, b * n_per, d, equal=True)
  r = np.repeat(F32(cell), d)
  g = pr.Grid(pts, bid, b, r)
  nb = pr.Neighborhood(g, r)
  pdf = orc.compute_pdf(g.sorted_points, nb.neighbors, nb.ranges,
                        np.repeat(F32(1 / bw), d), (F32(1) / r), 0)
  ref = np.zeros(len(pts))
  for i in range(b):
    sel = g.sorted_batch_ids == i
    x = g.sorted_points[sel].astype(np.float64) / cell
    kde = KernelDensity(bandwidth=bw).fit(x)
    ref[sel] = np.exp(kde.score_samples(x))
  if cell >= np.sqrt(d):   # the neighborhood then holds the whole cloud
    np.testing.assert_allclose(pdf / n_per, ref, rtol=1e-4)
  else:                    # truncated kernel: contributions beyond the radius
    assert np.all(pdf / n_per <= ref * (1 + 1e-4))   # are missing, never extra
    if cell / bw >= 5 * 0.2 / 0.1 * 0.5:
      np.testing.assert_allclose(pdf / n_per, ref, rtol=5e-2)


@pytest.mark.parametrize("c,k,d", [(1, 8, 2), (3, 16, 3), (8, 32, 3), (16, 8, 4)])
def test_basis_proj_matches_numpy_csr_sum(c, k, d):
  rng = np.random.default_rng(50 + c)
  b = 4
  pts, bid = random_cloud(rng, b, 800, d)
  smp, sbid = random_cloud(rng, b, 100, d)
  r = np.repeat(F32(0.3), d)
  g = pr.Grid(pts, bid, b, r)
  nb = pr.Neighborhood(g, r, smp, sbid)
  m = len(nb.neighbors)
  basis = rng.normal(size=(m, k)).astype(F32)
  feat = rng.normal(size=(len(pts), c)).astype(F32)
  out = orc.basis_proj(basis, feat, nb.original_neigh_ids, nb.ranges)
  ref = np.zeros((len(smp), c, k))
  np.add.at(ref, nb.original_neigh_ids[:, 1],
            feat[nb.original_neigh_ids[:, 0]][:, :, None].astype(np.float64)
            * basis[:, None, :])
  np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-4)
  # gradients against the transposed linear map
  g_in = rng.normal(size=out.shape).astype(F32)
  dbasis, dfeat = orc.basis_proj_grads(basis, feat, nb.original_neigh_ids,
                                       nb.ranges, g_in)
  ids = nb.original_neigh_ids
  ref_db = np.einsum('mck,mc->mk', g_in[ids[:, 1]].astype(np.float64),
                     feat[ids[:, 0]])
  ref_df = np.zeros(feat.shape)
  np.add.at(ref_df, ids[:, 0],
            np.einsum('mck,mk->mc', g_in[ids[:, 1]].astype(np.float64), basis))
  np.testing.assert_allclose(dbasis, ref_db, rtol=1e-4, atol=1e-4)
  np.testing.assert_allclose(dfeat, ref_df, rtol=1e-4, atol=1e-4)


def test_pdf_point_gradient_matches_finite_differences():
  rng = np.random.default_rng(60)
  d, b = 3, 2
  pts, bid = random_cloud(rng, b, 60, d, equal=True)
  r = np.repeat(F32(0.5), d)
  g = pr.Grid(pts, bid, b, r)
  nb = pr.Neighborhood(g, r)
  ib, ir = np.repeat(F32(1 / 0.5), d), F32(1) / r
  gvec = rng.normal(size=len(pts)).astype(F32)
  grad = orc.compute_pdf_pt_grads(g.sorted_points, nb.neighbors, nb.ranges, ib,
                                  ir, gvec, 0)

  def f(p):   # float64 KDE over the fixed neighbor lists
    x = p * ib * ir
    dif = x[nb.neighbors[:, 0]] - x[nb.neighbors[:, 1]]
    val = np.prod(ib * np.exp(-0.5 * dif * dif) * 0.39894228, axis=1)
    pdf = np.zeros(len(p))
    np.add.at(pdf, nb.neighbors[:, 1], val)
    return float((pdf * gvec).sum())

  p0 = g.sorted_points.astype(np.float64)
  num = np.zeros_like(p0)
  eps = 1e-5
  for i in range(p0.shape[0]):
    for j in range(d):
      pp, pm = p0.copy(), p0.copy()
      pp[i, j] += eps; pm[i, j] -= eps
      num[i, j] = (f(pp) - f(pm)) / (2 * eps)
  np.testing.assert_allclose(grad, num, rtol=2e-3, atol=2e-3 * np.abs(num).max())


@pytest.mark.parametrize("n,scale", [(6, 1), (100, 5)])
def test_poisson_on_lattice_lines(n, scale):
  """sample_test.py:61-78: the [n,n,2] lattice is a padded batch of n clouds,
  each one a line of n points; every second point survives."""
  t = np.linspace(0, scale, num=n)
  pts = np.array(np.meshgrid(t, t)).T.reshape(-1, 2)
  bid = np.repeat(np.arange(n), n).astype(np.int32)
  cs = scale * np.array([2, 2], F32) / n
  g = pr.Grid(pts, bid, n, cs)
  nb = pr.Neighborhood(g, cs)
  p, _, _ = pr.sample(nb, 0)
  assert len(p) == n * n // 2


@pytest.mark.parametrize("d,b", [(3, 8), (4, 16)])
def test_poisson_min_distance(d, b):
  rng = np.random.default_rng(70 + d)
  cell = 0.1
  pts, bid = random_cloud(rng, b, 100 * b, d, equal=True)
  cs = np.repeat(F32(cell), d)
  g = pr.Grid(pts, bid, b, cs)
  nb = pr.Neighborhood(g, cs)
  p, pb, idx = pr.sample(nb, 0)
  assert np.array_equal(pts[idx], p)
  for i in range(b):
    q = p[pb == i].astype(np.float64)
    dist = np.linalg.norm(q[:, None] - q[None], axis=2)
    dist[np.diag_indices(len(q))] = np.inf
    assert dist.min() >= cell * (1 - 1e-6)     # no two samples within the radius
  # maximality: every rejected point has a taken neighbor
  taken = np.zeros(len(pts), bool)
  inv = np.empty(len(pts), np.int64); inv[g.sorted_indices] = np.arange(len(pts))
  taken[inv[idx]] = True
  start = 0
  for s in range(len(pts)):
    lst = nb.neighbors[start:nb.ranges[s], 0]; start = nb.ranges[s]
    assert taken[s] or taken[lst].any()


@pytest.mark.parametrize("cell,b", [(0.1, 2), (0.7, 8), (np.sqrt(3), 2)])
def test_cell_average_matches_running_mean(cell, b):
  rng = np.random.default_rng(80 + b)
  d = 3
  pts, bid = random_cloud(rng, b, 100 * b, d, equal=True)
  cs = np.repeat(F32(cell), d)
  g = pr.Grid(pts, bid, b, cs)
  nb = pr.Neighborhood(g, cs)
  p, pb, _ = pr.sample(nb, 1)
  ref, refb = [], []
  cur, cnt, key = np.zeros(d), 0, None
  for i, k in enumerate(g.sorted_keys):      # sample_test.py:97-113
    if k != key and key is not None:
      ref.append(cur / cnt); refb.append(g.sorted_batch_ids[i - 1])
      cur, cnt = np.zeros(d), 0
    key = k
    cur = cur + g.sorted_points[i]; cnt += 1
  ref.append(cur / cnt); refb.append(g.sorted_batch_ids[-1])
  np.testing.assert_allclose(p, np.array(ref), atol=1e-4)
  assert np.array_equal(pb, np.array(refb))


def _layer_case(rng, d, n_pts, n_smp, b, radius):
  pts, bid = random_cloud(rng, b, n_pts, d)
  smp, sbid = random_cloud(rng, b, n_smp, d)
  r = np.repeat(F32(radius), d)
  g = pr.Grid(pts, bid, b, r)
  nb = pr.Neighborhood(g, r, smp, sbid)
  return pts, smp, nb


def _sum_per_sample(per_pair, ranges):
  """The reference tests' integration loop: rows of a sample are contiguous."""
  ends = np.concatenate(([0], ranges))
  return np.stack([per_pair[ends[i]:ends[i + 1]].sum(axis=0) for i in range(len(ranges))])


@pytest.mark.parametrize("n_pts,n_smp,feats,b,radius,num_kp,interp",
                         [(200, 20, (1, 3), 16, 0.7, 5, 'linear'),
                          (400, 40, (3, 3), 8, 0.7, 5, 'linear'),
                          (400, 10, (3, 1), 1, np.sqrt(3), 5, 'linear'),
                          (400, 40, (8, 4), 4, 0.7, 15, 'gaussian')])
def test_kpconv_matches_numpy_layer(n_pts, n_smp, feats, b, radius, num_kp, interp):
  """kernel_point_conv_test.py:53-99 (sizes from its parameter list): distances
  to the kernel points, linear weights, per-sample sums, product with the
  weights, all in float64."""
  rng = np.random.default_rng(n_pts + num_kp)
  pts, smp, nb = _layer_case(rng, 3, n_pts, n_smp, b, radius)
  feat = rng.uniform(size=(n_pts, feats[0])).astype(F32)
  kp = (rng.normal(size=(num_kp, 3)) * 0.4).astype(F32)
  w = rng.normal(size=(num_kp * feats[0], feats[1])).astype(F32)
  out = pr.kpconv_forward(feat, pts, smp, nb, kp, w, radius, 1.0, interp)
  ids = nb.original_neigh_ids
  diff = (pts[ids[:, 0]].astype(np.float64) - smp[ids[:, 1]]) / radius
  dist = np.linalg.norm(diff[:, None, :] - kp[None].astype(np.float64), axis=2)
  kw = np.maximum(1 - dist, 0) if interp == 'linear' else np.exp(-(dist / (1 / 3)) ** 2)
  per_pair = feat[ids[:, 0]][:, :, None].astype(np.float64) * kw[:, None, :]
  x = _sum_per_sample(per_pair, nb.ranges)
  ref = x.reshape(n_smp, -1) @ w.astype(np.float64)
  np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("n_pts,n_smp,feats,b,radius,hidden,d",
                         [(2000, 200, (3, 3), 16, 0.7, 8, 2), (2000, 200, (1, 3), 16, 0.7, 8, 3),
                          (4000, 100, (3, 1), 1, np.sqrt(3), 16, 3),
                          (2000, 200, (3, 3), 16, 0.7, 8, 4)])
def test_pointconv_matches_numpy_layer(n_pts, n_smp, feats, b, radius, hidden, d):
  """point_conv_test.py:38-113 (sizes from its parameter list)."""
  rng = np.random.default_rng(n_pts + hidden + d)
  pts, smp, nb = _layer_case(rng, d, n_pts, n_smp, b, radius)
  feat = rng.uniform(size=(n_pts, feats[0])).astype(F32)
  pdf = nb.get_pdf()
  hw = rng.normal(size=(d, hidden)).astype(F32)
  hb = (rng.normal(size=(1, hidden)) * 0.1).astype(F32)
  w = rng.normal(size=(hidden * feats[0], feats[1])).astype(F32)
  pw = [rng.normal(size=(1, 16)).astype(F32), np.abs(rng.normal(size=(16, 1))).astype(F32)]
  pb = [np.abs(rng.normal(size=(1, 16))).astype(F32), np.ones((1, 1), F32)]
  out, _ = pr.pointconv_forward(feat, pts, smp, nb, pdf, hw, hb, w, pw, pb, 'relu')
  ids = nb.original_neigh_ids
  mx = np.array([pdf[ids[:, 1] == s].max() if (ids[:, 1] == s).any() else 1.0
                 for s in range(n_smp)])
  cur = (pdf.astype(np.float64) / mx[ids[:, 1]]).reshape(-1, 1)
  cur = np.maximum(cur @ pw[0] + pb[0], 0) @ pw[1] + pb[1]
  latent = np.maximum((pts[ids[:, 0]].astype(np.float64) - smp[ids[:, 1]]) @ hw + hb, 0) / cur
  per_pair = feat[ids[:, 0]][:, :, None].astype(np.float64) * latent[:, None, :]
  x = _sum_per_sample(per_pair, nb.ranges)
  ref = x.reshape(n_smp, -1) @ w.astype(np.float64)
  np.testing.assert_allclose(out, ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("mode", ['max', 'avg'])
def test_pooling_matches_per_segment_loops(mode):
  """pooling_layers_test.py: the pooled value of a segment is numpy's max / mean
  over the rows that belong to it."""
  rng = np.random.default_rng(9)
  pts, smp, nb = _layer_case(rng, 3, 1500, 120, 4, 0.3)
  feat = rng.normal(size=(1500, 6)).astype(F32)
  out = pr.neighborhood_pool(feat, nb, mode)
  ids = nb.original_neigh_ids
  for s in range(120):
    rows = feat[ids[ids[:, 1] == s, 0]]
    if len(rows) == 0:
      assert np.all(out[s] == (pr.LOWEST if mode == 'max' else 0))
    else:
      ref = rows.max(axis=0) if mode == 'max' else rows.astype(np.float64).mean(axis=0)
      np.testing.assert_allclose(out[s], ref, rtol=1e-5, atol=1e-6)
  bid = rng.integers(0, 5, 1500).astype(np.int32)
  g = pr.global_pool(feat, bid, 6, mode)     # segment 5 stays empty
  for b in range(5):
    ref = feat[bid == b].max(axis=0) if mode == 'max' else feat[bid == b].mean(axis=0)
    np.testing.assert_allclose(g[b], ref, rtol=1e-5, atol=1e-6)
  assert np.all(g[5] == (pr.LOWEST if mode == 'max' else 0))


@pytest.mark.parametrize("hidden,act", [([8], 'elu'), ([8], 'leaky_relu'), ([6, 8], 'elu')])
def test_mcconv_layer_gradients_match_finite_differences(hidden, act):
  """monte_carlo_conv_test.py:110-219 (jacobians with respect to features, weights
  and points; atol 1e-4, delta 1e-3) restated on the float64 layer of the oracle:
  8 points, 4 samples, 2 clouds, radius sqrt(3) * 1.25, neighborhood and densities
  held fixed while the points move, as in the reference's test."""
  rng = np.random.default_rng(31)
  n, ns, b, d, cin, cout = 8, 4, 2, 3, 8, 8
  radius = float(np.sqrt(3) * 1.25)
  pts = rng.uniform(0, 1, (n, d)).astype(F32); bid = np.repeat(np.arange(b), n // b).astype(np.int32)
  smp = rng.uniform(0, 1, (ns, d)).astype(F32); sbid = np.repeat(np.arange(b), ns // b).astype(np.int32)
  feat = rng.uniform(0, 1, (n, cin)).astype(F32)
  grid = pr.Grid(pts, bid, b, radius)
  neigh = pr.Neighborhood(grid, radius, smp, sbid)
  pdf = neigh.get_pdf(bandwidth=0.2, mode=0)
  sizes = [d] + hidden
  ws = [rng.normal(size=(1, sizes[i], sizes[i + 1])) for i in range(len(hidden))]
  bs = [rng.normal(size=(1, 1, sizes[i + 1])) * 0.1 for i in range(len(hidden))]
  wf = rng.normal(size=(1, cin * hidden[-1], cout)) * 0.3
  d_out = rng.normal(size=(ns, cout))

  def loss(p=pts, s=smp, f=feat, w=ws, bb=bs, final=wf, dens=pdf):
    return float((pr.mcconv_layer(p, s, f, neigh, dens, w, bb, final, radius, act) * d_out).sum())

  g = pr.mcconv_layer_grads(pts, smp, feat, neigh, pdf, ws, bs, wf, radius, d_out, act)
  delta = 1e-3

  def fd(make):
    """Central difference of the loss along every entry of an array."""
    base, shape = make(None)
    out = np.zeros(shape)
    for idx in np.ndindex(*shape):
      hi = loss(**make((idx, +delta))[0]); lo = loss(**make((idx, -delta))[0])
      out[idx] = (hi - lo) / (2 * delta)
    return out

  def vary(name, arr):
    def make(step):
      if step is None:
        return None, arr.shape
      a = arr.astype(np.float64).copy()
      a[step[0]] += step[1]
      return {name: a}, arr.shape
    return make

  np.testing.assert_allclose(g["d_points_in"], fd(vary("p", pts)), atol=1e-4)
  np.testing.assert_allclose(g["d_points_out"], fd(vary("s", smp)), atol=1e-4)
  np.testing.assert_allclose(g["d_features"], fd(vary("f", feat)), atol=1e-4)
  np.testing.assert_allclose(g["d_wf"], fd(vary("final", wf)), atol=1e-4)
  np.testing.assert_allclose(g["d_pdf"], fd(vary("dens", pdf)), atol=2e-3, rtol=1e-3)
  for layer in range(len(hidden)):
    def make_w(step, layer=layer):
      if step is None:
        return None, ws[layer].shape
      w2 = [w.copy() for w in ws]; w2[layer][step[0]] += step[1]
      return {"w": w2}, ws[layer].shape
    def make_b(step, layer=layer):
      if step is None:
        return None, bs[layer].shape
      b2 = [x.copy() for x in bs]; b2[layer][step[0]] += step[1]
      return {"bb": b2}, bs[layer].shape
    np.testing.assert_allclose(g["d_weights"][layer], fd(make_w), atol=1e-4)
    np.testing.assert_allclose(g["d_biases"][layer], fd(make_b), atol=1e-4)
