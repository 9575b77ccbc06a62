"""NumPy restatement of the pylib glue around the custom ops (TEST
INFRASTRUCTURE ONLY; see ``oracle/__init__.py``).

Follows the reference's Python callers so that the oracle can be driven exactly
the way pylib drives the ops:
  AABB        pylib/pc/PointCloud.py:38-43
  Grid        pylib/pc/Grid.py:32-83
  Neighborhood pylib/pc/Neighborhood.py:218-311
  sample / PointHierarchy  pylib/pc/sampling.py:123-150, PointHierarchy.py:40-98
  MCConv      pylib/pc/layers/MCConv.py:137-278
All arithmetic that feeds the ops is done in float32 like the TF code.
"""
import numpy as np

import oracle as orc

F32 = np.float32


def aabb(points, batch_ids, batch_size):
  """PointCloud.py:38-43: unsorted_segment_min/max -+ 1e-9 (float32)."""
  points = np.asarray(points, F32)
  d = points.shape[1]
  mn = np.full((batch_size, d), np.inf, F32)
  mx = np.full((batch_size, d), -np.inf, F32)
  np.minimum.at(mn, batch_ids, points)
  np.maximum.at(mx, batch_ids, points)
  return (mn - F32(1e-9)).astype(F32), (mx + F32(1e-9)).astype(F32)


class Grid:
  """Grid.py:32-83."""

  def __init__(self, points, batch_ids, batch_size, cell_sizes, fused=True):
    points = np.ascontiguousarray(points, F32)
    batch_ids = np.ascontiguousarray(batch_ids, np.int32)
    d = points.shape[1]
    cell_sizes = np.asarray(cell_sizes, F32).reshape(-1)
    if cell_sizes.shape[0] == 1:
      cell_sizes = np.repeat(cell_sizes, d)
    self.points, self.batch_ids, self.batch_size = points, batch_ids, batch_size
    self.cell_sizes = cell_sizes
    self.aabb_min, self.aabb_max = aabb(points, batch_ids, batch_size)
    sizes = (self.aabb_max - self.aabb_min).astype(F32)
    bnc = np.ceil((sizes / cell_sizes).astype(F32)).astype(np.int32)
    self.num_cells = np.maximum(bnc.max(axis=0), 1).astype(np.int32)
    # custom_ops_wrapper.py:37-43
    self.scaled_aabb_min = (self.aabb_min / cell_sizes).astype(F32)
    self.inv_cell_sizes = (F32(1.0) / cell_sizes).astype(F32)
    self.keys = orc.compute_keys(points, batch_ids, self.scaled_aabb_min,
                                 self.num_cells, self.inv_cell_sizes, fused)
    self.sorted_indices, self.sorted_keys = orc.sort_keys_desc(self.keys)
    self.sorted_points = points[self.sorted_indices]
    self.sorted_batch_ids = batch_ids[self.sorted_indices]
    self.fused = fused
    self._ds = None

  def get_ds(self):
    if self._ds is None:
      self._ds = orc.build_grid_ds(self.sorted_keys, self.num_cells,
                                   self.batch_size)
    return self._ds


class Neighborhood:
  """Neighborhood.py:218-311."""

  def __init__(self, grid, radii, samples=None, samples_batch_ids=None,
               max_neighbors=0):
    d = grid.points.shape[1]
    radii = np.asarray(radii, F32).reshape(-1)
    if radii.shape[0] == 1:
      radii = np.repeat(radii, d)
    self.grid, self.radii = grid, radii
    self.equal_samples = samples is None
    if samples is None:
      samples, samples_batch_ids = grid.sorted_points, grid.sorted_batch_ids
    self.samples = np.ascontiguousarray(samples, F32)
    self.samples_batch_ids = np.ascontiguousarray(samples_batch_ids, np.int32)
    self.ranges, self.neighbors = orc.find_neighbors(
        self.samples, self.samples_batch_ids, grid.sorted_points,
        grid.sorted_keys, grid.num_cells, grid.scaled_aabb_min,
        grid.inv_cell_sizes, (F32(1.0) / radii).astype(F32), max_neighbors,
        grid.fused)
    self.original_neigh_ids = np.stack(
        [grid.sorted_indices[self.neighbors[:, 0]], self.neighbors[:, 1]],
        axis=1).astype(np.int32)
    self._pdf = None

  def get_pdf(self, bandwidth=0.2, mode=0):
    """Neighborhood.py:257-311 (KDEMode.constant = 0, num_points = 1)."""
    if self._pdf is None:
      d = self.samples.shape[1]
      bw = np.asarray(bandwidth, F32).reshape(-1)
      if bw.shape[0] == 1:
        bw = np.repeat(bw, d)
      nb = self if self.equal_samples else Neighborhood(self.grid, self.radii)
      self.point_pdf = orc.compute_pdf(
          self.grid.sorted_points, nb.neighbors, nb.ranges,
          (F32(1.0) / bw).astype(F32), (F32(1.0) / self.radii).astype(F32), mode)
      self._pdf = self.point_pdf[self.neighbors[:, 0]]
    return self._pdf


def sample(neigh, mode):
  """sampling.py:123-150; mode 0 = Poisson disk, 1 = cell average.  Returns
  (points, batch_ids, original indices or None)."""
  g = neigh.grid
  pts, bids, idx = orc.sampling(g.sorted_points, g.sorted_batch_ids,
                                g.sorted_keys, g.num_cells, neigh.neighbors,
                                neigh.ranges, mode)
  if mode == 0:
    return pts, bids, g.sorted_indices[idx]
  return pts, bids, None


def point_hierarchy(points, batch_ids, batch_size, cell_sizes, mode=0):
  """PointHierarchy.py:40-98: per level Grid -> self Neighborhood -> sample."""
  levels = [(np.asarray(points, F32), np.asarray(batch_ids, np.int32), None)]
  cur_p, cur_b = levels[0][0], levels[0][1]
  for cs in cell_sizes:
    g = Grid(cur_p, cur_b, batch_size, cs)
    nb = Neighborhood(g, cs)
    cur_p, cur_b, idx = sample(nb, mode)
    levels.append((cur_p, cur_b, idx))
  return levels


def brute_force_neighbors(samples, samples_batch_ids, points, batch_ids, radii):
  """custom_ops_tf.py:216-258 (find_neighbors_no_grid) with the strict `<` of
  the CUDA kernel; float32 arithmetic in the kernel's order.  Returns a list of
  sorted index arrays, one per sample (indices into `points`)."""
  samples = np.asarray(samples, F32); points = np.asarray(points, F32)
  inv_r = (F32(1.0) / np.asarray(radii, F32)).astype(F32)
  out = []
  for s in range(samples.shape[0]):
    t = ((samples[s][None, :] - points).astype(F32) * inv_r).astype(F32)
    d2 = (t[:, 0] * t[:, 0]).astype(F32)
    for d in range(1, points.shape[1]):
      # fma(t,t,d2): exact product in float64, one rounding
      d2 = (t[:, d].astype(np.float64) * t[:, d].astype(np.float64)
            + d2.astype(np.float64)).astype(F32)
    ok = (np.sqrt(d2).astype(F32) < F32(1.0)) & (batch_ids == samples_batch_ids[s])
    out.append(np.nonzero(ok)[0])
  return out


def leaky_relu(x, alpha=0.2):
  """tf.nn.leaky_relu default alpha (MCConv.py:27-31)."""
  return np.where(x > 0, x, x * F32(alpha)).astype(F32)


def mcconv_basis(points_in, points_out, neigh, pdf, w1, b1, radius):
  """MCConv.py:264-269 and :163-171 for a one-hidden-layer kernel MLP.
  w1 [num_mlps, D, H], b1 [num_mlps, 1, H] -> basis [M, num_mlps*H]."""
  ids = neigh.original_neigh_ids
  diff = ((points_in[ids[:, 0]] - points_out[ids[:, 1]]) / F32(radius)).astype(F32)
  hid = np.einsum('md,gdh->gmh', diff, w1).astype(F32) + b1
  hid = leaky_relu(hid)
  hid = np.transpose(hid, (1, 0, 2)).reshape(diff.shape[0], -1)
  return (hid / pdf.reshape(-1, 1)).astype(F32), diff, hid


def _act(x, name):
  """Activations of MCConv.py:27-31 and their derivatives (float64)."""
  name = name.lower()
  if name == 'elu':
    return np.where(x > 0, x, np.expm1(x)), np.where(x > 0, 1.0, np.exp(x))
  alpha = 0.0 if name == 'relu' else 0.2
  return np.where(x > 0, x, alpha * x), np.where(x > 0, 1.0, alpha)


def kernel_mlp_forward(diff, weights, biases, non_linearity='leaky_relu'):
  """The kernel MLP of MCConv.py:163-171 with any number of hidden layers:
  weights[l] [num_mlps, H_{l-1}, H_l], biases[l] [num_mlps, 1, H_l], every layer
  followed by the activation.  diff [M, D] -> (hidden [M, num_mlps * H_last]
  float64, the per-layer pre-activations)."""
  g = weights[0].shape[0]
  cur = np.tile(diff.astype(np.float64)[None], (g, 1, 1))
  pres = []
  for w, b in zip(weights, biases):
    pre = np.matmul(cur, w.astype(np.float64)) + b.astype(np.float64)
    pres.append((cur, pre))
    cur = _act(pre, non_linearity)[0]
  hid = np.transpose(cur, (1, 0, 2)).reshape(diff.shape[0], -1)
  return hid, pres


def kernel_mlp_backward(d_hid, pres, weights, non_linearity='leaky_relu'):
  """Gradients of kernel_mlp_forward: d_hid [M, num_mlps * H_last] ->
  (d_diff [M, D], [d_weights], [d_biases]) in float64."""
  g = weights[0].shape[0]
  m = d_hid.shape[0]
  cur = np.transpose(d_hid.reshape(m, g, -1), (1, 0, 2))
  d_w, d_b = [], []
  for (inp, pre), w in zip(reversed(pres), reversed(weights)):
    dpre = cur * _act(pre, non_linearity)[1]
    d_w.insert(0, np.matmul(np.transpose(inp, (0, 2, 1)), dpre))
    d_b.insert(0, dpre.sum(axis=1, keepdims=True))
    cur = np.matmul(dpre, np.transpose(w.astype(np.float64), (0, 2, 1)))
  return cur.sum(axis=0), d_w, d_b


def mcconv_layer(points_in, points_out, features, neigh, pdf, weights, biases, wf, radius,
                 non_linearity='leaky_relu'):
  """The whole layer of MCConv.py:196-278 for a given neighborhood and given
  per-pair densities, in float64 (multi-layer kernel MLP): [Ns, Cout]."""
  ids = neigh.original_neigh_ids
  diff = (points_in[ids[:, 0]].astype(np.float64) - points_out[ids[:, 1]]) / radius
  hid, _ = kernel_mlp_forward(diff, weights, biases, non_linearity)
  basis = hid / pdf.astype(np.float64).reshape(-1, 1)
  ns, cin, g = len(neigh.ranges), features.shape[1], wf.shape[0]
  k = basis.shape[1]
  x = np.zeros((ns, cin, k))
  np.add.at(x, ids[:, 1], features[ids[:, 0]].astype(np.float64)[:, :, None] * basis[:, None, :])
  xg = np.transpose(x.reshape(ns, cin, g, k // g), (2, 0, 1, 3)).reshape(g, ns, -1)
  out = np.matmul(xg, wf.astype(np.float64))
  return np.transpose(out, (1, 0, 2)).reshape(ns, -1)


def mcconv_layer_grads(points_in, points_out, features, neigh, pdf, weights, biases, wf, radius,
                       d_out, non_linearity='leaky_relu'):
  """Analytic gradients of mcconv_layer in float64: a dict with d_features,
  d_wf, d_weights, d_biases, d_points_in, d_points_out and d_pdf (per pair: the
  density enters as basis = hidden / pdf)."""
  ids = neigh.original_neigh_ids
  p_in, p_out = points_in.astype(np.float64), points_out.astype(np.float64)
  diff = (p_in[ids[:, 0]] - p_out[ids[:, 1]]) / radius
  hid, pres = kernel_mlp_forward(diff, weights, biases, non_linearity)
  pdf64 = pdf.astype(np.float64).reshape(-1, 1)
  basis = hid / pdf64
  ns, cin, g = len(neigh.ranges), features.shape[1], wf.shape[0]
  k = basis.shape[1]
  h = k // g
  f64 = features.astype(np.float64)
  x = np.zeros((ns, cin, k))
  np.add.at(x, ids[:, 1], f64[ids[:, 0]][:, :, None] * basis[:, None, :])
  co = wf.shape[2]
  dog = np.transpose(d_out.astype(np.float64).reshape(ns, g, co), (1, 0, 2))
  xg = np.transpose(x.reshape(ns, cin, g, h), (2, 0, 1, 3)).reshape(g, ns, cin * h)
  d_wf = np.matmul(np.transpose(xg, (0, 2, 1)), dog)
  dxg = np.matmul(dog, np.transpose(wf.astype(np.float64), (0, 2, 1)))
  dx = np.transpose(dxg.reshape(g, ns, cin, h), (1, 2, 0, 3)).reshape(ns, cin, k)
  dxm = dx[ids[:, 1]]                                     # [M, cin, k]
  d_basis = np.einsum('mck,mc->mk', dxm, f64[ids[:, 0]])
  d_feat = np.zeros_like(f64)
  np.add.at(d_feat, ids[:, 0], np.einsum('mck,mk->mc', dxm, basis))
  d_hid = d_basis / pdf64
  d_pdf = -(d_basis * hid).sum(axis=1) / (pdf64[:, 0] ** 2)
  d_diff, d_w, d_b = kernel_mlp_backward(d_hid, pres, weights, non_linearity)
  d_pin = np.zeros_like(p_in); d_pout = np.zeros_like(p_out)
  np.add.at(d_pin, ids[:, 0], d_diff / radius)
  np.add.at(d_pout, ids[:, 1], -d_diff / radius)
  return dict(d_features=d_feat, d_wf=d_wf, d_weights=d_w, d_biases=d_b, d_points_in=d_pin,
              d_points_out=d_pout, d_pdf=d_pdf, d_basis=d_basis)


def mcconv_forward(features, basis, neigh, wf):
  """MCConv.py:174-194.  wf [num_mlps, Cin*H, Cout/num_mlps] -> [Ns, Cout]."""
  g = wf.shape[0]
  cin = features.shape[1]
  x = orc.basis_proj(basis, features, neigh.original_neigh_ids, neigh.ranges)
  ns, _, k = x.shape
  h = k // g
  xg = np.transpose(x.reshape(ns, cin, g, h), (2, 0, 1, 3)).reshape(g, ns, cin * h)
  out = np.matmul(xg.astype(np.float64), wf.astype(np.float64))
  return np.transpose(out, (1, 0, 2)).reshape(ns, -1).astype(F32), x


def mcconv_backward(features, basis, neigh, wf, x, d_out):
  """Analytic gradients of mcconv_forward: returns (d_wf, d_basis, d_feat)."""
  g = wf.shape[0]
  ns, cin, k = x.shape
  h = k // g
  co = wf.shape[2]
  dog = np.transpose(d_out.reshape(ns, g, co), (1, 0, 2)).astype(np.float64)
  xg = np.transpose(x.reshape(ns, cin, g, h), (2, 0, 1, 3)).reshape(g, ns, cin * h)
  d_wf = np.matmul(np.transpose(xg, (0, 2, 1)).astype(np.float64), dog).astype(F32)
  dxg = np.matmul(dog, np.transpose(wf, (0, 2, 1)).astype(np.float64))
  dx = np.transpose(dxg.reshape(g, ns, cin, h), (1, 2, 0, 3)).reshape(ns, cin, k)
  d_basis, d_feat = orc.basis_proj_grads(basis, features,
                                         neigh.original_neigh_ids, neigh.ranges,
                                         dx.astype(F32))
  return d_wf, d_basis, d_feat, dx.astype(F32)


# ---- KPConv and PointConv (test infrastructure like the rest of this file) ----

def _projected_conv(basis, features, neigh, weights):
  """basis_proj followed by the [Ns, Cin*K] x [Cin*K, Cout] product both layers
  end with (KPConv.py:218-230, PointConv.py:189-200)."""
  x = orc.basis_proj(basis, features, neigh.original_neigh_ids, neigh.ranges)
  ns = x.shape[0]
  return (x.reshape(ns, -1).astype(np.float64) @ weights.astype(np.float64)).astype(F32), x


def kpconv_basis(points_in, points_out, neigh, kernel_points, radius, sigma=1.0,
                 interpolation='linear'):
  """KPConv.py:194-197 with the weightings of :28-56.  kernel_points are the
  layer's points after the 0.75 scaling of :129.  Returns [M, K] unpadded."""
  ids = neigh.original_neigh_ids
  diff = ((points_in[ids[:, 0]] - points_out[ids[:, 1]]) / F32(radius)).astype(F32)
  dist = np.linalg.norm(diff[:, None, :] - kernel_points[None, :, :].astype(F32),
                        axis=2).astype(F32)
  if interpolation == 'linear':
    return np.maximum(F32(1) - dist / F32(sigma), F32(0)).astype(F32)
  s = F32(sigma) / F32(3)
  return np.exp(-(dist / s) ** 2).astype(F32)


def kpconv_forward(features, points_in, points_out, neigh, kernel_points, weights, radius,
                   sigma=1.0, interpolation='linear'):
  """Rigid KPConv (KPConv.py:171-230): the zero padding of the basis and its
  removal (:199-221) cancel, so the unpadded basis is projected directly."""
  k = kernel_points.shape[0]
  basis = kpconv_basis(points_in, points_out, neigh, kernel_points, radius, sigma,
                       interpolation)
  pad = next(c for c in (8, 16, 32, 64) if k <= c)
  padded = np.zeros((basis.shape[0], pad), F32)
  padded[:, :k] = basis
  x = orc.basis_proj(padded, features, neigh.original_neigh_ids, neigh.ranges)[:, :, :k]
  ns = x.shape[0]
  return (x.reshape(ns, -1).astype(np.float64) @ weights.astype(np.float64)).astype(F32)


def pointconv_pdf(pdf, neigh, w1, b1, w2, b2):
  """PointConv.py:173-183: density over the largest density of the sample's
  pairs, then relu(x w1 + b1) w2 + b2."""
  sample = neigh.original_neigh_ids[:, 1]
  mx = np.full(len(neigh.ranges), -np.inf, F32)
  np.maximum.at(mx, sample, pdf.astype(F32))
  cur = (pdf / mx[sample]).astype(F32).reshape(-1, 1)
  hid = np.maximum(cur @ w1.reshape(1, 16).astype(F32) + b1.reshape(1, 16), 0).astype(F32)
  return (hid @ w2.reshape(16, 1).astype(F32) + b2.reshape(1, 1)).astype(F32).reshape(-1)


def pointconv_forward(features, points_in, points_out, neigh, pdf, hidden_w, hidden_b, weights,
                      pdf_weights, pdf_biases, non_linearity='relu'):
  """PointConv.py:160-200 with the kernel inputs of :266-272 (differences not
  divided by the radius)."""
  ids = neigh.original_neigh_ids
  diff = (points_in[ids[:, 0]] - points_out[ids[:, 1]]).astype(F32)
  hid = (diff @ hidden_w.astype(F32) + hidden_b.reshape(1, -1)).astype(F32)
  if non_linearity == 'relu':
    hid = np.maximum(hid, 0)
  elif non_linearity == 'elu':
    hid = np.where(hid > 0, hid, np.expm1(hid)).astype(F32)
  else:
    hid = leaky_relu(hid)
  scale = pointconv_pdf(pdf, neigh, pdf_weights[0], pdf_biases[0], pdf_weights[1],
                        pdf_biases[1])
  basis = (hid / scale.reshape(-1, 1)).astype(F32)
  return _projected_conv(basis, features, neigh, weights)[0], basis


# ---- pooling and 1x1 convolution ------------------------------------------------

LOWEST = np.finfo(F32).min   # what unsorted_segment_max writes for an empty segment


def segment_pool(data, segment_ids, num_segments, mode):
  """tf.math.unsorted_segment_max / _mean as the pooling layers call them
  (Pooling.py:54-57, 93-96, 155-158): mode 'max' or 'avg'."""
  data = np.asarray(data, F32)
  if mode == 'max':
    out = np.full((num_segments, data.shape[1]), LOWEST, F32)
    np.maximum.at(out, segment_ids, data)
    return out
  out = np.zeros((num_segments, data.shape[1]), np.float64)
  np.add.at(out, segment_ids, data)
  cnt = np.bincount(segment_ids, minlength=num_segments).astype(np.float64)
  return (out / np.maximum(cnt, 1)[:, None]).astype(F32)


def neighborhood_pool(features, neigh, mode):
  """Pooling.py:148-158: gather the neighbors' rows, pool them per sample."""
  ids = neigh.original_neigh_ids
  return segment_pool(features[ids[:, 0]], ids[:, 1], len(neigh.ranges), mode)


def global_pool(features, batch_ids, batch_size, mode):
  """Pooling.py:51-57 and :90-96."""
  return segment_pool(features, batch_ids, batch_size, mode)


def conv1x1(features, weights, bias):
  """Conv1x1.py:97."""
  return (features.astype(np.float64) @ weights.astype(np.float64)
          + bias.reshape(1, -1)).astype(F32)


def small_classifier_forward(points, batch_ids, batch_size, features, weights, sample_radii,
                             bn_eps=1e-3, leaky_alpha=0.3, pool_before_head=False):
  """modelnet40_small.py:121-261 (MCConv variant) at inference with freshly
  initialised batch normalisations: hierarchy (PointHierarchy.py:40-98), per
  level MCConv (MCConv.py:163-194, 254-269), BN + LeakyReLU + Conv1x1 + BN +
  LeakyReLU between levels, BN + LeakyReLU + Dense twice as head."""
  bn = F32(1.0 / np.sqrt(1.0 + bn_eps))
  act = lambda x: leaky_relu((x * bn).astype(F32), leaky_alpha)
  levels = point_hierarchy(points, batch_ids, batch_size, list(sample_radii), mode=0)
  x = np.asarray(features, F32)
  last = len(weights["conv"]) - 1
  for i, (w1, b1, wf) in enumerate(weights["conv"]):
    p_in, b_in = levels[i][0], levels[i][1]
    p_out, b_out = levels[i + 1][0], levels[i + 1][1]
    r = F32(sample_radii[i])
    grid = Grid(p_in, b_in, batch_size, r)
    nb = Neighborhood(grid, r, p_out, b_out)
    basis, _, _ = mcconv_basis(p_in, p_out, nb, nb.get_pdf(), w1, b1, r)
    x, _ = mcconv_forward(x, basis, nb, wf)
    if i < last:
      x = act(x)
      x = act(conv1x1(x, *weights["conv1x1"][i]))
  if pool_before_head:
    # a last radius that leaves several points per cloud: mean over the cloud
    # (GlobalAveragePooling, Pooling.py:90-96) instead of picking the single row
    x = global_pool(x, levels[-1][1], batch_size, 'avg')
  else:
    x = x[np.argsort(levels[-1][1], kind='stable')]
  x = act(x)
  for w, b in weights["dense"][:-1]:
    x = act(conv1x1(x, w, b))
  return conv1x1(x, *weights["dense"][-1])
