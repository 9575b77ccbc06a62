"""Seeded synthetic inputs with the shapes, sizes and value distributions of the
benchmark configurations (they stand in for ModelNet40-style data, which is not
shipped).  NumPy only; every generator is a pure function of its seed."""
import numpy as np

F32 = np.float32


def uniform_clouds(num_clouds, points_per_cloud, seed, dims=3):
  """Clouds of `points_per_cloud` points uniform in [0,1)^dims."""
  rng = np.random.default_rng(seed)
  pts = rng.random((num_clouds * points_per_cloud, dims), dtype=np.float64).astype(F32)
  bid = np.repeat(np.arange(num_clouds, dtype=np.int32), points_per_cloud)
  return pts, bid


def _sphere_surface(rng, n, centre, diameter):
  v = rng.normal(size=(n, 3))
  v /= np.linalg.norm(v, axis=1, keepdims=True)
  return centre + 0.5 * diameter * v


def _box_surface(rng, n, centre, edge):
  p = rng.random((n, 3)) - 0.5
  face = rng.integers(0, 6, n)
  axis, side = face // 2, (face % 2) - 0.5
  p[np.arange(n), axis] = side
  return centre + edge * p


def surface_clouds(num_clouds, seed, min_points=8192, max_points=65536, shapes=8, noise=0.005):
  """Clouds of `shapes` random spheres / axis-aligned boxes (centres uniform in
  [0,1)^3, sizes uniform in [0.1,0.4]) sampled on their surfaces plus Gaussian
  noise; point counts uniform in [min_points, max_points]."""
  rng = np.random.default_rng(seed)
  sizes = rng.integers(min_points, max_points + 1, num_clouds)
  pts, bid = [], []
  for c, n in enumerate(sizes):
    per = np.full(shapes, n // shapes)
    per[: n - per.sum()] += 1
    for s in range(shapes):
      centre = rng.random(3)
      size = rng.uniform(0.1, 0.4)
      gen = _sphere_surface if s % 2 == 0 else _box_surface
      pts.append(gen(rng, per[s], centre, size))
    bid.append(np.full(n, c, np.int32))
  pts = np.concatenate(pts) + rng.normal(scale=noise, size=(int(sizes.sum()), 3))
  return pts.astype(F32), np.concatenate(bid)


def gaussian_mixture_clouds(num_clouds, points_per_cloud, seed, components=12):
  """Clouds drawn from a mixture of anisotropic Gaussians (centres uniform in
  [0,1)^3, per-axis sigma uniform in [0.01, 0.1])."""
  rng = np.random.default_rng(seed)
  pts = []
  for _ in range(num_clouds):
    centres = rng.random((components, 3))
    sigma = rng.uniform(0.01, 0.1, (components, 3))
    comp = rng.integers(0, components, points_per_cloud)
    pts.append(centres[comp] + sigma[comp] * rng.normal(size=(points_per_cloud, 3)))
  bid = np.repeat(np.arange(num_clouds, dtype=np.int32), points_per_cloud)
  return np.concatenate(pts).astype(F32), bid


def glorot_uniform(rng, fan_in, fan_out, shape):
  lim = np.sqrt(6.0 / (fan_in + fan_out))
  return rng.uniform(-lim, lim, shape).astype(F32)


def mcconv_weights(seed, dims, cin, cout, num_mlps=1, hidden=16):
  """Glorot-uniform kernel-MLP and final weights in the reference's layouts
  (pylib/pc/layers/MCConv.py:104-135): w1 [num_mlps, dims, hidden],
  b1 [num_mlps, 1, hidden], wf [num_mlps, cin*hidden, cout/num_mlps]."""
  rng = np.random.default_rng(seed)
  w1 = glorot_uniform(rng, dims, hidden, (num_mlps, dims, hidden))
  b1 = np.zeros((num_mlps, 1, hidden), F32)
  wf = glorot_uniform(rng, cin * hidden, cout // num_mlps,
                      (num_mlps, cin * hidden, cout // num_mlps))
  return w1, b1, wf


def unit_sphere_shapes(num_clouds, points_per_cloud, seed):
  """Clouds of points on random ellipsoids, boxes and cylinders, centred and
  scaled into the unit sphere: stand-ins with the shape of the 1024-point
  ModelNet40 samples that modelnet40_small.py trains on."""
  rng = np.random.default_rng(seed)
  pts = np.empty((num_clouds, points_per_cloud, 3), F32)
  for c in range(num_clouds):
    kind = c % 3
    axes = rng.uniform(0.3, 1.0, 3)
    n = points_per_cloud
    if kind == 0:     # ellipsoid
      v = rng.normal(size=(n, 3))
      p = v / np.linalg.norm(v, axis=1, keepdims=True) * axes
    elif kind == 1:   # box
      p = rng.uniform(-1, 1, (n, 3))
      face = rng.integers(0, 3, n)
      p[np.arange(n), face] = np.sign(rng.uniform(-1, 1, n))
      p = p * axes
    else:             # cylinder along z, side and caps
      ang = rng.uniform(0, 2 * np.pi, n)
      side = rng.uniform(size=n) < 0.7
      rad = np.where(side, 1.0, np.sqrt(rng.uniform(size=n)))
      z = np.where(side, rng.uniform(-1, 1, n), np.sign(rng.uniform(-1, 1, n)))
      p = np.stack([rad * np.cos(ang) * axes[0], rad * np.sin(ang) * axes[0], z * axes[2]], 1)
    p = p - p.mean(axis=0)
    pts[c] = (p / np.linalg.norm(p, axis=1).max()).astype(F32)
  bid = np.repeat(np.arange(num_clouds, dtype=np.int32), points_per_cloud)
  return pts.reshape(-1, 3), bid


def small_classifier_weights(seed, feature_sizes=(1, 128, 256, 512, 1024, 1024, 40), num_mlps=4,
                             hidden=8, head_layers=2):
  """Random-init weights of the modelnet40_small.py network (MCConv variant):
  per level the MCConv weights, then a Conv1x1 except after the last level,
  then the dense layers of the head (feature_sizes = input, one size per level,
  one per head layer)."""
  rng = np.random.default_rng(seed)
  levels = len(feature_sizes) - 1 - head_layers
  out = {"conv": [], "conv1x1": [], "dense": []}
  for i in range(levels):
    cin, cout = feature_sizes[i], feature_sizes[i + 1]
    out["conv"].append(mcconv_weights(seed + 1 + i, 3, cin, cout, num_mlps, hidden))
    if i < levels - 1:
      out["conv1x1"].append((glorot_uniform(rng, cout, cout, (cout, cout)),
                             (rng.normal(size=(1, cout)) * 0.01).astype(F32)))
  for i in range(levels, levels + head_layers):
    cin, cout = feature_sizes[i], feature_sizes[i + 1]
    out["dense"].append((glorot_uniform(rng, cin, cout, (cin, cout)),
                         (rng.normal(size=(1, cout)) * 0.01).astype(F32)))
  return out
