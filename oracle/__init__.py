"""CPU oracle for the tfg_custom_ops hot path (TEST INFRASTRUCTURE ONLY).

ctypes bindings of ``tfgpc_oracle.c`` over NumPy arrays.  Only the tests, the
smoke check and the benchmark's CPU-baseline legs may import this package; the
product package never does.

The functions mirror the reference op signatures
(custom_ops/tfg_custom_ops/*/cc/ops/*_ops.cpp) with NumPy arrays in place of
tensors.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtfgpc_oracle.so")
_lib = None

_i64 = ctypes.c_int64
_int = ctypes.c_int
_vp = ctypes.c_void_p


def build(force=False):
  """Compiles the C oracle next to its source (gcc, seconds)."""
  src = os.path.join(_HERE, "tfgpc_oracle.c")
  if (not force and os.path.exists(_LIB_PATH)
      and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
    return _LIB_PATH
  subprocess.check_call(["make", "-s", "-B", "-C", _HERE])
  return _LIB_PATH


def lib():
  global _lib
  if _lib is None:
    build()
    _lib = ctypes.CDLL(_LIB_PATH)
    _lib.orc_find_neighbors.restype = _i64
    _lib.orc_sampling_poisson.restype = _i64
    _lib.orc_sampling_avg.restype = _i64
    _lib.orc_num_threads.restype = _int
  return _lib


def num_threads():
  return int(lib().orc_num_threads())


def set_num_threads(n):
  lib().orc_set_num_threads(_int(int(n)))


def _f32(a):
  return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
  return np.ascontiguousarray(a, dtype=np.int32)


def _i64a(a):
  return np.ascontiguousarray(a, dtype=np.int64)


def _p(a):
  return _vp(a.ctypes.data) if a is not None else _vp(0)


def compute_keys(points, batch_ids, scaled_aabb_min, num_cells, inv_cell_sizes,
                 fused=True):
  """ComputeKeys (compute_keys_ops.cpp:29-41)."""
  points = _f32(points); batch_ids = _i32(batch_ids)
  smin = _f32(scaled_aabb_min); nc = _i32(num_cells); ic = _f32(inv_cell_sizes)
  n, d = points.shape
  keys = np.empty(n, dtype=np.int64)
  lib().orc_compute_keys(_int(d), _i64(n), _p(points), _p(batch_ids), _p(smin),
                         _p(nc), _p(ic), _int(int(fused)), _p(keys))
  return keys


def sort_keys_desc(keys):
  """tf.argsort(keys, 'DESCENDING') of pylib/pc/Grid.py:56-57 (stable)."""
  keys = _i64a(keys)
  n = keys.shape[0]
  perm = np.empty(n, dtype=np.int32)
  skeys = np.empty(n, dtype=np.int64)
  lib().orc_sort_keys_desc(_i64(n), _p(keys), _p(perm), _p(skeys))
  return perm, skeys


def build_grid_ds(sorted_keys, num_cells, batch_size):
  """BuildGridDs (build_grid_ds_ops.cpp:27-40)."""
  sorted_keys = _i64a(sorted_keys); nc = _i32(num_cells)
  d = nc.shape[0]
  ds = np.zeros((batch_size, nc[0], nc[1], 2), dtype=np.int32)
  lib().orc_build_grid_ds(_int(d), _i64(sorted_keys.shape[0]), _p(sorted_keys),
                          _p(nc), _int(batch_size), _p(ds))
  return ds


def find_neighbors(samples, samples_batch_ids, points, point_keys, num_cells,
                   scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs=0,
                   fused=True):
  """FindNeighbors (find_neighbors_ops.cpp:42-61) in canonical order.

  The grid tube structure is not an input: the oracle searches the sorted keys
  directly, which visits the same candidate cells."""
  samples = _f32(samples); sb = _i32(samples_batch_ids); points = _f32(points)
  keys = _i64a(point_keys); nc = _i32(num_cells); smin = _f32(scaled_aabb_min)
  ic = _f32(inv_cell_sizes); ir = _f32(inv_radii)
  ns, d = samples.shape
  n = points.shape[0]
  ranges = np.zeros(ns, dtype=np.int32)
  args = (_int(d), _i64(ns), _p(samples), _p(sb), _i64(n), _p(points), _p(keys),
          _p(nc), _p(smin), _p(ic), _p(ir), _int(max_neighs), _int(int(fused)),
          _p(ranges))
  m = lib().orc_find_neighbors(*args, _vp(0))
  neigh = np.zeros((m, 2), dtype=np.int32)
  if m:
    lib().orc_find_neighbors(*args, _p(neigh))
  return ranges, neigh


def compute_pdf(points, neighbors, ranges, inv_bandwidth, inv_radii, mode=0):
  """ComputePdf / ComputePdfWithPtGrads (compute_pdf_ops.cpp:28-56)."""
  points = _f32(points); neighbors = _i32(neighbors); ranges = _i32(ranges)
  ib = _f32(inv_bandwidth); ir = _f32(inv_radii)
  n, d = points.shape
  pdf = np.zeros(n, dtype=np.float32)
  lib().orc_compute_pdf(_int(d), _int(mode), _i64(n), _p(points), _p(neighbors),
                        _p(ranges), _p(ib), _p(ir), _p(pdf))
  return pdf


def compute_pdf_pt_grads(points, neighbors, ranges, inv_bandwidth, inv_radii,
                         pdf_grads, mode=0):
  """ComputePdfPtGrads (compute_pdf_ops.cpp:58-74)."""
  points = _f32(points); neighbors = _i32(neighbors); ranges = _i32(ranges)
  ib = _f32(inv_bandwidth); ir = _f32(inv_radii); g = _f32(pdf_grads)
  n, d = points.shape
  out = np.zeros((n, d), dtype=np.float32)
  lib().orc_compute_pdf_pt_grads(_int(d), _int(mode), _i64(n), _p(points),
                                 _p(neighbors), _p(ranges), _p(ib), _p(ir),
                                 _p(g), _p(out))
  return out


def basis_proj(basis, features, neighbors, ranges):
  """BasisProj (basis_proj_ops.cpp:25-39)."""
  basis = _f32(basis); features = _f32(features)
  neighbors = _i32(neighbors); ranges = _i32(ranges)
  k = basis.shape[1]; c = features.shape[1]; ns = ranges.shape[0]
  out = np.zeros((ns, c, k), dtype=np.float32)
  lib().orc_basis_proj(_int(k), _int(c), _i64(ns), _p(basis), _p(features),
                       _p(neighbors), _p(ranges), _p(out))
  return out


def basis_proj_grads(basis, features, neighbors, ranges, in_grads):
  """BasisProjGrads (basis_proj_ops.cpp:41-53)."""
  basis = _f32(basis); features = _f32(features)
  neighbors = _i32(neighbors); ranges = _i32(ranges); g = _f32(in_grads)
  k = basis.shape[1]; c = features.shape[1]; ns = ranges.shape[0]
  dbasis = np.zeros_like(basis); dfeat = np.zeros_like(features)
  lib().orc_basis_proj_grads(_int(k), _int(c), _i64(ns),
                             _i64(features.shape[0]), _p(basis), _p(features),
                             _p(neighbors), _p(ranges), _p(g), _p(dbasis),
                             _p(dfeat))
  return dbasis, dfeat


def sampling(points, batch_ids, point_keys, num_cells, neighbors, ranges, mode):
  """Sampling (sampling_ops.cpp:33-53); mode 0 = Poisson disk, 1 = cell average
  (sampling_ops.cpp:141,174).  Canonical output order."""
  points = _f32(points); batch_ids = _i32(batch_ids); keys = _i64a(point_keys)
  nc = _i32(num_cells)
  n, d = points.shape
  if mode == 0:
    neighbors = _i32(neighbors); ranges = _i32(ranges)
    used = np.zeros(n, dtype=np.int32)
    idx = np.zeros(n, dtype=np.int32)
    s = lib().orc_sampling_poisson(_int(d), _i64(n), _p(keys), _p(nc),
                                   _p(neighbors), _p(ranges), _p(used), _p(idx))
    idx = idx[:s].copy()
    return points[idx], batch_ids[idx], idx
  s = lib().orc_sampling_avg(_int(d), _i64(n), _p(points), _p(keys), _p(nc),
                             _vp(0), _vp(0))
  out = np.zeros((s, d), dtype=np.float32)
  ob = np.zeros(s, dtype=np.int32)
  lib().orc_sampling_avg(_int(d), _i64(n), _p(points), _p(keys), _p(nc), _p(out),
                         _p(ob))
  return out, ob, np.zeros(1, dtype=np.int32)
