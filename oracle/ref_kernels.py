"""ctypes binding of oracle/_ref/libtfg_ref_kernels.so: the reference's own CUDA
kernels behind oracle/ref_kernels_harness.cu (TEST INFRASTRUCTURE ONLY; needs a
GPU).  NumPy arrays in, NumPy arrays out; D = 3."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libtfg_ref_kernels.so")
_lib = None

_vp = ctypes.c_void_p
_int = ctypes.c_int
_ll = ctypes.c_longlong


def available():
  return os.path.exists(LIB_PATH)


def lib():
  global _lib
  if _lib is None:
    _lib = ctypes.CDLL(LIB_PATH)
    _lib.ref_find_neighbors.restype = _ll
    _lib.ref_sampling.restype = _ll
  return _lib


def _p(a):
  return _vp(a.ctypes.data) if a is not None else _vp(0)


def _c(a, dt):
  return np.ascontiguousarray(a, dtype=dt)


def _check(rc):
  if rc != 0:
    raise RuntimeError("reference kernel harness reported CUDA error %d" % rc)


def compute_keys(points, batch_ids, scaled_aabb_min, num_cells, inv_cell_sizes):
  pts, bid = _c(points, np.float32), _c(batch_ids, np.int32)
  smin, nc, ic = _c(scaled_aabb_min, np.float32), _c(num_cells, np.int32), _c(inv_cell_sizes, np.float32)
  keys = np.empty(len(pts), np.int64)
  ms = ctypes.c_float(0)
  _check(lib().ref_compute_keys(_int(len(pts)), _p(pts), _p(bid), _int(len(smin)), _p(smin), _p(nc),
                                _p(ic), _p(keys), ctypes.byref(ms)))
  return keys, ms.value


def build_grid_ds(sorted_keys, num_cells, batch_size):
  keys, nc = _c(sorted_keys, np.int64), _c(num_cells, np.int32)
  ds = np.zeros((batch_size, nc[0], nc[1], 2), np.int32)
  ms = ctypes.c_float(0)
  _check(lib().ref_build_grid_ds(_int(len(keys)), _p(keys), _p(nc), _int(batch_size), _p(ds),
                                 ctypes.byref(ms)))
  return ds, ms.value


def find_neighbors(samples, samples_batch_ids, points, point_keys, grid_ds, num_cells,
                   scaled_aabb_min, inv_cell_sizes, inv_radii, capacity):
  smp, sb = _c(samples, np.float32), _c(samples_batch_ids, np.int32)
  pts, keys = _c(points, np.float32), _c(point_keys, np.int64)
  ds, nc = _c(grid_ds, np.int32), _c(num_cells, np.int32)
  smin, ic, ir = _c(scaled_aabb_min, np.float32), _c(inv_cell_sizes, np.float32), _c(inv_radii, np.float32)
  ranges = np.zeros(len(smp), np.int32)
  neigh = np.zeros((capacity, 2), np.int32)
  ms = ctypes.c_float(0)
  m = lib().ref_find_neighbors(_int(len(smp)), _p(smp), _p(sb), _int(len(pts)), _p(pts), _p(keys),
                               _p(ds), _int(ds.shape[0]), _p(nc), _p(smin), _p(ic), _p(ir),
                               _p(ranges), _p(neigh), _ll(capacity), ctypes.byref(ms))
  if m < 0:
    raise RuntimeError("reference FindNeighbors failed")
  return ranges, neigh[:m], ms.value


def compute_pdf(points, neighbors, ranges, inv_bandwidth, inv_radii, mode=0, pdf_grads=None):
  pts, nb, rg = _c(points, np.float32), _c(neighbors, np.int32), _c(ranges, np.int32)
  ib, ir = _c(inv_bandwidth, np.float32), _c(inv_radii, np.float32)
  pdf = np.zeros(len(pts), np.float32)
  g = _c(pdf_grads, np.float32) if pdf_grads is not None else None
  go = np.zeros((len(pts), 3), np.float32) if g is not None else None
  ms = ctypes.c_float(0)
  _check(lib().ref_compute_pdf(_int(mode), _int(len(pts)), _p(pts), _ll(len(nb)), _p(nb), _p(rg),
                               _p(ib), _p(ir), _p(pdf), _p(g), _p(go), ctypes.byref(ms)))
  return pdf, go, ms.value


def basis_proj(basis, features, neighbors, ranges, in_grads=None):
  bs, ft = _c(basis, np.float32), _c(features, np.float32)
  nb, rg = _c(neighbors, np.int32), _c(ranges, np.int32)
  k, c, ns = bs.shape[1], ft.shape[1], len(rg)
  out = np.zeros((ns, c, k), np.float32)
  g = _c(in_grads, np.float32) if in_grads is not None else None
  db = np.zeros_like(bs) if g is not None else None
  df = np.zeros_like(ft) if g is not None else None
  ms = ctypes.c_float(0)
  _check(lib().ref_basis_proj(_int(k), _int(c), _int(ns), _int(len(ft)), _ll(len(nb)), _p(bs),
                              _p(ft), _p(nb), _p(rg), _p(out), _p(g), _p(db), _p(df),
                              ctypes.byref(ms)))
  return out, db, df, ms.value


def sampling(points, batch_ids, point_keys, num_cells, neighbors, ranges, mode):
  pts, bid = _c(points, np.float32), _c(batch_ids, np.int32)
  keys, nc = _c(point_keys, np.int64), _c(num_cells, np.int32)
  nb, rg = _c(neighbors, np.int32), _c(ranges, np.int32)
  n = len(pts)
  op, ob, oi = np.zeros((n, 3), np.float32), np.zeros(n, np.int32), np.zeros(n, np.int32)
  ms = ctypes.c_float(0)
  s = lib().ref_sampling(_int(mode), _int(n), _p(pts), _p(bid), _p(keys), _p(nc), _ll(len(nb)),
                         _p(nb), _p(rg), _p(op), _p(ob), _p(oi), ctypes.byref(ms))
  if s < 0:
    raise RuntimeError("reference Sampling failed")
  return op[:s], ob[:s], oi[:s], ms.value
