"""The eight callables of the reference's `tfg_custom_ops` package
(custom_ops/tfg_custom_ops/__init__.py:16-26) over torch CUDA tensors.

Names, argument order and meaning follow the TensorFlow op registrations; each
function marshals its tensors into one or two C-ABI calls (include/tfgpc.h) on
torch's current stream.  torch only owns the device memory.  Argument errors
raise `TfgpcError` with the reference's InvalidArgument conditions.
"""
import ctypes

import torch

from . import _lib
from ._lib import c_i64, c_int, c_sz, ptr


def _stream():
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32(t):
  return t.contiguous().to(torch.float32)


def _i32(t):
  return t.contiguous().to(torch.int32)


def _dev_check(*tensors):
  for t in tensors:
    if not t.is_cuda:
      raise ValueError("tfg_custom_ops are registered for the GPU only: got a CPU tensor")


def _workspace(nbytes, device):
  return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


def compute_keys(points, batch_ids, scaled_aabb_min, num_cells, inv_cell_sizes):
  """ComputeKeys (compute_keys/cc/ops/compute_keys_ops.cpp:29-41)."""
  points, smin, inv = _f32(points), _f32(scaled_aabb_min), _f32(inv_cell_sizes)
  batch_ids, num_cells = _i32(batch_ids), _i32(num_cells)
  _dev_check(points, batch_ids, smin, num_cells, inv)
  n, d = points.shape
  if batch_ids.shape[0] != n:
    raise _lib.TfgpcError(1, "ComputeKeysOp expects the same number of points as batch ids")
  if smin.dim() != 2 or smin.shape[1] != d or num_cells.shape[0] != d or inv.shape[0] != d:
    raise _lib.TfgpcError(1, "ComputeKeysOp expects inputs with the dimension of the points")
  keys = torch.empty(n, dtype=torch.int64, device=points.device)
  _lib.check(_lib.lib().tfgpc_compute_keys(
      _stream(), c_int(d), c_i64(n), ptr(points), ptr(batch_ids), c_i64(smin.shape[0]),
      ptr(smin), ptr(num_cells), ptr(inv), ptr(keys)))
  return keys


def compute_aabb(points, batch_ids, batch_size):
  """Per-cloud bounding box (unsorted_segment_min/max of PointCloud.py:38-43)."""
  points, batch_ids = _f32(points), _i32(batch_ids)
  _dev_check(points, batch_ids)
  n, d = points.shape
  mn = torch.empty((batch_size, d), dtype=torch.float32, device=points.device)
  mx = torch.empty_like(mn)
  _lib.check(_lib.lib().tfgpc_compute_aabb(
      _stream(), c_int(d), c_i64(n), ptr(points), ptr(batch_ids), c_i64(batch_size), ptr(mn),
      ptr(mx)))
  return mn, mx


def sort_keys_desc(keys, points=None, batch_ids=None, key_bits=0):
  """tf.argsort(keys, 'DESCENDING') plus the gathers of pylib/pc/Grid.py:56-64
  in one call.  Returns (perm, sorted_keys[, sorted_points, sorted_batch_ids])."""
  keys = keys.contiguous()
  _dev_check(keys)
  n = keys.shape[0]
  dev = keys.device
  perm = torch.empty(n, dtype=torch.int32, device=dev)
  skeys = torch.empty(n, dtype=torch.int64, device=dev)
  spts = sbid = None
  d = 3
  if points is not None:
    points, batch_ids = _f32(points), _i32(batch_ids)
    d = points.shape[1]
    spts = torch.empty_like(points)
    sbid = torch.empty_like(batch_ids)
  nbytes = _lib.lib().tfgpc_sort_keys_workspace_bytes(c_i64(n))
  ws = _workspace(nbytes, dev)
  _lib.check(_lib.lib().tfgpc_sort_keys_desc(
      _stream(), c_int(d), c_i64(n), c_int(key_bits), ptr(keys), ptr(points), ptr(batch_ids),
      ptr(perm), ptr(skeys), ptr(spts), ptr(sbid), ptr(ws), c_sz(nbytes)))
  if points is None:
    return perm, skeys
  return perm, skeys, spts, sbid


def build_grid_ds(keys, num_cells_gpu, num_cells_cpu, batch_size):
  """BuildGridDs (build_grid_ds/cc/ops/build_grid_ds_ops.cpp:27-40).  The third
  input lives in host memory, as the op's HostMemory("num_cells_cpu") asks."""
  keys = keys.contiguous()
  num_cells_gpu = _i32(num_cells_gpu)
  _dev_check(keys, num_cells_gpu)
  host = _i32(torch.as_tensor(num_cells_cpu).cpu())
  d = host.shape[0]
  if batch_size <= 0:
    raise _lib.TfgpcError(1, "BuildGridDsOp expects a positive batch size")
  ds = torch.empty((batch_size, int(host[0]), int(host[1]), 2), dtype=torch.int32,
                   device=keys.device)
  _lib.check(_lib.lib().tfgpc_build_grid_ds(
      _stream(), c_int(d), c_i64(keys.shape[0]), ptr(keys), ptr(num_cells_gpu),
      ctypes.c_void_p(host.data_ptr()), c_i64(batch_size), ptr(ds)))
  return ds


class NeighborCount:
  """Result of the count pass of FindNeighbors: the ranges [Ns], the number of
  pairs, and the checked arguments the fill pass needs again."""

  def __init__(self, ranges, total, args, order, dims):
    self.ranges, self.total, self.args, self.order, self.dims = ranges, total, args, order, dims


def find_neighbors_count(samples, samples_batch_ids, points, point_keys, grid_acc_ds, num_cells,
                         scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs=0,
                         sample_order=None):
  """First half of FindNeighbors (find_neighbors_ops.cpp:158-187): ranges and the
  number of pairs.  Blocks until the count is on the host."""
  samples, points = _f32(samples), _f32(points)
  sbid, nc = _i32(samples_batch_ids), _i32(num_cells)
  keys, ds = point_keys.contiguous(), _i32(grid_acc_ds)
  smin, inv_c, inv_r = _f32(scaled_aabb_min), _f32(inv_cell_sizes), _f32(inv_radii)
  _dev_check(samples, sbid, points, keys, ds, nc, smin, inv_c, inv_r)
  ns, d = samples.shape
  n = points.shape[0]
  if not (nc.shape[0] == d and points.shape[1] == d and smin.shape[1] == d
          and inv_c.shape[0] == d and inv_r.shape[0] == d):
    raise _lib.TfgpcError(1, "FindNeighborsOp expects inputs with the dimension of the samples")
  if sbid.shape[0] != ns:
    raise _lib.TfgpcError(1, "FindNeighborsOp expects the same number of batch ids as samples.")
  if keys.shape[0] != n:
    raise _lib.TfgpcError(1, "FindNeighborsOp expects the same number of keys as points.")
  if ds.dim() != 4 or ds.shape[3] != 2:
    raise _lib.TfgpcError(1, "FindNeighborsOp expects a grid acceleration data structure with "
                          "the right format (B, X, Y, 2).")
  dev = samples.device
  ranges = torch.empty(ns, dtype=torch.int32, device=dev)
  nbytes = _lib.lib().tfgpc_find_neighbors_workspace_bytes(c_i64(ns))
  ws = _workspace(nbytes, dev)
  total = c_i64(0)
  order = None
  if sample_order is not None:
    order = _i32(sample_order)
    _dev_check(samples, order)
    if order.shape[0] != ns:
      raise _lib.TfgpcError(1, "FindNeighborsOp expects one entry of the order per sample.")
  # (tensors are kept alive by the object: the pointers below are reused by the fill pass)
  keep = (samples, sbid, points, keys, ds, nc, smin, inv_c, inv_r)
  head = (c_int(d), c_i64(ns), ptr(samples), ptr(sbid))
  tail = (c_i64(n), ptr(points), ptr(keys), ptr(ds), c_i64(ds.shape[0]), ptr(nc), ptr(smin),
          ptr(inv_c), ptr(inv_r), c_int(int(max_neighs)))
  lib = _lib.lib()
  if order is None:
    _lib.check(lib.tfgpc_find_neighbors_count(_stream(), *head, *tail, ptr(ranges), ptr(ws),
                                              c_sz(nbytes), ctypes.byref(total)))
  else:
    _lib.check(lib.tfgpc_find_neighbors_count_ordered(_stream(), *head, ptr(order), *tail,
                                                      ptr(ranges), ptr(ws), c_sz(nbytes),
                                                      ctypes.byref(total)))
  return NeighborCount(ranges, int(total.value), (head, tail, keep), order, d)


def find_neighbors_fill(count, sorted_indices=None, inv_bandwidth=None, pdf_mode=None):
  """Second half of FindNeighbors (find_neighbors_ops.cpp:188-249) for a
  NeighborCount: neigh_indices [M, 2].  With sorted_indices the same pass also
  writes the pairs with the neighbor's original index: (neigh_indices,
  original_ids [M, 2]); with a pdf_mode (and inv_bandwidth for mode 0) also the
  density at every sample: (neigh_indices, original_ids, sample_pdf [Ns])."""
  head, tail, _ = count.args
  dev = count.ranges.device
  m = count.total
  neigh = torch.empty((m, 2), dtype=torch.int32, device=dev)
  lib = _lib.lib()
  if sorted_indices is None:
    if count.order is None:
      _lib.check(lib.tfgpc_find_neighbors_fill(_stream(), *head, *tail, ptr(count.ranges),
                                               c_i64(m), ptr(neigh)))
    else:
      _lib.check(lib.tfgpc_find_neighbors_fill_ordered(_stream(), *head, ptr(count.order), *tail,
                                                       ptr(count.ranges), c_i64(m), ptr(neigh)))
    return neigh
  sorted_indices = _i32(sorted_indices)
  inv_bw = None if inv_bandwidth is None else _f32(inv_bandwidth)
  if pdf_mode == 0 and (inv_bw is None or inv_bw.shape[0] != count.dims):
    raise _lib.TfgpcError(1, "ComputePDFOp expects one inverse bandwidth per dimension")
  ids = torch.empty((m, 2), dtype=torch.int32, device=dev)
  pdf = (None if pdf_mode is None else
         torch.empty(count.ranges.shape[0], dtype=torch.float32, device=dev))
  _lib.check(lib.tfgpc_find_neighbors_fill_fused(
      _stream(), *head, ptr(count.order), *tail, ptr(count.ranges), c_i64(m), ptr(sorted_indices),
      ptr(inv_bw), c_int(int(pdf_mode or 0)), ptr(neigh), ptr(ids), ptr(pdf)))
  return (neigh, ids) if pdf is None else (neigh, ids, pdf)


def find_neighbors(samples, samples_batch_ids, points, point_keys, grid_acc_ds, num_cells,
                   scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs=0, sample_order=None):
  """FindNeighbors (find_neighbors/cc/ops/find_neighbors_ops.cpp:42-61).
  Returns (samples_neigh_indices [Ns], neigh_indices [M, 2]).  sample_order, a
  permutation of the sample indices, only sets the sequence the samples are
  worked on in (same result; faster when it keeps spatial neighbors together)."""
  count = find_neighbors_count(samples, samples_batch_ids, points, point_keys, grid_acc_ds,
                               num_cells, scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs,
                               sample_order)
  return count.ranges, find_neighbors_fill(count)


def _host_floats(values, d):
  return (ctypes.c_float * d)(*[float(v) for v in values])


def grid_cells(points, batch_ids, batch_size, cell_sizes, radii):
  """Bounding boxes (widened by 1e-9), cells per dimension, scaled box minima and
  inverse cell sizes / radii of a cloud, all left on the device, without a
  blocking read (tfgpc_grid_cells): the part of Grid.py:38-48 before the cell
  counts are needed on the host.  For a shard of a distributed batch the caller
  max-reduces `num_cells` over the ranks and hands the dict to
  grid_neighborhood_count(cells=...)."""
  points, bid = _f32(points), _i32(batch_ids)
  _dev_check(points, bid)
  n, d = points.shape
  dev, b = points.device, int(batch_size)
  f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
  c = dict(aabb_min=f32(b, d), aabb_max=f32(b, d),
           num_cells=torch.empty(d, dtype=torch.int32, device=dev), scaled_aabb_min=f32(b, d),
           inv_cell_sizes=f32(d), inv_radii=f32(d))
  _lib.check(_lib.lib().tfgpc_grid_cells(
      _stream(), c_int(d), c_i64(n), ptr(points), ptr(bid), c_i64(b), _host_floats(cell_sizes, d),
      _host_floats(radii, d), ptr(c["aabb_min"]), ptr(c["aabb_max"]), ptr(c["num_cells"]),
      ptr(c["scaled_aabb_min"]), ptr(c["inv_cell_sizes"]), ptr(c["inv_radii"])))
  return c


def grid_neighborhood_count(points, batch_ids, batch_size, cell_sizes, radii, max_cells,
                            samples=None, samples_batch_ids=None, samples_are_points=0,
                            max_neighs=0, cells=None):
  """Grid of a cloud and the count pass of one neighborhood on it in a single
  call with a single blocking read (tfgpc_grid_neighborhood_count).  cell_sizes
  and radii are sequences of D floats (host).  Returns a dict with the grid's
  arrays, the NeighborCount of the neighborhood and the cell counts on the host;
  raises TfgpcError(3) if a dimension needs more than max_cells cells (the
  exception's `num_cells` attribute then holds what the grid asked for).
  cells: the dict of grid_cells for this cloud, its num_cells possibly reduced
  over the shards of a batch; the call then continues from those counts."""
  points, bid = _f32(points), _i32(batch_ids)
  _dev_check(points, bid)
  n, d = points.shape
  dev = points.device
  if samples_are_points == 0:
    samples, sbid = _f32(samples), _i32(samples_batch_ids)
    ns = samples.shape[0]
  else:
    samples = sbid = None
    ns = n
  b = int(batch_size)
  lib = _lib.lib()
  f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
  i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device=dev)
  i64 = lambda *shape: torch.empty(shape, dtype=torch.int64, device=dev)
  g = dict(keys=i64(n), sorted_indices=i32(n), sorted_keys=i64(n), sorted_points=f32(n, d),
           sorted_batch_ids=i32(n), num_cells=i32(d))
  if cells is None:
    g.update(aabb_min=f32(b, d), aabb_max=f32(b, d), scaled_aabb_min=f32(b, d),
             inv_cell_sizes=f32(d), inv_radii=f32(d))
    cells_in = None
  else:
    g.update({k: cells[k] for k in ("aabb_min", "aabb_max", "scaled_aabb_min", "inv_cell_sizes",
                                     "inv_radii")})
    cells_in = _i32(cells["num_cells"])
  ds_elems = lib.tfgpc_grid_neighborhood_ds_elems(c_int(d), c_i64(b), c_int(int(max_cells)))
  ds_flat = i32(ds_elems)
  ranges = i32(ns)
  nbytes = lib.tfgpc_grid_neighborhood_workspace_bytes(c_i64(n), c_i64(ns))
  ws = _workspace(nbytes, dev)
  cs, rr = _host_floats(cell_sizes, d), _host_floats(radii, d)
  nc_host = (ctypes.c_int32 * d)()
  total = c_i64(0)
  code = lib.tfgpc_grid_neighborhood_count(
      _stream(), c_int(d), c_i64(n), ptr(points), ptr(bid), c_i64(b), cs, rr, c_int(int(max_cells)),
      ptr(cells_in), c_i64(ns), ptr(samples), ptr(sbid), c_int(int(samples_are_points)), c_int(int(max_neighs)),
      ptr(g["aabb_min"]), ptr(g["aabb_max"]), ptr(g["num_cells"]), ptr(g["scaled_aabb_min"]),
      ptr(g["inv_cell_sizes"]), ptr(g["inv_radii"]), ptr(g["keys"]), ptr(g["sorted_indices"]),
      ptr(g["sorted_keys"]), ptr(g["sorted_points"]), ptr(g["sorted_batch_ids"]), ptr(ds_flat),
      ptr(ranges), ptr(ws), c_sz(nbytes), nc_host, ctypes.byref(total))
  g["num_cells_host"] = torch.tensor(list(nc_host), dtype=torch.int32)
  if code != 0:
    err = _lib.TfgpcError(code, lib.tfgpc_last_error().decode())
    err.num_cells = list(nc_host)
    raise err
  c0, c1 = int(nc_host[0]), int(nc_host[1])
  g["ds"] = ds_flat[:b * c0 * c1 * 2].reshape(b, c0, c1, 2)
  # what the fill pass needs again (see find_neighbors_count)
  if samples_are_points == 1:
    smp, sb, order = points, bid, g["sorted_indices"]
  elif samples_are_points == 2:
    smp, sb, order = g["sorted_points"], g["sorted_batch_ids"], None
  else:
    smp, sb, order = samples, sbid, None
  keep = (smp, sb, g["sorted_points"], g["sorted_keys"], ds_flat, g["num_cells"],
          g["scaled_aabb_min"], g["inv_cell_sizes"], g["inv_radii"])
  head = (c_int(d), c_i64(ns), ptr(smp), ptr(sb))
  tail = (c_i64(n), ptr(g["sorted_points"]), ptr(g["sorted_keys"]), ptr(ds_flat), c_i64(b),
          ptr(g["num_cells"]), ptr(g["scaled_aabb_min"]), ptr(g["inv_cell_sizes"]),
          ptr(g["inv_radii"]), c_int(int(max_neighs)))
  g["count"] = NeighborCount(ranges, int(total.value), (head, tail, keep), order, d)
  return g


def original_neighbor_ids(neighbors, sorted_indices, pdf_by_original=None):
  """(sorted_indices[neighbors[:, 0]], neighbors[:, 1]) and, optionally, the
  density of every pair's neighbor point (tfgpc_original_neighbor_ids)."""
  neighbors, sorted_indices = _i32(neighbors), _i32(sorted_indices)
  _dev_check(neighbors, sorted_indices)
  m = neighbors.shape[0]
  ids = torch.empty((m, 2), dtype=torch.int32, device=neighbors.device)
  pdf = None
  if pdf_by_original is not None:
    pdf_by_original = _f32(pdf_by_original)
    pdf = torch.empty(m, dtype=torch.float32, device=neighbors.device)
  _lib.check(_lib.lib().tfgpc_original_neighbor_ids(
      _stream(), c_i64(m), ptr(neighbors), c_i64(sorted_indices.shape[0]), ptr(sorted_indices),
      ptr(pdf_by_original), ptr(ids), ptr(pdf)))
  return ids, pdf


def _pdf_args(points, neighbors, sample_neigh_indices, inv_bandwidth, inv_radii, mode):
  points = _f32(points)
  neighbors, ranges = _i32(neighbors), _i32(sample_neigh_indices)
  inv_bw, inv_r = _f32(inv_bandwidth), _f32(inv_radii)
  _dev_check(points, neighbors, ranges, inv_bw, inv_r)
  n, d = points.shape
  if ranges.shape[0] != n:
    raise _lib.TfgpcError(1, "ComputePDFOp expects the same number of points as samples")
  if neighbors.dim() != 2 or neighbors.shape[1] != 2:
    raise _lib.TfgpcError(1, "ComputePDFOp expects a neighbor tensor with 2 dimensions and 2 "
                          "indices per neighbor.")
  if inv_bw.shape[0] != d or inv_r.shape[0] != d:
    raise _lib.TfgpcError(1, "ComputePDFOp expects bandwidths and radii with the dimension of "
                          "the points")
  return points, neighbors, ranges, inv_bw, inv_r, n, d, int(mode)


def compute_pdf_with_pt_grads(points, neighbors, sample_neigh_indices, inv_bandwidth, inv_radii,
                              mode):
  """ComputePdfWithPtGrads (compute_pdf/cc/ops/compute_pdf_ops.cpp:43-56)."""
  points, neighbors, ranges, inv_bw, inv_r, n, d, mode = _pdf_args(
      points, neighbors, sample_neigh_indices, inv_bandwidth, inv_radii, mode)
  pdf = torch.empty(n, dtype=torch.float32, device=points.device)
  _lib.check(_lib.lib().tfgpc_compute_pdf(
      _stream(), c_int(d), c_int(mode), c_i64(n), ptr(points), ptr(neighbors),
      c_i64(neighbors.shape[0]), ptr(ranges), ptr(inv_bw), ptr(inv_r), ptr(pdf)))
  return pdf


compute_pdf = compute_pdf_with_pt_grads  # same kernel class (compute_pdf_ops.cpp:257-258)


def compute_pdf_at_samples(samples, points, neighbors, sample_neigh_indices, inv_bandwidth,
                           inv_radii, mode):
  """Density estimate centred on `samples` over their neighbor lists into
  `points` (tfgpc_compute_pdf_at_samples)."""
  samples = _f32(samples)
  points = _f32(points)
  neighbors, ranges = _i32(neighbors), _i32(sample_neigh_indices)
  inv_bw, inv_r = _f32(inv_bandwidth), _f32(inv_radii)
  _dev_check(samples, points, neighbors, ranges, inv_bw, inv_r)
  ns, d = samples.shape
  if ranges.shape[0] != ns:
    raise _lib.TfgpcError(1, "ComputePdfAtSamples expects one range per sample")
  pdf = torch.empty(ns, dtype=torch.float32, device=samples.device)
  _lib.check(_lib.lib().tfgpc_compute_pdf_at_samples(
      _stream(), c_int(d), c_int(int(mode)), c_i64(ns), ptr(samples), c_i64(points.shape[0]),
      ptr(points), ptr(neighbors), c_i64(neighbors.shape[0]), ptr(ranges), ptr(inv_bw),
      ptr(inv_r), ptr(pdf)))
  return pdf


def compute_pdf_pt_grads(points, neighbors, sample_neigh_indices, inv_bandwidth, inv_radii,
                         pdf_grads, mode):
  """ComputePdfPtGrads (compute_pdf/cc/ops/compute_pdf_ops.cpp:58-74)."""
  points, neighbors, ranges, inv_bw, inv_r, n, d, mode = _pdf_args(
      points, neighbors, sample_neigh_indices, inv_bandwidth, inv_radii, mode)
  pdf_grads = _f32(pdf_grads)
  if pdf_grads.shape[0] != n:
    raise _lib.TfgpcError(1, "ComputePDFPtGradsOp expects one pdf gradient per point")
  out = torch.empty((n, d), dtype=torch.float32, device=points.device)
  _lib.check(_lib.lib().tfgpc_compute_pdf_pt_grads(
      _stream(), c_int(d), c_int(mode), c_i64(n), ptr(points), ptr(neighbors),
      c_i64(neighbors.shape[0]), ptr(ranges), ptr(inv_bw), ptr(inv_r), ptr(pdf_grads), ptr(out)))
  return out


def _bp_args(basis, features, neighbors, ranges):
  basis, features = _f32(basis), _f32(features)
  neighbors, ranges = _i32(neighbors), _i32(ranges)
  _dev_check(basis, features, neighbors, ranges)
  if neighbors.dim() != 2 or neighbors.shape[1] != 2:
    raise _lib.TfgpcError(1, "BasisProjOp expects a neighbor tensor with 2 dimensions and 2 "
                          "indices per neighbor.")
  if basis.shape[0] != neighbors.shape[0]:
    raise _lib.TfgpcError(1, "BasisProjOp expects the same number of basis as the number of "
                          "neighbors.")
  return basis, features, neighbors, ranges


def read_device(values):
  """Blocking read of a small device tensor (at most 4096 bytes of int32,
  int64 or float32) into a CPU tensor, through mapped host memory instead of a
  copy engine: it does not wait behind bulk transfers on other streams."""
  v = values.contiguous()
  if not v.is_cuda:
    return v.clone()
  nbytes = v.numel() * v.element_size()
  if nbytes == 0 or nbytes > 4096 or nbytes % 4 != 0:
    return v.cpu()
  out = torch.empty(v.shape, dtype=v.dtype)
  _lib.check(_lib.lib().tfgpc_read_device(_stream(), ptr(v), c_sz(nbytes),
                                          ctypes.c_void_p(out.data_ptr())))
  return out


def _bp_scratch(k, c, feat):
  """Scratch of the tensor-core BasisProj kernels (None where the shape has none)."""
  nbytes = _lib.lib().tfgpc_basis_proj_workspace_bytes(c_int(k), c_int(c), c_i64(feat.shape[0]))
  if nbytes == 0:
    return None, 0
  return torch.empty(nbytes, dtype=torch.uint8, device=feat.device), nbytes


def basis_proj(basis_neighbors, pt_features, neighbors, sample_neigh_indices, scratch=True):
  """BasisProj (basis_proj/cc/ops/basis_proj_ops.cpp:25-39) -> [Ns, C, K].
  scratch=False keeps the call free of temporary device memory (fp32 kernels)."""
  basis, feat, neighbors, ranges = _bp_args(basis_neighbors, pt_features, neighbors,
                                            sample_neigh_indices)
  k, c, ns = basis.shape[1], feat.shape[1], ranges.shape[0]
  out = torch.empty((ns, c, k), dtype=torch.float32, device=basis.device)
  ws, ws_bytes = _bp_scratch(k, c, feat) if scratch else (None, 0)
  _lib.check(_lib.lib().tfgpc_basis_proj_ws(
      _stream(), c_int(k), c_int(c), c_i64(ns), c_i64(feat.shape[0]), c_i64(basis.shape[0]),
      ptr(basis), ptr(feat), ptr(neighbors), ptr(ranges), ptr(out), ptr(ws), c_sz(ws_bytes)))
  return out


def basis_proj_grads(basis_neighbors, pt_features, neighbors, sample_neigh_indices,
                     in_gradients, scratch=True):
  """BasisProjGrads (basis_proj/cc/ops/basis_proj_ops.cpp:41-53) ->
  (basis_gradients [M, K], feat_gradients [Nin, C])."""
  basis, feat, neighbors, ranges = _bp_args(basis_neighbors, pt_features, neighbors,
                                            sample_neigh_indices)
  grads = _f32(in_gradients)
  k, c, ns = basis.shape[1], feat.shape[1], ranges.shape[0]
  if tuple(grads.shape) != (ns, c, k):
    raise _lib.TfgpcError(1, "BasisProjGradsOp expects gradients of shape [Ns, C, K]")
  dbasis = torch.empty_like(basis)
  dfeat = torch.empty_like(feat)
  ws, ws_bytes = _bp_scratch(k, c, feat) if scratch else (None, 0)
  _lib.check(_lib.lib().tfgpc_basis_proj_grads_ws(
      _stream(), c_int(k), c_int(c), c_i64(ns), c_i64(feat.shape[0]), c_i64(basis.shape[0]),
      ptr(basis), ptr(feat), ptr(neighbors), ptr(ranges), ptr(grads), ptr(dbasis), ptr(dfeat),
      ptr(ws), c_sz(ws_bytes)))
  return dbasis, dfeat


def sampling(points, batch_ids, point_keys, num_cells, neighbors, sample_neigh_indices, mode,
             symmetric=False):
  """Sampling (sampling/cc/ops/sampling_ops.cpp:33-53).  mode 0 = Poisson disk,
  1 = cell average.  Returns (sample_pts [S, D], sample_batch_ids [S],
  sample_indices [S] or an unwritten [1] tensor for mode 1).  symmetric=True
  promises that point j is listed for point i exactly when i is listed for j
  (a self neighborhood found without a neighbor limit): same result, and the
  Poisson passes only walk the lists of the points they take."""
  points, batch_ids, nc = _f32(points), _i32(batch_ids), _i32(num_cells)
  keys = point_keys.contiguous()
  neighbors, ranges = _i32(neighbors), _i32(sample_neigh_indices)
  _dev_check(points, batch_ids, keys, nc, neighbors, ranges)
  n, d = points.shape
  if batch_ids.shape[0] != n or keys.shape[0] != n:
    raise _lib.TfgpcError(1, "SamplingOp expects the same number of keys as number of points.")
  if nc.shape[0] != d:
    raise _lib.TfgpcError(1, "SamplingOp expects a number of dimensions in inNumCells equal to "
                          "the number of dimensions in the input points")
  if neighbors.dim() != 2 or neighbors.shape[1] != 2:
    raise _lib.TfgpcError(1, "SamplingOp expects a neighbor tensor with 2 dimensions and 2 "
                          "indices per neighbor.")
  if ranges.shape[0] != n:
    raise _lib.TfgpcError(1, "SamplingOp expects the same number of points in inStartNeighIds "
                          "as in the points tensor.")
  dev = points.device
  nbytes = _lib.lib().tfgpc_sampling_workspace_bytes(c_i64(n))
  ws = _workspace(nbytes, dev)
  total = c_i64(0)
  common = (_stream(), c_int(d), c_int(int(mode)), c_i64(n), ptr(points), ptr(batch_ids),
            ptr(keys), ptr(nc))
  count = (_lib.lib().tfgpc_sampling_count_symmetric if symmetric
           else _lib.lib().tfgpc_sampling_count)
  _lib.check(count(
      *common, ptr(neighbors), c_i64(neighbors.shape[0]), ptr(ranges), ptr(ws), c_sz(nbytes),
      ctypes.byref(total)))
  s = int(total.value)
  out_pts = torch.empty((s, d), dtype=torch.float32, device=dev)
  out_bid = torch.empty(s, dtype=torch.int32, device=dev)
  out_idx = torch.empty(s if int(mode) == 0 else 1, dtype=torch.int32, device=dev)
  _lib.check(_lib.lib().tfgpc_sampling_store(
      *common, c_i64(s), ptr(ws), c_sz(nbytes), ptr(out_pts), ptr(out_bid), ptr(out_idx)))
  return out_pts, out_bid, out_idx
