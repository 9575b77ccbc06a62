"""Callers of the custom ops: torch mirrors of the reference's pylib classes.

  PointCloud / AABB   pylib/pc/PointCloud.py:23-134, 235-247
  Grid                pylib/pc/Grid.py:20-83
  Neighborhood        pylib/pc/Neighborhood.py:203-329
  sample              pylib/pc/sampling.py:23-28, 123-150
  PointHierarchy      pylib/pc/PointHierarchy.py:25-98

Only what feeds the ops is kept (segmented [N, D] input with batch ids); the
arithmetic around the ops is float32 torch code that follows the TensorFlow
expressions of the reference one to one, and the ops themselves run through
`custom_ops` (the C ABI).
"""
import math

import torch

from . import custom_ops as ops

SAMPLE_MODES = {'average': 1, 'cell average': 1, 'cell_average': 1,
                'poisson': 0, 'poisson disk': 0, 'poisson_disk': 0}


# Small per-dimension constants (radii, bandwidths) given as Python numbers are
# uploaded once per value and device: creating a device tensor from host data
# blocks the host until the stream has drained, once per call otherwise.  The
# cached tensors are never written to.
_DIMS_CACHE = {}


def _to_dims(value, dims, device):
  if not torch.is_tensor(value):
    flat = [float(v) for v in (value if hasattr(value, '__len__') else [value])]
    key = (tuple(flat), dims, str(device))
    t = _DIMS_CACHE.get(key)
    if t is None:
      if len(_DIMS_CACHE) > 256:
        _DIMS_CACHE.clear()
      t = torch.tensor(flat * dims if len(flat) == 1 else flat, dtype=torch.float32,
                       device=device)
      _DIMS_CACHE[key] = t
    return t
  t = torch.as_tensor(value, dtype=torch.float32, device=device).reshape(-1)
  if t.shape[0] == 1:
    t = t.repeat(dims)
  return t


class PointCloud:
  """Segmented point cloud: points [N, D] float32 and batch ids [N] int32."""

  def __init__(self, points, batch_ids, batch_size=None, num_cells_reduce=None):
    # num_cells_reduce: for a cloud that is one shard of a batch spread over
    # several ranks.  Grid.py:44-48 takes the cell counts as the maximum over the
    # WHOLE batch; the callable gets this shard's counts ([D] int32 on the device)
    # and returns the maximum over all shards (dist.allreduce_max_), so that every
    # rank builds the keys the unsharded batch would have.
    self._num_cells_reduce = num_cells_reduce
    self._points = torch.as_tensor(points).to(torch.float32).contiguous()
    self._batch_ids = torch.as_tensor(batch_ids, device=self._points.device).to(
        torch.int32).contiguous()
    if batch_size is None:
      batch_size = int(ops.read_device(self._batch_ids.max().reshape(1))[0]) + 1
    self._batch_size = int(batch_size)
    self._dimension = self._points.shape[1]
    self._aabb = None

  def get_AABB(self):
    """PointCloud.py:38-43: per-cloud min - 1e-9 and max + 1e-9 in float32."""
    if self._aabb is None:
      mn, mx = ops.compute_aabb(self._points, self._batch_ids, self._batch_size)
      self._aabb = (mn - 1e-9, mx + 1e-9)
    return self._aabb


class Grid:
  """Grid.py:32-83: keys, descending sort, sorted copies, lazy tube ranges."""

  def __init__(self, point_cloud, cell_sizes):
    pc = point_cloud
    dev = pc._points.device
    self._point_cloud = pc
    self._batch_size = pc._batch_size
    self._cell_sizes = _to_dims(cell_sizes, pc._dimension, dev)
    self._aabb_min, self._aabb_max = pc.get_AABB()
    sizes = self._aabb_max - self._aabb_min
    batch_num_cells = torch.ceil(sizes / self._cell_sizes).to(torch.int32)
    self._num_cells = torch.clamp(batch_num_cells.max(dim=0).values, min=1).to(torch.int32)
    if pc._num_cells_reduce is not None:
      self._num_cells = pc._num_cells_reduce(self._num_cells).to(torch.int32)
    self._num_cells_host = ops.read_device(self._num_cells)
    # custom_ops_wrapper.py:37-43
    self._scaled_aabb_min = self._aabb_min / self._cell_sizes
    self._inv_cell_sizes = torch.reciprocal(self._cell_sizes)
    self._cur_keys = ops.compute_keys(pc._points, pc._batch_ids, self._scaled_aabb_min,
                                      self._num_cells, self._inv_cell_sizes)
    total = self._batch_size
    for c in self._num_cells_host.tolist():
      total *= int(c)
    key_bits = max(1, int(math.ceil(math.log2(total + 1))))
    (self._sorted_indices, self._sorted_keys, self._sorted_points,
     self._sorted_batch_ids) = ops.sort_keys_desc(self._cur_keys, pc._points, pc._batch_ids,
                                                  key_bits=min(64, key_bits))
    self._fast_DS = None

  def get_DS(self):
    if self._fast_DS is None:
      self._fast_DS = ops.build_grid_ds(self._sorted_keys, self._num_cells,
                                        self._num_cells_host, self._batch_size)
    return self._fast_DS


class Neighborhood:
  """Neighborhood.py:218-329.  The count pass runs in the constructor (ranges and
  the number of pairs are known from then on); the neighbor list is written when
  it is first asked for, in one pass together with the list in original ids."""

  def __init__(self, grid, radius, point_cloud_sample=None, max_neighbors=0):
    dev = grid._sorted_points.device
    self._radii = _to_dims(radius, grid._point_cloud._dimension, dev)
    if point_cloud_sample is None:
      self._equal_samples = True
      self._point_cloud_sampled = PointCloud(grid._sorted_points, grid._sorted_batch_ids,
                                             grid._batch_size)
    else:
      self._equal_samples = False
      self._point_cloud_sampled = point_cloud_sample
    self._grid = grid
    self.max_neighbors = max_neighbors
    smp = self._point_cloud_sampled
    # samples that are the grid's own cloud in its unsorted order: the key sort's
    # permutation lists them cell by cell, the sequence the search is fastest in
    order = grid._sorted_indices if smp is grid._point_cloud else None
    # a sequence that visits the samples cell by cell, where one is known (the
    # samples of a self neighborhood are the sorted points: already in it)
    self._sample_order = order
    self._count = ops.find_neighbors_count(
        smp._points, smp._batch_ids, grid._sorted_points, grid._sorted_keys, grid.get_DS(),
        grid._num_cells, grid._scaled_aabb_min, grid._inv_cell_sizes,
        torch.reciprocal(self._radii), max_neighbors, sample_order=order)
    self._samples_neigh_ranges = self._count.ranges
    self._nbrs = None
    self._orig_ids = None
    self._pdf = None
    self._point_pdf = None
    self._sample_pdf = None
    self._pdf_ready = False
    self._transposed = None

  @property
  def num_pairs(self):
    return self._count.total

  def _fill(self):
    """Writes the neighbor list [M, 2] (index into the sorted points, sample
    index) and, in the same pass, the list with the neighbors' indices in the
    unsorted point order (Neighborhood.py:246-250)."""
    if self._nbrs is not None:
      return
    if self._equal_samples:
      # a self neighborhood mostly feeds the density estimate and the sampling,
      # which read sorted ids only: the original-id list is built if asked for
      self._nbrs = ops.find_neighbors_fill(self._count)
    else:
      self._nbrs, self._orig_ids = ops.find_neighbors_fill(self._count,
                                                            self._grid._sorted_indices)

  @property
  def _neighbors(self):
    self._fill()
    return self._nbrs

  @property
  def _original_neigh_ids(self):
    self._fill()
    if self._orig_ids is None:
      self._orig_ids, _ = ops.original_neighbor_ids(self._nbrs, self._grid._sorted_indices)
    return self._orig_ids

  def _samples_are_grid_points(self):
    return self._equal_samples or (self._point_cloud_sampled is self._grid._point_cloud
                                   and self.max_neighbors == 0)

  def compute_pdf(self, bandwidth=0.2, mode=0):
    """Neighborhood.py:257-311 (mode: 0 constant bandwidth, 1 by point count).
    The density is needed at every neighbor point.  pylib gets it from a second,
    self neighborhood of the grid (Neighborhood.py:284); when the samples are the
    grid's own cloud that second search is skipped: the density at sample s is
    the density of the point it coincides with."""
    d = self._point_cloud_sampled._dimension
    bw = _to_dims(bandwidth, d, self._radii.device)
    inv_bw, inv_r = torch.reciprocal(bw), torch.reciprocal(self._radii)
    g = self._grid
    self._pdf = None
    if self._equal_samples:
      self._point_pdf = ops.compute_pdf_with_pt_grads(
          g._sorted_points, self._neighbors, self._samples_neigh_ranges, inv_bw, inv_r, mode)
    elif self._samples_are_grid_points():
      # sample s is point s of the unsorted cloud
      self._sample_pdf = ops.compute_pdf_at_samples(
          self._point_cloud_sampled._points, g._sorted_points, self._neighbors,
          self._samples_neigh_ranges, inv_bw, inv_r, mode)
      self._point_pdf = None
    else:
      nb = Neighborhood(g, self._radii)
      self._point_pdf = ops.compute_pdf_with_pt_grads(
          g._sorted_points, nb._neighbors, nb._samples_neigh_ranges, inv_bw, inv_r, mode)
    self._pdf_ready = True

  def pdf_by_neighbor_id(self, **kwargs):
    """The densities as a table indexed by the FIRST column of _original_neigh_ids
    (one value per point of the grid's cloud), where the neighborhood has them in
    that form, else None: kernels that take the table read it in place of the
    per-pair array of get_pdf."""
    if not self._pdf_ready:
      self.compute_pdf(**kwargs)
    return self._sample_pdf

  def point_pdf(self, **kwargs):
    """Density of every point of the grid, in the SORTED order of the grid."""
    if not self._pdf_ready:
      self.compute_pdf(**kwargs)
    if self._point_pdf is None:
      self._point_pdf = self._sample_pdf[self._grid._sorted_indices.to(torch.int64)]
    return self._point_pdf

  def transpose(self):
    """Neighborhood.py:318-329: the neighborhood with the roles of samples and
    points exchanged (the samples' cloud on a grid of its own, searched around the
    points of this one); a self neighborhood is its own transpose."""
    if self._transposed is None:
      if self._equal_samples:
        self._transposed = self
      else:
        grid = Grid(self._point_cloud_sampled, self._radii)
        self._transposed = Neighborhood(grid, self._radii, self._grid._point_cloud)
    return self._transposed

  def get_pdf(self, **kwargs):
    """[M] density of every pair's neighbor point (Neighborhood.py:287)."""
    if not self._pdf_ready:
      self.compute_pdf(**kwargs)
    if self._pdf is None:
      if self._sample_pdf is not None:
        self._pdf = self._sample_pdf[self._original_neigh_ids[:, 0].to(torch.int64)]
      else:
        self._pdf = self._point_pdf[self._neighbors[:, 0].to(torch.int64)]
    return self._pdf

  def pdf_point_grads(self, pdf_grads, bandwidth=0.2, mode=0):
    """Gradient of a loss with respect to the grid's points [N, D] (in their
    original order) through the per-pair densities of get_pdf, given the loss's
    gradient pdf_grads [M] with respect to those densities.  The chain of the
    reference's autodiff: pdf[m] = point_pdf[neighbors[m, 0]] (Neighborhood.py:287),
    point_pdf = ComputePdfWithPtGrads(sorted points, self neighborhood), whose
    registered gradient is ComputePdfPtGrads (custom_ops_wrapper.py:159-169), and
    sorted points = gather(points, sorted indices) (Grid.py:60-62)."""
    g = self._grid
    d = g._point_cloud._dimension
    n = g._sorted_points.shape[0]
    per_point = torch.zeros(n, dtype=torch.float32, device=g._sorted_points.device)
    per_point.index_add_(0, self._neighbors[:, 0].to(torch.int64),
                         torch.as_tensor(pdf_grads, dtype=torch.float32))
    nb = self if self._equal_samples else Neighborhood(g, self._radii)
    bw = _to_dims(bandwidth, d, self._radii.device)
    grads_sorted = ops.compute_pdf_pt_grads(
        g._sorted_points, nb._neighbors, nb._samples_neigh_ranges, torch.reciprocal(bw),
        torch.reciprocal(self._radii), per_point, mode)
    out = torch.empty_like(grads_sorted)
    out[g._sorted_indices.to(torch.int64)] = grads_sorted
    return out


# Upper bound of cells per dimension that grid_neighborhood sizes its tube array
# and sort keys for, per (dimension, batch size): it starts at 64 and is raised
# to what a grid asked for when one did not fit.
_MAX_CELLS = {}
_ONE_CALL_CELLS_LIMIT = 1024


def grid_neighborhood(point_cloud, radius, point_cloud_sample=None, max_neighbors=0):
  """Grid(point_cloud, radius) and Neighborhood(grid, radius, point_cloud_sample,
  max_neighbors) built by ONE library call with ONE blocking read
  (tfgpc_grid_neighborhood_count) where pylib's two constructors read back twice
  (Grid.py:44-48 cell counts, Neighborhood.py:242-245 pair count).  Same objects,
  same contents.  For a cloud that is one shard of a distributed batch
  (num_cells_reduce set) the cell counts are reduced over the ranks on the device,
  between tfgpc_grid_cells and the main call: still one blocking read."""
  pc = point_cloud
  if pc._points.shape[0] == 0:
    return Neighborhood(Grid(pc, radius), radius, point_cloud_sample, max_neighbors)
  dev = pc._points.device
  d = pc._dimension
  radii = _to_dims(radius, d, dev)
  # (a radius given as a device tensor costs a read of its own)
  radii_host = (radius.detach().reshape(-1).cpu().tolist() if torch.is_tensor(radius) else
                [float(v) for v in (radius if hasattr(radius, '__len__') else [radius])])
  if len(radii_host) == 1:
    radii_host = radii_host * d
  if point_cloud_sample is None:
    mode, smp = 2, None
  elif point_cloud_sample is pc:
    mode, smp = 1, None
  else:
    mode, smp = 0, point_cloud_sample
  key = (d, pc._batch_size)
  max_cells = _MAX_CELLS.get(key, 64)
  cells = None
  if pc._num_cells_reduce is not None:
    # (the reduced counts are the same on every rank, so every rank takes the same
    # turns through the loop below; the reduction itself happens once)
    cells = ops.grid_cells(pc._points, pc._batch_ids, pc._batch_size, radii_host, radii_host)
    cells["num_cells"] = pc._num_cells_reduce(cells["num_cells"]).to(torch.int32)
  while True:
    try:
      g = ops.grid_neighborhood_count(
          pc._points, pc._batch_ids, pc._batch_size, radii_host, radii_host, max_cells,
          None if smp is None else smp._points, None if smp is None else smp._batch_ids,
          mode, max_neighbors, cells=cells)
      break
    except ops._lib.TfgpcError as err:
      asked = max(getattr(err, 'num_cells', [0]))
      if err.code != 3 or asked <= max_cells:
        raise
      bigger = 1 << (asked - 1).bit_length()
      if bigger > _ONE_CALL_CELLS_LIMIT or pc._batch_size * float(bigger) ** d >= 4e18:
        # a grid this fine would make the call's fixed-size tube array (or its sort
        # keys) too large: the separate constructors size both exactly
        return Neighborhood(Grid(pc, radius), radius, point_cloud_sample, max_neighbors)
      max_cells = bigger
      _MAX_CELLS[key] = max_cells
  grid = object.__new__(Grid)
  grid._point_cloud = pc
  grid._batch_size = pc._batch_size
  grid._cell_sizes = radii
  grid._aabb_min, grid._aabb_max = g["aabb_min"], g["aabb_max"]
  if pc._aabb is None:
    pc._aabb = (grid._aabb_min, grid._aabb_max)
  grid._num_cells = g["num_cells"]
  grid._num_cells_host = g["num_cells_host"]
  grid._scaled_aabb_min = g["scaled_aabb_min"]
  grid._inv_cell_sizes = g["inv_cell_sizes"]
  grid._cur_keys = g["keys"]
  grid._sorted_indices, grid._sorted_keys = g["sorted_indices"], g["sorted_keys"]
  grid._sorted_points, grid._sorted_batch_ids = g["sorted_points"], g["sorted_batch_ids"]
  grid._fast_DS = g["ds"]
  nb = object.__new__(Neighborhood)
  nb._radii = radii
  nb._equal_samples = point_cloud_sample is None
  nb._point_cloud_sampled = (PointCloud(grid._sorted_points, grid._sorted_batch_ids,
                                        grid._batch_size)
                             if point_cloud_sample is None else point_cloud_sample)
  nb._grid = grid
  nb.max_neighbors = max_neighbors
  nb._sample_order = grid._sorted_indices if mode == 1 else None
  nb._count = g["count"]
  nb._samples_neigh_ranges = nb._count.ranges
  nb._nbrs = nb._orig_ids = nb._pdf = nb._point_pdf = nb._sample_pdf = None
  nb._pdf_ready = False
  nb._transposed = None
  return nb


def sample(neighborhood, sample_mode='poisson'):
  """sampling.py:123-150 -> (PointCloud of the samples, original indices or None)."""
  mode = SAMPLE_MODES[sample_mode.lower()]
  g = neighborhood._grid
  pts, bids, idx = ops.sampling(g._sorted_points, g._sorted_batch_ids, g._sorted_keys,
                                g._num_cells, neighborhood._neighbors,
                                neighborhood._samples_neigh_ranges, mode,
                                symmetric=(neighborhood._equal_samples
                                           and neighborhood.max_neighbors == 0))
  if mode == 0:
    idx = g._sorted_indices[idx.to(torch.int64)]
  else:
    idx = None
  return PointCloud(pts, bids, g._batch_size), idx


class PointHierarchy:
  """PointHierarchy.py:40-98: per level Grid -> self Neighborhood -> sample."""

  def __init__(self, point_cloud, cell_sizes, sample_mode='poisson'):
    self._point_clouds = [point_cloud]
    self._neighborhoods = []
    self._sample_indices = []
    cur = point_cloud
    for cs in cell_sizes:
      neigh = grid_neighborhood(cur, cs)
      cur, idx = sample(neigh, sample_mode)
      self._neighborhoods.append(neigh)
      self._point_clouds.append(cur)
      self._sample_indices.append(idx)
