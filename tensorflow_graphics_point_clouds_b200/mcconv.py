"""Monte-Carlo convolution on the fused C-ABI entry points.

Mirrors `MCConv` of the reference (pylib/pc/layers/MCConv.py:36-278): the
kernel MLP on the relative neighbor positions gives the per-neighbor basis
(divided by the density estimate), the basis projection aggregates it with the
input features, and the final weights map [C_in * K] to C_out.  The projection
and the final matrix product run as one C-ABI call (tfgpc_mcconv_forward) and
their gradients as another (tfgpc_mcconv_backward); the small kernel MLP
([M, D] x [D, K]) stays in torch, like it stays in TensorFlow in the reference.
"""
import ctypes

import torch

from . import _lib
from ._lib import c_i64, c_int, c_sz, ptr
from .custom_ops import _stream, _f32, _i32, _workspace


def matmul_f32(a, b, a_transposed=False, b_transposed=False):
  """c = op(a) @ op(b) in fp32 accuracy on the tensor cores (tfgpc_matmul_f32)."""
  a, b = _f32(a), _f32(b)
  m, k = (a.shape[1], a.shape[0]) if a_transposed else a.shape
  n = b.shape[0] if b_transposed else b.shape[1]
  kb = b.shape[1] if b_transposed else b.shape[0]
  if kb != k:
    raise _lib.TfgpcError(1, "matmul expects matching inner dimensions")
  c = torch.empty((m, n), dtype=torch.float32, device=a.device)
  nbytes = _lib.lib().tfgpc_matmul_workspace_bytes(c_i64(m), c_i64(n), c_i64(k))
  ws = _workspace(nbytes, a.device)
  _lib.check(_lib.lib().tfgpc_matmul_f32(
      _stream(), c_i64(m), c_i64(n), c_i64(k), ptr(a), c_int(int(a_transposed)), ptr(b),
      c_int(int(b_transposed)), ptr(c), ptr(ws), c_sz(nbytes)))
  status = c_int(0)
  _lib.check(_lib.lib().tfgpc_mcconv_status(_stream(), ptr(ws), ctypes.byref(status)))
  return c


class ProjectionGemm:
  """Holds the workspace of one (K, C, Cout, Ns) problem and runs the fused
  forward / backward entry points on it.  The workspace also depends on the
  number of input points; it is allocated on first use (or up front when
  `n_in` is given) and grown if a later call brings more points."""

  def __init__(self, k, c, cout, ns, device, backward=True, n_in=None):
    self.k, self.c, self.cout, self.ns = int(k), int(c), int(cout), int(ns)
    self.backward_ws = bool(backward)
    self.device = device
    self.n_in, self.nbytes, self.ws = -1, 0, None
    self._x_valid = False
    if n_in is not None:
      self._ensure_workspace(int(n_in))

  def _ensure_workspace(self, n_in):
    if self.ws is not None and n_in <= self.n_in:
      return
    self.n_in = n_in
    self.nbytes = _lib.lib().tfgpc_mcconv_workspace_bytes(
        c_int(self.k), c_int(self.c), c_int(self.cout), c_i64(self.ns), c_i64(n_in),
        c_int(int(self.backward_ws)))
    self.ws = _workspace(self.nbytes, self.device)
    self._x_valid = False

  def forward(self, basis, features, neighbors, ranges, weights):
    basis, features, weights = _f32(basis), _f32(features), _f32(weights)
    neighbors, ranges = _i32(neighbors), _i32(ranges)
    out = torch.empty((self.ns, self.cout), dtype=torch.float32, device=basis.device)
    self._ensure_workspace(features.shape[0])
    _lib.check(_lib.lib().tfgpc_mcconv_forward(
        _stream(), c_int(self.k), c_int(self.c), c_int(self.cout), c_i64(self.ns),
        c_i64(features.shape[0]), c_i64(basis.shape[0]), ptr(basis), ptr(features),
        ptr(neighbors), ptr(ranges), ptr(weights), ptr(out), ptr(self.ws), c_sz(self.nbytes)))
    self._x_valid = self.backward_ws
    self._x_grouped = False
    return out

  def backward(self, basis, features, neighbors, ranges, weights, out_grads, reuse_forward=True):
    if not self.backward_ws:
      raise RuntimeError("this ProjectionGemm was created without backward workspace")
    basis, features, weights = _f32(basis), _f32(features), _f32(weights)
    neighbors, ranges, out_grads = _i32(neighbors), _i32(ranges), _f32(out_grads)
    dbasis = torch.empty_like(basis)
    dfeat = torch.empty_like(features)
    dw = torch.empty_like(weights)
    self._ensure_workspace(features.shape[0])
    _lib.check(_lib.lib().tfgpc_mcconv_backward(
        _stream(), c_int(self.k), c_int(self.c), c_int(self.cout), c_i64(self.ns),
        c_i64(features.shape[0]), c_i64(basis.shape[0]), ptr(basis), ptr(features),
        ptr(neighbors), ptr(ranges), ptr(weights), ptr(out_grads),
        c_int(int(reuse_forward and self._x_valid and not getattr(self, '_x_grouped', False))),
        ptr(dbasis), ptr(dfeat), ptr(dw), ptr(self.ws), c_sz(self.nbytes)))
    return dbasis, dfeat, dw

  def forward_grouped(self, basis_pair, features, weights, order, plan):
    """The forward pass through tfgpc_mcconv_forward_grouped: the projection runs
    once per distinct neighbor of a group of four samples (taken in `order`)
    instead of once per pair; basis_pair [M, 2, K] bf16."""
    features, weights = _f32(features), _f32(weights)
    out = torch.empty((self.ns, self.cout), dtype=torch.float32, device=features.device)
    self._ensure_workspace(features.shape[0])
    _lib.check(_lib.lib().tfgpc_mcconv_forward_grouped(
        _stream(), c_int(self.k), c_int(self.c), c_int(self.cout), c_i64(self.ns),
        c_i64(features.shape[0]), c_i64(basis_pair.shape[0]), ptr(basis_pair), ptr(features),
        ptr(weights), ptr(_i32(order)), ptr(plan), ptr(out), ptr(self.ws), c_sz(self.nbytes)))
    self._x_valid = self.backward_ws
    self._x_grouped = True
    return out

  def backward_grouped(self, basis_pair, features, ranges, weights, out_grads, order, plan,
                       reuse_forward=True):
    """The gradients through tfgpc_mcconv_backward_grouped (dbasis [M, K] fp32,
    dfeat, dweights)."""
    features, weights = _f32(features), _f32(weights)
    ranges, out_grads = _i32(ranges), _f32(out_grads)
    m, k = basis_pair.shape[0], basis_pair.shape[2]
    dbasis = torch.empty((m, k), dtype=torch.float32, device=features.device)
    dfeat = torch.empty_like(features)
    dw = torch.empty_like(weights)
    self._ensure_workspace(features.shape[0])
    reuse = reuse_forward and self._x_valid and getattr(self, '_x_grouped', False)
    _lib.check(_lib.lib().tfgpc_mcconv_backward_grouped(
        _stream(), c_int(self.k), c_int(self.c), c_int(self.cout), c_i64(self.ns),
        c_i64(features.shape[0]), c_i64(m), ptr(basis_pair), ptr(features), ptr(ranges),
        ptr(weights), ptr(out_grads), c_int(int(reuse)), ptr(_i32(order)), ptr(plan), ptr(dbasis),
        ptr(dfeat), ptr(dw), ptr(self.ws), c_sz(self.nbytes)))
    return dbasis, dfeat, dw

  def check_status(self):
    """Blocks on the stream; raises TfgpcError(4) if a GEMM wait timed out."""
    status = c_int(0)
    _lib.check(_lib.lib().tfgpc_mcconv_status(_stream(), ptr(self.ws), ctypes.byref(status)))


def dense_final_weights(wf, cin, hidden):
  """MCConv stores its final weights per kernel MLP, [G, cin*hidden, cout/G]
  (MCConv.py:123-135), and multiplies the projection's columns (c, g*hidden+h)
  with row c*hidden+h of block g (MCConv.py:174-191).  This returns the same
  linear map as one [cin*G*hidden, cout] matrix in the projection's own column
  order c*K + k (zero where a column belongs to another MLP's outputs)."""
  g, _, co = wf.shape
  k = g * hidden
  dense = torch.zeros((cin, k, g * co), dtype=wf.dtype, device=wf.device)
  w4 = wf.reshape(g, cin, hidden, co)
  for i in range(g):
    dense[:, i * hidden:(i + 1) * hidden, i * co:(i + 1) * co] = w4[i]
  return dense.reshape(cin * k, g * co)


def blocks_of_dense_grad(dw_dense, num_mlps, cin, hidden):
  """Inverse of dense_final_weights for gradients: [cin*K, cout] -> [G, cin*hidden, cout/G]."""
  k = num_mlps * hidden
  co = dw_dense.shape[1] // num_mlps
  d3 = dw_dense.reshape(cin, k, num_mlps * co)
  out = [d3[:, i * hidden:(i + 1) * hidden, i * co:(i + 1) * co].reshape(cin * hidden, co)
         for i in range(num_mlps)]
  return torch.stack(out, dim=0)


def pack_points_density(points, pdf):
  """[n, 4] table (x, y, z, 1 / density) of a 3-D cloud and its per-point
  densities (tfgpc_pack_points_density): points_in of the kernel-basis entries
  with pdf_by_neighbor=2."""
  points, pdf = _f32(points), _f32(pdf).reshape(-1)
  n = points.shape[0]
  if points.shape[1] != 3 or pdf.shape[0] != n:
    raise _lib.TfgpcError(1, "PackPointsDensity expects [n, 3] points and [n] densities")
  out = torch.empty((n, 4), dtype=torch.float32, device=points.device)
  _lib.check(_lib.lib().tfgpc_pack_points_density(_stream(), c_i64(n), ptr(points), ptr(pdf),
                                                  ptr(out)))
  return out


def kernel_basis(points_in, points_out, neighbors, pdf, w1, b1, radius, activation=0,
                 alpha=0.2, pdf_by_neighbor=False):
  """basis[m, k] = act(diff_m . w1[:, k] + b1[k]) / pdf[m] (tfgpc_kernel_basis).
  w1 [D, K], b1 [K]; neighbors hold (index into points_in, index into points_out).
  pdf_by_neighbor: pdf is a table with one density per point of points_in, read
  at the pair's neighbor index, instead of the per-pair array."""
  points_in, points_out = _f32(points_in), _f32(points_out)
  pdf = None if pdf is None else _f32(pdf)
  w1, b1, neighbors = _f32(w1), _f32(b1).reshape(-1), _i32(neighbors)
  d, k = w1.shape
  m = neighbors.shape[0]
  basis = torch.empty((m, k), dtype=torch.float32, device=points_in.device)
  _lib.check(_lib.lib().tfgpc_kernel_basis(
      _stream(), c_int(d), c_int(k), c_i64(m), ptr(points_in), ptr(points_out), ptr(neighbors),
      ptr(pdf), ptr(w1), ptr(b1), ctypes.c_float(1.0 / float(radius)), c_int(activation),
      ctypes.c_float(alpha), c_int(int(pdf_by_neighbor)), ptr(basis)))
  return basis


def kernel_basis_split(points_in, points_out, neighbors, pdf, w1, b1, radius, activation=0,
                       alpha=0.2, want_fp32=True, pdf_by_neighbor=False):
  """kernel_basis that returns every row as the bf16 (hi, mid) pair the
  tensor-core kernels multiply with: (basis [M, K] float32 or None, pair
  [M, 2, K] bf16)."""
  points_in, points_out = _f32(points_in), _f32(points_out)
  pdf = None if pdf is None else _f32(pdf)
  w1, b1, neighbors = _f32(w1), _f32(b1).reshape(-1), _i32(neighbors)
  d, k = w1.shape
  m = neighbors.shape[0]
  basis = (torch.empty((m, k), dtype=torch.float32, device=points_in.device) if want_fp32
           else None)
  pair = torch.empty((m, 2, k), dtype=torch.bfloat16, device=points_in.device)
  _lib.check(_lib.lib().tfgpc_kernel_basis_split(
      _stream(), c_int(d), c_int(k), c_i64(m), ptr(points_in), ptr(points_out), ptr(neighbors),
      ptr(pdf), ptr(w1), ptr(b1), ctypes.c_float(1.0 / float(radius)), c_int(activation),
      ctypes.c_float(alpha), c_int(int(pdf_by_neighbor)), ptr(basis), ptr(pair)))
  return basis, pair


def group_plan(neighborhood, order=None):
  """Row plan of the grouped kernels for a neighborhood (tfgpc_mcconv_group_plan):
  the samples four at a time in `order` (default: the neighborhood's own visiting
  order, else the sample order), every group's distinct neighbors and the pairs
  that reach them.  Returns (order [ns] int32, plan buffer)."""
  ranges = _i32(neighborhood._samples_neigh_ranges)
  ns, m = ranges.shape[0], neighborhood._neighbors.shape[0]
  if order is None:
    order = getattr(neighborhood, '_sample_order', None)
  if order is None:
    order = torch.arange(ns, dtype=torch.int32, device=ranges.device)
  order = _i32(order)
  nbytes = _lib.lib().tfgpc_mcconv_group_plan_bytes(c_i64(ns), c_i64(m))
  plan = _workspace(nbytes, ranges.device)
  _lib.check(_lib.lib().tfgpc_mcconv_group_plan(
      _stream(), c_i64(ns), c_i64(m), ptr(order), ptr(ranges), ptr(_i32(neighborhood._neighbors)),
      ptr(_i32(neighborhood._original_neigh_ids)), ptr(plan), c_sz(nbytes)))
  return order, plan


def _mlp_blocks(weights, biases):
  """Per-layer tensors [G, H_{l-1}, H_l] / [G, 1, H_l] -> (flat weights, flat
  biases, layer sizes as a host int32 array, D, G)."""
  weights = [_f32(w) for w in weights]
  biases = [_f32(b) for b in biases]
  g, d, _ = weights[0].shape
  sizes = (ctypes.c_int32 * len(weights))(*[int(w.shape[2]) for w in weights])
  flat_w = torch.cat([w.reshape(-1) for w in weights]).contiguous()
  flat_b = torch.cat([b.reshape(-1) for b in biases]).contiguous()
  return flat_w, flat_b, sizes, int(d), int(g)


def kernel_mlp_basis(points_in, points_out, neighbors, pdf, weights, biases, radius,
                     activation=0, alpha=0.2, pdf_by_neighbor=False):
  """The kernel MLP with any number of hidden layers (tfgpc_kernel_mlp_basis):
  weights[l] [G, H_{l-1}, H_l], biases[l] [G, 1, H_l] -> basis [M, G * H_last]."""
  points_in, points_out, pdf, neighbors = _f32(points_in), _f32(points_out), _f32(pdf), _i32(neighbors)
  flat_w, flat_b, sizes, d, g = _mlp_blocks(weights, biases)
  m = neighbors.shape[0]
  basis = torch.empty((m, g * int(sizes[len(sizes) - 1])), dtype=torch.float32,
                      device=points_in.device)
  _lib.check(_lib.lib().tfgpc_kernel_mlp_basis(
      _stream(), c_int(d), c_int(g), c_int(len(sizes)), sizes, c_i64(m), ptr(points_in),
      ptr(points_out), ptr(neighbors), ptr(pdf), ptr(flat_w), ptr(flat_b),
      ctypes.c_float(1.0 / float(radius)), c_int(activation), ctypes.c_float(alpha),
      c_int(int(pdf_by_neighbor)), ptr(basis)))
  return basis


def kernel_mlp_grads(points_in, points_out, neighbors, pdf, weights, biases, radius, basis_grads,
                     activation=0, alpha=0.2, point_grads=False, pdf_by_neighbor=False):
  """All gradients of kernel_mlp_basis (tfgpc_kernel_mlp_grads): ([d_weights],
  [d_biases]) in the layouts of the inputs and, with point_grads, also
  (d_points_in, d_points_out, d_pdf [M]); when points_in and points_out are the
  same tensor, d_points_in and d_points_out are one tensor holding the sum."""
  points_in, points_out, pdf, neighbors = _f32(points_in), _f32(points_out), _f32(pdf), _i32(neighbors)
  basis_grads = _f32(basis_grads)
  flat_w, flat_b, sizes, d, g = _mlp_blocks(weights, biases)
  dw, db = torch.empty_like(flat_w), torch.empty_like(flat_b)
  dpin = dpout = dpdf = None
  if point_grads:
    dpin = torch.empty_like(points_in)
    dpout = dpin if points_out.data_ptr() == points_in.data_ptr() else torch.empty_like(points_out)
    dpdf = torch.empty(neighbors.shape[0], dtype=torch.float32, device=pdf.device)
  _lib.check(_lib.lib().tfgpc_kernel_mlp_grads(
      _stream(), c_int(d), c_int(g), c_int(len(sizes)), sizes, c_i64(neighbors.shape[0]),
      c_i64(points_in.shape[0]), c_i64(points_out.shape[0]), ptr(points_in), ptr(points_out),
      ptr(neighbors), ptr(pdf), ptr(flat_w), ptr(flat_b), ctypes.c_float(1.0 / float(radius)),
      c_int(activation), ctypes.c_float(alpha), c_int(int(pdf_by_neighbor)), ptr(basis_grads),
      ptr(dw), ptr(db), ptr(dpin), ptr(dpout), ptr(dpdf)))
  d_weights, d_biases, ow, ob = [], [], 0, 0
  for w, b in zip(weights, biases):
    d_weights.append(dw[ow:ow + w.numel()].reshape(w.shape)); ow += w.numel()
    d_biases.append(db[ob:ob + b.numel()].reshape(b.shape)); ob += b.numel()
  if point_grads:
    return d_weights, d_biases, dpin, dpout, dpdf
  return d_weights, d_biases


def kernel_basis_grads(points_in, points_out, neighbors, pdf, w1, b1, radius, basis_grads,
                       activation=0, alpha=0.2, pdf_by_neighbor=False):
  """Gradients of kernel_basis with respect to w1 and b1 (tfgpc_kernel_basis_grads)."""
  points_in, points_out = _f32(points_in), _f32(points_out)
  pdf = None if pdf is None else _f32(pdf)
  w1, b1, neighbors = _f32(w1), _f32(b1).reshape(-1), _i32(neighbors)
  basis_grads = _f32(basis_grads)
  d, k = w1.shape
  dw1 = torch.empty_like(w1)
  db1 = torch.empty_like(b1)
  _lib.check(_lib.lib().tfgpc_kernel_basis_grads(
      _stream(), c_int(d), c_int(k), c_i64(neighbors.shape[0]), ptr(points_in), ptr(points_out),
      ptr(neighbors), ptr(pdf), ptr(w1), ptr(b1), ctypes.c_float(1.0 / float(radius)),
      c_int(activation), ctypes.c_float(alpha), c_int(int(pdf_by_neighbor)), ptr(basis_grads),
      ptr(dw1), ptr(db1)))
  return dw1, db1


# MCConv.py:27-31 / PointConv.py:27-31: name -> (activation code, slope) of the kernel-basis entries
NON_LINEARITIES = {'relu': (0, 0.0), 'lrelu': (0, 0.2), 'leakyrelu': (0, 0.2),
                   'leaky_relu': (0, 0.2), 'elu': (1, 0.0)}


class MCConv:
  """Monte-Carlo convolution layer (MCConv.py:36-278) with explicit backward.

  Weights use the reference's layouts: w1 [G, D, H], b1 [G, 1, H] for a kernel
  MLP with one hidden layer, or lists of per-layer tensors ([G, H_{l-1}, H_l],
  [G, 1, H_l]) for deeper ones (MCConv.py:92-135, 165-168); wf
  [G, C_in*H_last, C_out/G].  non_linearity_type as in MCConv.py:27-31
  ('relu', 'leaky_relu', 'elu')."""

  def __init__(self, w1, b1, wf, num_features_in, grouped=True, non_linearity_type='leaky_relu'):
    multi = isinstance(w1, (list, tuple))
    self.kernel_weights = [_f32(w) for w in (w1 if multi else [w1])]
    self.kernel_biases = [_f32(b) for b in (b1 if multi else [b1])]
    self._list_form = multi
    self.wf = _f32(wf)
    self.w1, self.b1 = self.kernel_weights[0], self.kernel_biases[0]
    self.grouped = bool(grouped)
    self._grouped = None
    self.num_mlps, self.dims, _ = self.kernel_weights[0].shape
    self.hidden = int(self.kernel_weights[-1].shape[2])
    self.activation, self.alpha = NON_LINEARITIES[non_linearity_type.lower()]
    self.cin = int(num_features_in)
    self.cout = self.wf.shape[2] * self.num_mlps
    self.k = self.num_mlps * self.hidden
    self._op = None
    self._saved = None

  def _dense_weights(self):
    if self.num_mlps == 1:
      return self.wf[0]
    return dense_final_weights(self.wf, self.cin, self.hidden)

  def _flat_kernel_weights(self):
    # [G, D, H] -> [D, G*H]: column k = g*H + h (MCConv.py:169-171)
    return (self.w1.permute(1, 0, 2).reshape(self.dims, self.k).contiguous(),
            self.b1.reshape(self.k).contiguous())

  def build_neighborhood(self, point_cloud_in, point_cloud_out, radius):
    """MCConv.py:254-261: grid of the input cloud, neighborhood around the
    output points."""
    from . import pc
    return pc.grid_neighborhood(point_cloud_in, radius, point_cloud_out)

  def forward(self, features, point_cloud_in, point_cloud_out, radius, neighborhood=None,
              bandwidth=0.2, keep_for_backward=True):
    neigh = neighborhood or self.build_neighborhood(point_cloud_in, point_cloud_out, radius)
    # the densities as a per-point table where the neighborhood has them so (it
    # then never forms the per-pair array), else per pair
    pdf = neigh.pdf_by_neighbor_id(bandwidth=bandwidth, mode=0)
    by_nbr = pdf is not None
    if not by_nbr:
      pdf = neigh.get_pdf(bandwidth=bandwidth, mode=0)
    ns = point_cloud_out._points.shape[0]
    p_in, p_out, ids = point_cloud_in._points, point_cloud_out._points, neigh._original_neigh_ids
    one_layer = len(self.kernel_weights) == 1
    w1, b1 = self._flat_kernel_weights() if one_layer else (None, None)
    # wide layers run on a group plan (see group_plan)
    grouped = (one_layer and self.grouped and neigh._neighbors.shape[0] > 0 and
               self.cout >= 128 and
               _lib.lib().tfgpc_mcconv_grouped_supported(c_int(self.k), c_int(self.cin)) != 0)
    # (points, 1 / density) as one 16-byte row per point: one gather per pair
    kb_in, kb_pdf, kb_mode = p_in, pdf, int(by_nbr)
    if one_layer and by_nbr and self.dims == 3:
      kb_in, kb_pdf, kb_mode = pack_points_density(p_in, pdf), None, 2
    if grouped:
      # the basis only as the bf16 pair the tensor-core kernels read
      basis, pair = kernel_basis_split(kb_in, p_out, ids, kb_pdf, w1, b1, radius, self.activation,
                                       self.alpha, want_fp32=False, pdf_by_neighbor=kb_mode)
      self._grouped = (pair,) + group_plan(neigh)
    elif one_layer:
      basis = kernel_basis(kb_in, p_out, ids, kb_pdf, w1, b1, radius, self.activation, self.alpha,
                           pdf_by_neighbor=kb_mode)
      self._grouped = None
    else:
      basis = kernel_mlp_basis(p_in, p_out, ids, pdf, self.kernel_weights, self.kernel_biases,
                               radius, self.activation, self.alpha, pdf_by_neighbor=by_nbr)
      self._grouped = None
    if (self._op is None or self._op.ns != ns or self._op.backward_ws != keep_for_backward):
      self._op = ProjectionGemm(self.k, self.cin, self.cout, ns, features.device,
                                backward=keep_for_backward)
    wd = self._dense_weights()
    if grouped:
      out = self._op.forward_grouped(self._grouped[0], features, wd, self._grouped[1],
                                     self._grouped[2])
    else:
      out = self._op.forward(basis, features, ids, neigh._samples_neigh_ranges, wd)
    if keep_for_backward:
      self._saved = (neigh, point_cloud_in, point_cloud_out, radius, pdf, basis,
                     _f32(features), wd, w1, b1)
      self._pdf_by_nbr = by_nbr
      self._kb_inputs = (kb_in, kb_pdf, kb_mode)
    return out

  def saved_basis(self):
    """The kernel basis [M, K] of the last forward call as float32 (on the grouped
    path it is kept as a bf16 pair: the sum of the two terms is returned)."""
    basis = self._saved[5]
    if basis is None:
      pair = self._grouped[0]
      basis = pair[:, 0, :].float() + pair[:, 1, :].float()
    return basis

  def backward(self, out_grads, point_grads=False):
    """Gradients of the last forward call: (d_features, d_w1, d_b1, d_wf) in the
    layouts of the weights (d_w1 / d_b1 are lists if the layer was built from
    lists).  With point_grads=True three more values follow: d_points_in,
    d_points_out (the gradients through the kernel inputs, MCConv.py:264-269;
    one tensor holding the sum of both if the two clouds share their point
    tensor) and d_pdf [M], the gradient with respect to the per-pair densities,
    which Neighborhood.pdf_point_grads carries on to the points."""
    neigh, pc_in, pc_out, radius, pdf, basis, features, wd, w1, b1 = self._saved
    ids = neigh._original_neigh_ids
    if self._grouped is not None:
      pair, order, plan = self._grouped
      dbasis, dfeat, dwd = self._op.backward_grouped(
          pair, features, neigh._samples_neigh_ranges, wd, out_grads, order, plan)
    else:
      dbasis, dfeat, dwd = self._op.backward(basis, features, ids, neigh._samples_neigh_ranges,
                                             wd, out_grads)
    dwf = (dwd.unsqueeze(0) if self.num_mlps == 1
           else blocks_of_dense_grad(dwd, self.num_mlps, self.cin, self.hidden))
    if point_grads or len(self.kernel_weights) > 1:
      res = kernel_mlp_grads(pc_in._points, pc_out._points, ids, pdf, self.kernel_weights,
                             self.kernel_biases, radius, dbasis, self.activation, self.alpha,
                             point_grads=point_grads, pdf_by_neighbor=self._pdf_by_nbr)
      dws, dbs = res[0], res[1]
      head = (dfeat, dws if self._list_form else dws[0], dbs if self._list_form else dbs[0], dwf)
      return head + tuple(res[2:]) if point_grads else head
    kb_in, kb_pdf, kb_mode = self._kb_inputs
    dw1, db1 = kernel_basis_grads(kb_in, pc_out._points, ids, kb_pdf, w1, b1, radius, dbasis,
                                  self.activation, self.alpha, pdf_by_neighbor=kb_mode)
    dw1 = dw1.reshape(self.dims, self.num_mlps, self.hidden).permute(1, 0, 2).contiguous()
    db1 = db1.reshape(self.num_mlps, 1, self.hidden)
    if self._list_form:
      return dfeat, [dw1], [db1], dwf
    return dfeat, dw1, db1, dwf


# ---- KPConv and PointConv: other bases on the same projection + weight product

def _basis_count(k):
  """Smallest basis count the projection accepts that holds k functions
  (the padding rule of KPConv.py:199-212)."""
  for cand in (8, 16, 32, 64):
    if k <= cand:
      return cand
  raise _lib.TfgpcError(1, "at most 64 basis functions are supported")


def _pad_weights(w, cin, k, k_pad, cout_pad):
  """[cin*k, cout] -> [cin*k_pad, cout_pad] with zero rows for the padding
  basis functions and zero columns up to a multiple of 8."""
  cout = w.shape[1]
  wp = torch.zeros((cin, k_pad, cout_pad), dtype=torch.float32, device=w.device)
  wp[:, :k, :cout] = w.reshape(cin, k, cout)
  return wp.reshape(cin * k_pad, cout_pad)


def kp_basis(points_in, points_out, neighbors, kernel_points, radius, sigma, k_pad,
             interpolation='linear'):
  """basis[m, k] = weighting(|diff_m - kernel_points[k]|, sigma), zero for the
  padding columns (tfgpc_kp_basis; KPConv.py:194-212)."""
  points_in, points_out = _f32(points_in), _f32(points_out)
  kernel_points, neighbors = _f32(kernel_points), _i32(neighbors)
  num_kp, d = kernel_points.shape
  m = neighbors.shape[0]
  basis = torch.empty((m, k_pad), dtype=torch.float32, device=points_in.device)
  _lib.check(_lib.lib().tfgpc_kp_basis(
      _stream(), c_int(d), c_int(k_pad), c_int(num_kp), c_i64(m), ptr(points_in),
      ptr(points_out), ptr(neighbors), ptr(kernel_points), ctypes.c_float(1.0 / float(radius)),
      ctypes.c_float(float(sigma)), c_int({'linear': 0, 'gaussian': 1}[interpolation]),
      ptr(basis)))
  return basis


def pointconv_pdf(pdf, ranges, w1, b1, w2, b2):
  """Per pair relu(pdf / max over the sample * w1 + b1) . w2 + b2
  (tfgpc_pointconv_pdf; PointConv.py:168-183)."""
  pdf, ranges = _f32(pdf), _i32(ranges)
  w1, b1 = _f32(w1).reshape(-1), _f32(b1).reshape(-1)
  w2, b2 = _f32(w2).reshape(-1), _f32(b2).reshape(-1)
  if w1.numel() != 16 or b1.numel() != 16 or w2.numel() != 16 or b2.numel() != 1:
    raise _lib.TfgpcError(1, "PointConv's density transform has 16 hidden units")
  out = torch.empty_like(pdf)
  _lib.check(_lib.lib().tfgpc_pointconv_pdf(
      _stream(), c_i64(ranges.shape[0]), c_i64(pdf.shape[0]), ptr(ranges), ptr(pdf), ptr(w1),
      ptr(b1), ptr(w2), ptr(b2), ptr(out)))
  return out


class _ProjectedConv:
  """Shared part of the layers below: neighborhood, projection + weight
  product on a padded weight matrix, explicit backward for features and
  weights."""

  def _setup(self, cin, k, cout):
    self.cin, self.k, self.cout = int(cin), int(k), int(cout)
    self.k_pad = _basis_count(self.k)
    self.cout_pad = (self.cout + 7) // 8 * 8
    self._op = None
    self._saved = None

  def _neighborhood(self, point_cloud_in, point_cloud_out, radius, neighborhood):
    if neighborhood is not None:
      return neighborhood
    from . import pc
    return pc.grid_neighborhood(point_cloud_in, radius, point_cloud_out)

  def _project(self, basis, features, neigh, weights, ns, keep_for_backward):
    if self._op is None or self._op.ns != ns or self._op.backward_ws != keep_for_backward:
      self._op = ProjectionGemm(self.k_pad, self.cin, self.cout_pad, ns, features.device,
                                backward=keep_for_backward)
    wp = _pad_weights(_f32(weights), self.cin, self.k, self.k_pad, self.cout_pad)
    out = self._op.forward(basis, _f32(features), neigh._original_neigh_ids,
                           neigh._samples_neigh_ranges, wp)
    if keep_for_backward:
      self._saved = (neigh, basis, _f32(features), wp)
    return out[:, :self.cout] if self.cout_pad != self.cout else out

  def _backward(self, out_grads):
    neigh, basis, features, wp = self._saved
    g = _f32(out_grads)
    if self.cout_pad != self.cout:
      g = torch.nn.functional.pad(g, (0, self.cout_pad - self.cout))
    dbasis, dfeat, dwp = self._op.backward(basis, features, neigh._original_neigh_ids,
                                           neigh._samples_neigh_ranges, wp, g)
    dw = dwp.reshape(self.cin, self.k_pad, self.cout_pad)[:, :self.k, :self.cout]
    return dbasis, dfeat, dw.reshape(self.cin * self.k, self.cout).contiguous()


class KPConv(_ProjectedConv):
  """Rigid kernel-point convolution (KPConv.py:59-296).  kernel_points [K, D]
  are the layer's points before the 0.75 scaling of KPConv.py:129; weights
  [K * C_in, C_out] in the reference's layout (row c * K + k)."""

  def __init__(self, kernel_points, weights, num_features_in, kp_interpolation='linear'):
    self.kernel_points = _f32(kernel_points) * 0.75
    self.weights = _f32(weights)
    self.interpolation = kp_interpolation
    self._setup(num_features_in, self.kernel_points.shape[0], self.weights.shape[1])

  def forward(self, features, point_cloud_in, point_cloud_out, conv_radius, neighborhood=None,
              kernel_influence_dist=None, keep_for_backward=True):
    neigh = self._neighborhood(point_cloud_in, point_cloud_out, conv_radius, neighborhood)
    # KPConv.py:283-288: sigma is 1 unless an influence distance is given
    sigma = 1.0 if kernel_influence_dist is None else kernel_influence_dist / conv_radius
    basis = kp_basis(point_cloud_in._points, point_cloud_out._points, neigh._original_neigh_ids,
                     self.kernel_points, conv_radius, sigma, self.k_pad, self.interpolation)
    return self._project(basis, features, neigh, self.weights,
                         point_cloud_out._points.shape[0], keep_for_backward)

  def backward(self, out_grads):
    """(d_features, d_weights) of the last forward call; the kernel points of the
    rigid layer are not trained."""
    _, dfeat, dw = self._backward(out_grads)
    return dfeat, dw




class PointConv(_ProjectedConv):
  """PointConv layer (PointConv.py:37-281): one hidden layer on the unscaled
  point differences, divided by a learned transform of the normalised density.
  hidden_w [D, H], hidden_b [1, H] or [H], weights [H * C_in, C_out];
  pdf_weights = (w1 [1, 16], w2 [16, 1]), pdf_biases = (b1 [1, 16], b2 [1, 1])."""

  def __init__(self, hidden_w, hidden_b, weights, pdf_weights, pdf_biases, num_features_in,
               non_linearity_type='relu'):
    self.hidden_w, self.hidden_b = _f32(hidden_w), _f32(hidden_b).reshape(-1)
    self.weights = _f32(weights)
    self.pdf_weights = [_f32(w) for w in pdf_weights]
    self.pdf_biases = [_f32(b) for b in pdf_biases]
    self.activation, self.alpha = NON_LINEARITIES[non_linearity_type.lower()]
    hidden = self.hidden_w.shape[1]
    if hidden not in (8, 16, 32, 64):
      # BasisProj accepts these sizes only (basis_proj_ops.cpp:99-103)
      raise _lib.TfgpcError(1, "BasisProjOp expects a valid number of basis functions.")
    self._setup(num_features_in, hidden, self.weights.shape[1])

  def forward(self, features, point_cloud_in, point_cloud_out, radius, neighborhood=None,
              bandwidth=0.2, keep_for_backward=True):
    neigh = self._neighborhood(point_cloud_in, point_cloud_out, radius, neighborhood)
    pdf = neigh.get_pdf(bandwidth=bandwidth, mode=0)
    scale = pointconv_pdf(pdf, neigh._samples_neigh_ranges, self.pdf_weights[0],
                          self.pdf_biases[0], self.pdf_weights[1], self.pdf_biases[1])
    # PointConv.py:272: the kernel input is the point difference itself (radius 1)
    basis = kernel_basis(point_cloud_in._points, point_cloud_out._points,
                         neigh._original_neigh_ids, scale, self.hidden_w, self.hidden_b, 1.0,
                         self.activation, self.alpha)
    out = self._project(basis, features, neigh, self.weights,
                        point_cloud_out._points.shape[0], keep_for_backward)
    if keep_for_backward:
      self._kernel_inputs = (point_cloud_in, point_cloud_out, scale)
    return out

  def backward(self, out_grads):
    """(d_features, d_hidden_w, d_hidden_b, d_weights) of the last forward call.
    The 50 parameters of the density transform get no gradient here."""
    dbasis, dfeat, dw = self._backward(out_grads)
    neigh = self._saved[0]
    pc_in, pc_out, scale = self._kernel_inputs
    dhw, dhb = kernel_basis_grads(pc_in._points, pc_out._points, neigh._original_neigh_ids,
                                  scale, self.hidden_w, self.hidden_b, 1.0, dbasis,
                                  self.activation, self.alpha)
    return dfeat, dhw, dhb, dw


# ---- pooling and 1x1 convolution (Pooling.py, Conv1x1.py) ----------------------

POOL_MODES = {'max': 0, 'avg': 1, 'average': 1, 'mean': 1}


def neighborhood_pool(features, neighborhood, mode='max'):
  """MaxPooling / AveragePooling over a neighborhood (Pooling.py:148-162):
  [N_in, C] -> [N_out, C]."""
  features = _f32(features)
  nb, ranges = _i32(neighborhood._original_neigh_ids), _i32(neighborhood._samples_neigh_ranges)
  ns, c = ranges.shape[0], features.shape[1]
  out = torch.empty((ns, c), dtype=torch.float32, device=features.device)
  _lib.check(_lib.lib().tfgpc_neighborhood_pool(
      _stream(), c_int(POOL_MODES[mode]), c_int(c), c_i64(ns), c_i64(features.shape[0]),
      c_i64(nb.shape[0]), ptr(features), ptr(nb), ptr(ranges), ptr(out)))
  return out


def local_pool(features, point_cloud_in, point_cloud_out, pooling_radius, mode='max'):
  """Pooling.py:140-162: grid of the input cloud, neighborhood around the output
  points, pooled features."""
  from . import pc
  grid = pc.Grid(point_cloud_in, pooling_radius)
  return neighborhood_pool(features, pc.Neighborhood(grid, pooling_radius, point_cloud_out), mode)


def global_pool(features, point_cloud, mode='max'):
  """GlobalMaxPooling / GlobalAveragePooling (Pooling.py:51-57, 90-96):
  [N, C] -> [batch_size, C]."""
  features, bids = _f32(features), _i32(point_cloud._batch_ids)
  n, c = features.shape
  b = int(point_cloud._batch_size)
  out = torch.empty((b, c), dtype=torch.float32, device=features.device)
  nbytes = _lib.lib().tfgpc_global_pool_workspace_bytes(c_i64(b))
  ws = _workspace(nbytes, features.device)
  _lib.check(_lib.lib().tfgpc_global_pool(
      _stream(), c_int(POOL_MODES[mode]), c_int(c), c_i64(n), c_i64(b), ptr(features), ptr(bids),
      ptr(out), ptr(ws), c_sz(nbytes)))
  return out


def conv1x1(features, weights, bias):
  """Conv1x1.py:97: features [N, C_in] @ weights [C_in, C_out] + bias [1, C_out].
  The product runs on the tensor cores; channel counts that are not multiples
  of 8 are zero padded for it."""
  features, weights, bias = _f32(features), _f32(weights), _f32(bias).reshape(-1)
  n, cin = features.shape
  cout = weights.shape[1]
  cin_p, cout_p = (cin + 7) // 8 * 8, (cout + 7) // 8 * 8
  if cin_p != cin:
    features = torch.nn.functional.pad(features, (0, cin_p - cin))
  if cin_p != cin or cout_p != cout:
    weights = torch.nn.functional.pad(weights, (0, cout_p - cout, 0, cin_p - cin))
    bias = torch.nn.functional.pad(bias, (0, cout_p - cout))
  out = matmul_f32(features, weights)
  _lib.check(_lib.lib().tfgpc_add_bias(_stream(), c_i64(n), c_int(cout_p), ptr(out), ptr(bias)))
  return out[:, :cout] if cout_p != cout else out


def scale_bias_activation_(x, scale=1.0, bias=None, leaky_alpha=None):
  """In place x = act(x * scale + bias) (tfgpc_scale_bias_activation): inference
  batch normalisation folded into scale / bias, then an optional leaky ReLU."""
  if not x.is_contiguous() or x.dtype != torch.float32:
    raise _lib.TfgpcError(1, "scale_bias_activation_ expects a contiguous float32 tensor")
  n, c = x.shape
  b = None if bias is None else _f32(bias).reshape(-1)
  _lib.check(_lib.lib().tfgpc_scale_bias_activation(
      _stream(), c_i64(n), c_int(c), ptr(x), ctypes.c_float(float(scale)),
      ptr(b) if b is not None else ctypes.c_void_p(0), c_int(0 if leaky_alpha is None else 1),
      ctypes.c_float(0.0 if leaky_alpha is None else float(leaky_alpha))))
  return x
