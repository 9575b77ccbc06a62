"""The layer step at the benchmark's full size (32 clouds x 16384 points, C_in
128, K 16, C_out 256; 1.67e7 neighbor pairs) checked against fp64 arithmetic
on the device.

The CPU oracle needs minutes for this size, so the check is built from what does
not depend on size: every output of the step is a sum of products of values
the library itself hands out (neighbor lists, densities, basis), and the same
sums are formed here in fp64 with torch index_add / matmul.  Tolerance 1e-4 of
max(|value|, rms), the one the small-size oracle tests use.
"""
import types

import pytest
import torch

import bench
from tensorflow_graphics_point_clouds_b200 import custom_ops as ops
from tensorflow_graphics_point_clouds_b200 import mcconv, pc

pytestmark = pytest.mark.gpu
REL = 1e-4


def rel_err(got, ref):
  got = got.double().reshape(ref.shape)
  scale = torch.maximum(ref.abs(), ref.pow(2).mean().sqrt())
  return float(((got - ref).abs() / scale).max())


def test_layer_step_full_size_against_fp64():
  args = types.SimpleNamespace(clouds=32, points=16384, radius=0.079, cin=128, cout=256,
                               hidden=16)
  pts, bid, feat, d_out, w1, b1, wf = bench.make_inputs(args, 0)
  dev = torch.device("cuda", 0)
  pts, bid, feat, d_out = (torch.from_numpy(v).to(dev) for v in (pts, bid, feat, d_out))
  layer = mcconv.MCConv(torch.from_numpy(w1).to(dev), torch.from_numpy(b1).to(dev),
                        torch.from_numpy(wf).to(dev), args.cin)
  cloud = pc.PointCloud(pts, bid, args.clouds)
  out = layer.forward(feat, cloud, cloud, args.radius)
  dfeat, dw1, db1, dwf = layer.backward(d_out)
  layer._op.check_status()
  neigh, _, _, radius, _, _, features, wd, w1f, b1f = layer._saved
  pdf = neigh.get_pdf()            # per pair (the layer itself reads the per-point table)
  basis = layer.saved_basis()      # the grouped path keeps it as a bf16 pair: hi + mid
  nb = neigh._original_neigh_ids.long()
  n, c, k = features.shape[0], args.cin, args.hidden
  m = nb.shape[0]
  assert m > 16_000_000

  # kernel basis
  p64 = pts.double()
  delta = (p64[nb[:, 0]] - p64[nb[:, 1]]) / radius
  pre = delta @ w1f.double() + b1f.double()
  basis64 = torch.where(pre > 0, pre, 0.2 * pre) / pdf.double()[:, None]
  assert rel_err(basis, basis64) < REL

  # projection, forward product, weight gradients
  f64, b64 = features.double(), basis.double()
  x64 = torch.zeros(n, c * k, dtype=torch.float64, device=dev)
  chunk = 1 << 19
  for i in range(0, m, chunk):
    sl = slice(i, min(m, i + chunk))
    x64.index_add_(0, nb[sl, 1],
                   (f64[nb[sl, 0]][:, :, None] * b64[sl][:, None, :]).reshape(-1, c * k))
  x_lib = ops.basis_proj(basis, features, neigh._original_neigh_ids,
                         neigh._samples_neigh_ranges)
  assert rel_err(x_lib, x64) < REL
  del x_lib
  w64, g64 = wd.double(), d_out.double()
  assert rel_err(out, x64 @ w64) < REL
  # the sum over 524 288 samples: tensor-core accumulators truncate, the library
  # keeps every accumulation chain at 2048 terms or fewer
  assert rel_err(dwf, x64.T @ g64) < REL
  del x64

  # gradients of the features and of the kernel MLP
  dx64 = g64 @ w64.T
  df64 = torch.zeros(n, c, dtype=torch.float64, device=dev)
  db64 = torch.empty(m, k, dtype=torch.float64, device=dev)
  for i in range(0, m, chunk):
    sl = slice(i, min(m, i + chunk))
    dx = dx64[nb[sl, 1]].reshape(-1, c, k)
    df64.index_add_(0, nb[sl, 0], torch.einsum("pck,pk->pc", dx, b64[sl]))
    db64[sl] = torch.einsum("pck,pc->pk", dx, f64[nb[sl, 0]])
  assert rel_err(dfeat, df64) < REL
  # The leaky-ReLU slope is taken from the sign the library's own fp32
  # pre-activation had (the sign of its basis value): a handful of the 2.7e8
  # pre-activations lie within fp32 rounding of zero, and each such pair alone
  # moves a weight gradient by 2e-4 of its size.
  assert int(((basis > 0) != (pre > 0)).sum()) < 64
  dpre = db64 / pdf.double()[:, None] * torch.where(basis > 0, 1.0, 0.2).double()
  assert rel_err(dw1.reshape(3, k), delta.T @ dpre) < REL
  assert rel_err(db1.reshape(k), dpre.sum(0)) < REL
