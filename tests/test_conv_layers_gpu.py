"""KPConv and PointConv on the projection + weight-product path against the
NumPy restatements of pylib/pc/layers/KPConv.py and PointConv.py."""
import numpy as np
import pytest

from oracle import pylib_ref as pr
from tensorflow_graphics_point_clouds_b200 import mcconv, pc
from test_ops_gpu import close, t, grid_pair, neigh_pair, random_cloud

pytestmark = pytest.mark.gpu
F32 = np.float32


def layer_case(rng, d, n_pts, n_smp, b, radius):
  pts, bid = random_cloud(rng, b, n_pts, d)
  smp, sbid = random_cloud(rng, b, n_smp, d)
  g_ref, g = grid_pair(pts, bid, b, radius)
  nb_ref, nb = neigh_pair(g_ref, g, radius, smp, sbid)
  clouds = (pc.PointCloud(t(pts), t(bid), b), pc.PointCloud(t(smp), t(sbid), b))
  return pts, smp, nb_ref, nb, clouds


@pytest.mark.parametrize("n_pts,n_smp,cin,cout,b,radius,num_kp,interp,sigma_dist",
                         [(200, 20, 1, 3, 16, 0.7, 5, 'linear', None),
                          (400, 40, 3, 3, 8, 0.7, 5, 'linear', None),
                          (400, 10, 3, 1, 1, np.sqrt(3), 5, 'linear', None),
                          (3000, 600, 8, 16, 4, 0.3, 15, 'linear', 0.2),
                          (3000, 600, 16, 32, 4, 0.3, 15, 'gaussian', None),
                          (3000, 500, 128, 64, 3, 0.25, 16, 'linear', None),
                          (2000, 300, 32, 20, 3, 0.3, 33, 'gaussian', 0.25)])
def test_kpconv_forward_backward(n_pts, n_smp, cin, cout, b, radius, num_kp, interp, sigma_dist):
  rng = np.random.default_rng(n_pts + num_kp + cin)
  pts, smp, nb_ref, nb, (cloud_in, cloud_out) = layer_case(rng, 3, n_pts, n_smp, b, radius)
  feat = rng.uniform(size=(n_pts, cin)).astype(F32)
  kp = rng.normal(size=(num_kp, 3)).astype(F32) * F32(0.5)
  w = (rng.normal(size=(num_kp * cin, cout)) / np.sqrt(num_kp * cin)).astype(F32)
  sigma = 1.0 if sigma_dist is None else sigma_dist / radius
  ref = pr.kpconv_forward(feat, pts, smp, nb_ref, kp * F32(0.75), w, radius, sigma, interp)
  layer = mcconv.KPConv(t(kp), t(w), cin, interp)
  out = layer.forward(t(feat), cloud_in, cloud_out, radius, neighborhood=nb,
                      kernel_influence_dist=sigma_dist)
  close(out.cpu().numpy(), ref)
  # backward: the layer is linear in the features and in the weights
  g_out = rng.normal(size=(n_smp, cout)).astype(F32)
  dfeat, dw = layer.backward(t(g_out))
  basis = pr.kpconv_basis(pts, smp, nb_ref, kp * F32(0.75), radius, sigma, interp)
  ids = nb_ref.original_neigh_ids
  x = np.zeros((n_smp, cin, num_kp))
  np.add.at(x, ids[:, 1], feat[ids[:, 0]][:, :, None].astype(np.float64) * basis[:, None, :])
  close(dw.cpu().numpy(), x.reshape(n_smp, -1).T @ g_out.astype(np.float64))
  dx = (g_out.astype(np.float64) @ w.T.astype(np.float64)).reshape(n_smp, cin, num_kp)
  ref_df = np.zeros((n_pts, cin))
  np.add.at(ref_df, ids[:, 0], np.einsum('mck,mk->mc', dx[ids[:, 1]], basis))
  close(dfeat.cpu().numpy(), ref_df)


@pytest.mark.parametrize("n_pts,n_smp,cin,cout,b,radius,hidden,d,act",
                         [(2000, 200, 3, 3, 16, 0.7, 8, 2, 'relu'),
                          (2000, 200, 1, 3, 16, 0.7, 8, 3, 'relu'),
                          (4000, 100, 3, 1, 1, np.sqrt(3), 16, 3, 'relu'),
                          (2000, 200, 3, 3, 16, 0.7, 8, 4, 'lrelu'),
                          (3000, 500, 64, 32, 3, 0.25, 32, 3, 'elu'),
                          (3000, 500, 128, 128, 3, 0.25, 16, 3, 'relu')])
def test_pointconv_forward_backward(n_pts, n_smp, cin, cout, b, radius, hidden, d, act):
  rng = np.random.default_rng(n_pts + hidden + d + cin)
  pts, smp, nb_ref, nb, (cloud_in, cloud_out) = layer_case(rng, d, n_pts, n_smp, b, radius)
  feat = rng.uniform(size=(n_pts, cin)).astype(F32)
  hw = rng.normal(size=(d, hidden)).astype(F32)
  hb = (rng.normal(size=(1, hidden)) * 0.1).astype(F32)
  w = (rng.normal(size=(hidden * cin, cout)) / np.sqrt(hidden * cin)).astype(F32)
  # positive second-layer weights and biases keep the learned density scale away from zero
  pw = [rng.normal(size=(1, 16)).astype(F32), np.abs(rng.normal(size=(16, 1))).astype(F32)]
  pb = [np.abs(rng.normal(size=(1, 16))).astype(F32), np.ones((1, 1), F32)]
  pdf_ref = nb_ref.get_pdf()
  ref, basis = pr.pointconv_forward(feat, pts, smp, nb_ref, pdf_ref, hw, hb, w, pw, pb, act)
  layer = mcconv.PointConv(t(hw), t(hb), t(w), [t(x) for x in pw], [t(x) for x in pb], cin, act)
  out = layer.forward(t(feat), cloud_in, cloud_out, radius, neighborhood=nb)
  close(out.cpu().numpy(), ref)
  scale = mcconv.pointconv_pdf(nb.get_pdf(), nb._samples_neigh_ranges, t(pw[0]), t(pb[0]),
                               t(pw[1]), t(pb[1]))
  close(scale.cpu().numpy(), pr.pointconv_pdf(pdf_ref, nb_ref, pw[0], pb[0], pw[1], pb[1]))
  g_out = rng.normal(size=(n_smp, cout)).astype(F32)
  dfeat, dhw, dhb, dw = layer.backward(t(g_out))
  ids = nb_ref.original_neigh_ids
  x = np.zeros((n_smp, cin, hidden))
  np.add.at(x, ids[:, 1], feat[ids[:, 0]][:, :, None].astype(np.float64) * basis[:, None, :])
  close(dw.cpu().numpy(), x.reshape(n_smp, -1).T @ g_out.astype(np.float64))
  dx = (g_out.astype(np.float64) @ w.T.astype(np.float64)).reshape(n_smp, cin, hidden)
  ref_df = np.zeros((n_pts, cin))
  np.add.at(ref_df, ids[:, 0], np.einsum('mck,mk->mc', dx[ids[:, 1]], basis))
  close(dfeat.cpu().numpy(), ref_df)
  assert dhw.shape == (d, hidden) and dhb.reshape(-1).shape == (hidden,)


@pytest.mark.parametrize("c", [1, 6, 64, 129])
@pytest.mark.parametrize("mode", ['max', 'avg'])
def test_pooling_layers(c, mode):
  rng = np.random.default_rng(c + len(mode))
  pts, smp, nb_ref, nb, (cloud_in, cloud_out) = layer_case(rng, 3, 4000, 700, 4, 0.12)
  feat = rng.normal(size=(4000, c)).astype(F32)
  out = mcconv.neighborhood_pool(t(feat), nb, mode).cpu().numpy()
  ref = pr.neighborhood_pool(feat, nb_ref, mode)
  assert (np.diff(np.concatenate(([0], nb_ref.ranges))) == 0).any()   # empty samples occur
  if mode == 'max':
    assert np.array_equal(out, ref)
  else:
    close(out, ref)
  out2 = mcconv.local_pool(t(feat), cloud_in, cloud_out, 0.12, mode).cpu().numpy()
  assert np.array_equal(out2, out)
  # global pooling, with one cloud of the batch left empty
  cloud = pc.PointCloud(cloud_in._points, cloud_in._batch_ids, 6)
  g = mcconv.global_pool(t(feat), cloud, mode).cpu().numpy()
  g_ref = pr.global_pool(feat, cloud_in._batch_ids.cpu().numpy(), 6, mode)
  if mode == 'max':
    assert np.array_equal(g, g_ref)
  else:
    close(g, g_ref)


@pytest.mark.parametrize("n,cin,cout", [(1000, 8, 16), (3000, 1, 128), (5000, 128, 40),
                                        (777, 20, 3), (4096, 1024, 40)])
def test_conv1x1(n, cin, cout):
  rng = np.random.default_rng(n + cin)
  feat = rng.normal(size=(n, cin)).astype(F32)
  w = (rng.normal(size=(cin, cout)) / np.sqrt(cin)).astype(F32)
  bias = rng.normal(size=(1, cout)).astype(F32)
  out = mcconv.conv1x1(t(feat), t(w), t(bias))
  close(out.cpu().numpy(), pr.conv1x1(feat, w, bias))


def test_small_classifier_forward():
  """The classification network of modelnet40_small.py (MCConv variant, widths
  1-128-256-512-1024-1024-40, sampling radii 0.1 / 0.2 / 0.4 / 2 sqrt(3)) on 32
  clouds of 1024 points: logits against the NumPy / C restatement."""
  from tensorflow_graphics_point_clouds_b200 import classifier, synthetic
  b = 32
  radii = [0.1, 0.2, 0.4, 2 * np.sqrt(3)]
  pts, bid = synthetic.unit_sphere_shapes(b, 1024, seed=4)
  feat = np.ones((len(pts), 1), F32)
  weights = synthetic.small_classifier_weights(40)
  ref = pr.small_classifier_forward(pts, bid, b, feat, weights, radii)
  net = classifier.SmallClassifier(weights, radii, "cuda")
  out = net.forward(t(pts), t(bid), b, t(feat))
  assert out.shape == (b, 40)
  close(out.cpu().numpy(), ref)


def test_three_level_classifier_forward():
  """Three levels with sampling radii 0.1 / 0.2 / sqrt(3), widths 128 / 256 / 1024
  and a 1024 -> 40 head on 32 clouds of 1024 points (the layout of the
  benchmark's classifier configuration); the points the last radius leaves in a
  cloud are averaged before the head."""
  from tensorflow_graphics_point_clouds_b200 import classifier, synthetic
  b = 32
  preset = classifier.PRESETS['three_level']
  pts, bid = synthetic.unit_sphere_shapes(b, 1024, seed=4)
  feat = np.ones((len(pts), 1), F32)
  weights = synthetic.small_classifier_weights(41, preset['feature_sizes'],
                                               head_layers=preset['head_layers'])
  ref = pr.small_classifier_forward(pts, bid, b, feat, weights, preset['radii'],
                                    pool_before_head=True)
  net = classifier.SmallClassifier(weights, preset['radii'], "cuda", pool_before_head=True)
  out = net.forward(t(pts), t(bid), b, t(feat))
  assert out.shape == (b, 40)
  close(out.cpu().numpy(), ref)
