"""Tensor-core GEMM and fused MCConv parity (fp32 within rel 1e-4)."""
import numpy as np
import pytest
import torch

import oracle as orc
from oracle import pylib_ref as pr
from tensorflow_graphics_point_clouds_b200 import mcconv, pc, synthetic
from test_ops_gpu import close, t, grid_pair, neigh_pair, random_cloud

pytestmark = pytest.mark.gpu
F32 = np.float32


@pytest.mark.parametrize("at,bt", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (304, 64, 192), (1000, 256, 2048),
                                   (256, 2048, 256), (2048, 256, 5000 // 8 * 8), (64, 16, 128),
                                   (19144, 384, 200)])
def test_matmul_f32_layouts(at, bt, m, n, k):
  rng = np.random.default_rng(m + n + k)
  a = rng.normal(size=(m, k)).astype(F32)
  b = (rng.uniform(-1, 1, size=(k, n)) * 0.05).astype(F32)
  ref = a.astype(np.float64) @ b.astype(np.float64)
  a_dev = t(a.T.copy() if at else a)
  b_dev = t(b.T.copy() if bt else b)
  got = mcconv.matmul_f32(a_dev, b_dev, a_transposed=at, b_transposed=bt)
  close(got.cpu().numpy(), ref, rel=1e-4)


def test_matmul_f32_long_reduction():
  """The shape of the layer's weight-gradient product at full batch size: the
  reduction runs over 2^19 samples.  Tensor cores accumulate by truncation, so
  the error of one accumulator grows with the number of terms it takes (7e-4
  when the reduction was cut into 9 slices); the library cuts it into slices of
  2048 terms.  Checked against fp64 on the device."""
  import torch
  gen = torch.Generator(device="cuda").manual_seed(5)
  m, n, k = 256, 128, 1 << 19
  a = torch.randn((k, m), generator=gen, device="cuda")           # [K, M]: a transposed
  b = torch.randn((k, n), generator=gen, device="cuda")           # [K, N]
  got = mcconv.matmul_f32(a, b, a_transposed=True, b_transposed=False)
  ref = torch.zeros((m, n), dtype=torch.float64, device="cuda")
  for i in range(0, k, 1 << 16):
    ref += a[i:i + (1 << 16)].double().T @ b[i:i + (1 << 16)].double()
  close(got.cpu().numpy(), ref.cpu().numpy(), rel=1e-4)


def mc_case(rng, c, k, cout, n_pts=3000, n_smp=700, radius=0.25, b=3):
  pts, bid = random_cloud(rng, b, n_pts, 3)
  smp, sbid = random_cloud(rng, b, n_smp, 3)
  g_ref, g = grid_pair(pts, bid, b, radius)
  nb_ref, nb = neigh_pair(g_ref, g, radius, smp, sbid)
  m = len(nb_ref.neighbors)
  basis = rng.normal(size=(m, k)).astype(F32)
  feat = rng.normal(size=(n_pts, c)).astype(F32)
  w = synthetic.glorot_uniform(rng, c * k, cout, (1, c * k, cout))
  return nb_ref, nb, basis, feat, w


@pytest.mark.parametrize("c,k,cout", [(8, 16, 16), (128, 16, 256), (32, 8, 64), (64, 32, 128),
                                      (3, 16, 32), (16, 64, 40), (256, 16, 64), (128, 32, 32),
                                      (128, 64, 16), (384, 16, 32)])
def test_mcconv_forward_backward(c, k, cout):
  rng = np.random.default_rng(c * 1000 + k + cout)
  nb_ref, nb, basis, feat, w = mc_case(rng, c, k, cout)
  ref_out, ref_x = pr.mcconv_forward(feat, basis, nb_ref, w)
  ns = len(nb_ref.ranges)
  op = mcconv.ProjectionGemm(k, c, cout, ns, "cuda", backward=True)
  out = op.forward(t(basis), t(feat), nb._original_neigh_ids, nb._samples_neigh_ranges, t(w[0]))
  op.check_status()
  close(out.cpu().numpy(), ref_out)
  d_out = rng.normal(size=ref_out.shape).astype(F32)
  ref_dw, ref_db, ref_df, _ = pr.mcconv_backward(feat, basis, nb_ref, w, ref_x, d_out)
  for reuse in (True, False):
    db, df, dw = op.backward(t(basis), t(feat), nb._original_neigh_ids,
                             nb._samples_neigh_ranges, t(w[0]), t(d_out), reuse_forward=reuse)
    op.check_status()
    close(dw.cpu().numpy(), ref_dw[0])
    close(db.cpu().numpy(), ref_db)
    close(df.cpu().numpy(), ref_df)


@pytest.mark.parametrize("n_pts,n_smp,radius", [(3000, 701, 0.25), (3000, 702, 0.45),
                                                (20000, 5003, 0.12), (500, 3, 0.5),
                                                (3000, 700, 0.08), (40, 5, 0.9)])
def test_mcconv_wide_layer_ragged_shapes(n_pts, n_smp, radius):
  """C = 128, K = 16 (the tensor-core projection kernels) on sample counts that
  are not multiples of four, samples with more pairs than one MMA block holds,
  samples without neighbors, and more sample groups than the GPU has SMs."""
  c, k, cout = 128, 16, 64
  rng = np.random.default_rng(n_pts + n_smp)
  nb_ref, nb, basis, feat, w = mc_case(rng, c, k, cout, n_pts=n_pts, n_smp=n_smp, radius=radius)
  ref_out, ref_x = pr.mcconv_forward(feat, basis, nb_ref, w)
  ns = len(nb_ref.ranges)
  op = mcconv.ProjectionGemm(k, c, cout, ns, "cuda", backward=True)
  out = op.forward(t(basis), t(feat), nb._original_neigh_ids, nb._samples_neigh_ranges, t(w[0]))
  op.check_status()
  close(out.cpu().numpy(), ref_out)
  d_out = rng.normal(size=ref_out.shape).astype(F32)
  ref_dw, ref_db, ref_df, _ = pr.mcconv_backward(feat, basis, nb_ref, w, ref_x, d_out)
  db, df, dw = op.backward(t(basis), t(feat), nb._original_neigh_ids, nb._samples_neigh_ranges,
                           t(w[0]), t(d_out))
  op.check_status()
  close(dw.cpu().numpy(), ref_dw[0])
  close(db.cpu().numpy(), ref_db)
  close(df.cpu().numpy(), ref_df)


def test_dense_final_weights_matches_reference_layout():
  rng = np.random.default_rng(5)
  cin, g, h, co = 8, 4, 8, 16
  nb_ref, nb, basis, feat, _ = mc_case(rng, cin, g * h, g * co)
  wf = rng.normal(size=(g, cin * h, co)).astype(F32) * 0.1
  ref_out, _ = pr.mcconv_forward(feat, basis, nb_ref, wf)
  dense = mcconv.dense_final_weights(t(wf), cin, h)
  op = mcconv.ProjectionGemm(g * h, cin, g * co, len(nb_ref.ranges), "cuda", backward=False)
  out = op.forward(t(basis), t(feat), nb._original_neigh_ids, nb._samples_neigh_ranges, dense)
  op.check_status()
  close(out.cpu().numpy(), ref_out)
  back = mcconv.blocks_of_dense_grad(dense, g, cin, h)
  assert torch.equal(back, t(wf))


@pytest.mark.parametrize("d,g,h", [(3, 1, 16), (3, 4, 8), (2, 1, 8), (4, 2, 32)])
def test_mcconv_layer_matches_oracle(d, g, h):
  """Whole layer from raw points (MCConv.py:196-278): output and all gradients."""
  rng = np.random.default_rng(900 + d + g)
  b, n_pts, cin, cout, radius = 3, 2500, 16, 32, 0.3
  pts, bid = random_cloud(rng, b, n_pts, d)
  feat = rng.normal(size=(n_pts, cin)).astype(F32)
  w1 = rng.normal(size=(g, d, h)).astype(F32)
  b1 = (rng.normal(size=(g, 1, h)) * 0.1).astype(F32)
  wf = (rng.normal(size=(g, cin * h, cout // g)) * 0.05).astype(F32)
  d_out = rng.normal(size=(n_pts, cout)).astype(F32)
  # oracle
  g_ref = pr.Grid(pts, bid, b, radius)
  nb_ref = pr.Neighborhood(g_ref, radius, pts, bid)
  pdf = nb_ref.get_pdf(bandwidth=0.2, mode=0)
  basis, diff, hid = pr.mcconv_basis(pts, pts, nb_ref, pdf, w1, b1, radius)
  ref_out, x = pr.mcconv_forward(feat, basis, nb_ref, wf)
  ref_dwf, ref_db, ref_df, _ = pr.mcconv_backward(feat, basis, nb_ref, wf, x, d_out)
  dpre = ref_db.astype(np.float64) / pdf.reshape(-1, 1) * np.where(hid > 0, 1.0, 0.2)
  ref_dw1 = (diff.astype(np.float64).T @ dpre).reshape(d, g, h).transpose(1, 0, 2)
  ref_db1 = dpre.sum(axis=0).reshape(g, 1, h)
  # library
  cloud = pc.PointCloud(t(pts), t(bid), b)
  layer = mcconv.MCConv(t(w1), t(b1), t(wf), cin)
  out = layer.forward(t(feat), cloud, cloud, radius)
  dfeat, dw1, db1, dwf = layer.backward(t(d_out))
  layer._op.check_status()
  close(layer.saved_basis().cpu().numpy(), basis)
  close(out.cpu().numpy(), ref_out)
  close(dfeat.cpu().numpy(), ref_df)
  close(dwf.cpu().numpy(), ref_dwf)
  close(dw1.cpu().numpy(), ref_dw1)         # measured: 2.0e-5
  close(db1.cpu().numpy(), ref_db1)         # measured: 2.1e-5


def test_bounded_wait_runs_out_and_is_reported():
  """Every device-side wait of the tensor-core kernels gives up after a time
  limit and reports through the workspace's status word.  Here one warp waits
  (1 ms limit) for a barrier phase that nothing completes: the kernel must
  return by itself, tfgpc_mcconv_status must report TFGPC_ETIMEOUT, and the
  next product on the same workspace must clear the word and be correct."""
  import ctypes
  from tensorflow_graphics_point_clouds_b200 import _lib
  from tensorflow_graphics_point_clouds_b200._lib import c_i64, c_int, c_sz, ptr
  lib = _lib.lib()
  m, n, k = 256, 128, 512
  nbytes = lib.tfgpc_matmul_workspace_bytes(c_i64(m), c_i64(n), c_i64(k))
  ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  returned = c_int(0)
  _lib.check(lib.tfgpc_debug_bounded_wait(stream, ptr(ws), c_sz(nbytes), ctypes.c_uint(1000),
                                          ctypes.byref(returned)))
  assert returned.value == 1                      # the kernel ran to its end
  status = c_int(0)
  rc = lib.tfgpc_mcconv_status(stream, ptr(ws), ctypes.byref(status))
  assert rc == 4 and status.value == 4            # TFGPC_ETIMEOUT
  assert b"bounded wait" in lib.tfgpc_last_error()
  # the context is intact: a product on the same workspace succeeds
  rng = np.random.default_rng(1)
  a = rng.normal(size=(m, k)).astype(F32); b = rng.normal(size=(k, n)).astype(F32)
  c = torch.empty((m, n), dtype=torch.float32, device="cuda")
  ta, tb = t(a), t(b)
  _lib.check(lib.tfgpc_matmul_f32(stream, c_i64(m), c_i64(n), c_i64(k), ptr(ta), c_int(0),
                                  ptr(tb), c_int(0), ptr(c), ptr(ws), c_sz(nbytes)))
  _lib.check(lib.tfgpc_mcconv_status(stream, ptr(ws), ctypes.byref(status)))
  assert status.value == 0
  close(c.cpu().numpy(), a.astype(np.float64) @ b.astype(np.float64))
  # argument checks
  assert lib.tfgpc_debug_bounded_wait(stream, ptr(ws), c_sz(nbytes), ctypes.c_uint(0),
                                      ctypes.byref(returned)) == 1


@pytest.mark.parametrize("hidden,g,act,own", [([8], 1, 'elu', False), ([6, 8], 1, 'leaky_relu', True),
                                              ([8, 4], 2, 'elu', False), ([16], 1, 'relu', True),
                                              ([5, 7, 8], 1, 'elu', True)])
def test_mcconv_deep_kernel_mlp_and_point_gradients(hidden, g, act, own):
  """Kernel MLPs with several hidden layers (MCConv.py:165-168) and the gradients
  with respect to the point coordinates (monte_carlo_conv_test.py:182-219),
  against the float64 layer of the oracle, whose analytic gradients are pinned
  to finite differences in tests/test_oracle_known_answers.py."""
  rng = np.random.default_rng(1000 + sum(hidden) + g)
  b, n_pts, d, cin, cout, radius = 3, 1500, 3, 16, 32, 0.3
  pts, bid = random_cloud(rng, b, n_pts, d)
  if own:
    smp, sbid = pts, bid
  else:
    smp, sbid = random_cloud(rng, b, 400, d)
  feat = rng.normal(size=(n_pts, cin)).astype(F32)
  sizes = [d] + hidden
  ws = [rng.normal(size=(g, sizes[i], sizes[i + 1])).astype(F32) for i in range(len(hidden))]
  bs = [(rng.normal(size=(g, 1, sizes[i + 1])) * 0.1).astype(F32) for i in range(len(hidden))]
  wf = (rng.normal(size=(g, cin * hidden[-1], cout // g)) * 0.05).astype(F32)
  d_out = rng.normal(size=(len(smp), cout)).astype(F32)
  g_ref = pr.Grid(pts, bid, b, radius)
  nb_ref = pr.Neighborhood(g_ref, radius, smp, sbid)
  pdf = nb_ref.get_pdf(bandwidth=0.2, mode=0)
  ref_out = pr.mcconv_layer(pts, smp, feat, nb_ref, pdf, ws, bs, wf, radius, act)
  ref = pr.mcconv_layer_grads(pts, smp, feat, nb_ref, pdf, ws, bs, wf, radius, d_out, act)
  cloud = pc.PointCloud(t(pts), t(bid), b)
  smp_cloud = cloud if own else pc.PointCloud(t(smp), t(sbid), b)
  layer = mcconv.MCConv([t(w) for w in ws], [t(x) for x in bs], t(wf), cin,
                        non_linearity_type=act)
  out = layer.forward(t(feat), cloud, smp_cloud, radius)
  dfeat, dws, dbs, dwf, dpin, dpout, dpdf = layer.backward(t(d_out), point_grads=True)
  layer._op.check_status()
  close(out.cpu().numpy(), ref_out)
  close(dfeat.cpu().numpy(), ref["d_features"])
  close(dwf.cpu().numpy(), ref["d_wf"])
  for a, r in zip(dws, ref["d_weights"]):
    close(a.cpu().numpy(), r)
  for a, r in zip(dbs, ref["d_biases"]):
    close(a.cpu().numpy(), r)
  close(dpdf.cpu().numpy(), ref["d_pdf"])
  if own:
    assert dpin is dpout           # one cloud: one gradient, the sum of both roles
    close(dpin.cpu().numpy(), ref["d_points_in"] + ref["d_points_out"])
  else:
    close(dpin.cpu().numpy(), ref["d_points_in"])
    close(dpout.cpu().numpy(), ref["d_points_out"])


@pytest.mark.parametrize("own", [True, False])
def test_pdf_point_grads_follow_the_reference_chain(own):
  """Neighborhood.pdf_point_grads: per-pair density gradients -> per-point sums ->
  ComputePdfPtGrads on the sorted self neighborhood -> original point order."""
  rng = np.random.default_rng(77)
  b, n_pts, radius = 3, 2000, 0.25
  pts, bid = random_cloud(rng, b, n_pts, 3)
  g_ref = pr.Grid(pts, bid, b, radius)
  cloud = pc.PointCloud(t(pts), t(bid), b)
  grid = pc.Grid(cloud, radius)
  if own:
    nb_ref, nb = pr.Neighborhood(g_ref, radius, pts, bid), pc.Neighborhood(grid, radius, cloud)
  else:
    smp, sbid = random_cloud(rng, b, 300, 3)
    nb_ref = pr.Neighborhood(g_ref, radius, smp, sbid)
    nb = pc.Neighborhood(grid, radius, pc.PointCloud(t(smp), t(sbid), b))
  nb.get_pdf(bandwidth=0.2, mode=0)
  gp = rng.normal(size=len(nb_ref.neighbors)).astype(F32)
  got = nb.pdf_point_grads(t(gp), bandwidth=0.2, mode=0).cpu().numpy()
  per_point = np.zeros(n_pts, np.float64)
  np.add.at(per_point, nb_ref.neighbors[:, 0], gp)
  self_ref = pr.Neighborhood(g_ref, radius)
  inv = np.repeat(F32(1 / radius), 3); inv_bw = np.repeat(F32(1 / 0.2), 3)
  ref_sorted = orc.compute_pdf_pt_grads(g_ref.sorted_points, self_ref.neighbors, self_ref.ranges,
                                        inv_bw, inv, per_point.astype(F32), 0)
  ref = np.empty_like(ref_sorted)
  ref[g_ref.sorted_indices] = ref_sorted
  close(got, ref)


@pytest.mark.parametrize("act,alpha", [(0, 0.2), (1, 0.0)])
def test_kernel_basis_packed_point_table(act, alpha):
  """points_in as the packed (x, y, z, 1 / density) table gives the results of
  the density table read at the neighbor index: the basis (fp32 rows and bf16
  pair) bit for bit, the weight gradients up to the order of their atomic sums."""
  rng = np.random.default_rng(41)
  n, ns, m, k = 5000, 900, 40000, 16
  p_in = t(rng.uniform(0, 1, (n, 3)).astype(np.float32))
  p_out = t(rng.uniform(0, 1, (ns, 3)).astype(np.float32))
  nbrs = t(np.stack([rng.integers(0, n, m), np.sort(rng.integers(0, ns, m))], 1).astype(np.int32))
  pdf = t(rng.uniform(0.5, 30.0, n).astype(np.float32))
  w1 = t(rng.standard_normal((3, k)).astype(np.float32))
  b1 = t(rng.standard_normal(k).astype(np.float32))
  packed = mcconv.pack_points_density(p_in, pdf)
  assert torch.equal(packed[:, :3], p_in) and torch.equal(packed[:, 3], 1.0 / pdf)
  ref, ref_pair = mcconv.kernel_basis_split(p_in, p_out, nbrs, pdf, w1, b1, 0.3, act, alpha,
                                            pdf_by_neighbor=1)
  got, got_pair = mcconv.kernel_basis_split(packed, p_out, nbrs, None, w1, b1, 0.3, act, alpha,
                                            pdf_by_neighbor=2)
  assert torch.equal(got, ref) and torch.equal(got_pair.view(torch.int16), ref_pair.view(torch.int16))
  assert torch.equal(mcconv.kernel_basis(packed, p_out, nbrs, None, w1, b1, 0.3, act, alpha,
                                         pdf_by_neighbor=2), ref)
  dbasis = t(rng.standard_normal((m, k)).astype(np.float32))
  dw_ref, db_ref = mcconv.kernel_basis_grads(p_in, p_out, nbrs, pdf, w1, b1, 0.3, dbasis, act,
                                             alpha, pdf_by_neighbor=1)
  dw, db = mcconv.kernel_basis_grads(packed, p_out, nbrs, None, w1, b1, 0.3, dbasis, act, alpha,
                                     pdf_by_neighbor=2)
  close(dw.cpu().numpy(), dw_ref.cpu().numpy(), 1e-5)
  close(db.cpu().numpy(), db_ref.cpu().numpy(), 1e-5)
  # the packed table exists for D = 3 only
  with pytest.raises(mcconv._lib.TfgpcError):
    mcconv.kernel_basis(packed[:, :2].contiguous(), p_out[:, :2].contiguous(), nbrs, None,
                        w1[:2].contiguous(), b1, 0.3, act, alpha, pdf_by_neighbor=2)
