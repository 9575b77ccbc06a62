"""Host-side multi-GPU logic on CPU ranks (gloo, world size 2): cloud sharding
covers the batch exactly once, and summing the per-shard weight gradients with
one all-reduce reproduces the gradient of the whole batch (the oracle is the
compute here; the GPU path uses the same helpers around the CUDA library)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from tensorflow_graphics_point_clouds_b200 import dist as tdist
from tensorflow_graphics_point_clouds_b200 import synthetic

F32 = np.float32


@pytest.mark.parametrize("clouds,world", [(32, 1), (32, 2), (32, 8), (7, 4), (3, 8)])
def test_shards_cover_the_batch_once(clouds, world):
  seen = []
  for r in range(world):
    b, e = tdist.shard_clouds(clouds, world, r)
    assert 0 <= b <= e <= clouds
    seen.extend(range(b, e))
  assert seen == list(range(clouds))
  sizes = [tdist.shard_clouds(clouds, world, r) for r in range(world)]
  assert max(e - b for b, e in sizes) - min(e - b for b, e in sizes) <= 1


def layer_grads(pts, bid, feat, d_out, w1, b1, wf, clouds, radius):
  from oracle import pylib_ref as pr
  grid = pr.Grid(pts, bid, clouds, radius)
  neigh = pr.Neighborhood(grid, radius, pts, bid)
  pdf = neigh.get_pdf(bandwidth=0.2, mode=0)
  basis, diff, hid = pr.mcconv_basis(pts, pts, neigh, pdf, w1, b1, radius)
  out, x = pr.mcconv_forward(feat, basis, neigh, wf)
  d_wf, d_basis, d_feat, _ = pr.mcconv_backward(feat, basis, neigh, wf, x, d_out)
  return out, d_feat, d_wf


def make_case():
  clouds, per, cin, cout, k = 4, 300, 8, 16, 8
  pts, bid = synthetic.uniform_clouds(clouds, per, seed=5)
  rng = np.random.default_rng(6)
  feat = rng.standard_normal((clouds * per, cin), dtype=F32)
  d_out = rng.standard_normal((clouds * per, cout), dtype=F32)
  w1, b1, wf = synthetic.mcconv_weights(9, 3, cin, cout, 1, k)
  return clouds, pts, bid, feat, d_out, w1, b1, wf


def _worker(rank, world, port, result_dir):
  sys.path.insert(0, ROOT)
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    clouds, pts, bid, feat, d_out, w1, b1, wf = make_case()
    b, e = tdist.shard_clouds(clouds, world, rank)
    mask, local_bid = tdist.shard_points(torch.from_numpy(bid), b, e)
    mask = mask.numpy()
    out, d_feat, d_wf = layer_grads(pts[mask], local_bid.numpy().astype(np.int32), feat[mask],
                                    d_out[mask], w1, b1, wf, e - b, 0.25)
    g = [torch.from_numpy(d_wf.copy())]
    tdist.allreduce_sum_(g)
    # cell counts of the whole batch = maximum of the shards' counts
    from oracle import pylib_ref as pr
    own = pr.Grid(pts[mask], local_bid.numpy().astype(np.int32), e - b, 0.25).num_cells
    cells = tdist.allreduce_max_(torch.from_numpy(np.asarray(own, np.int32).copy()))
    slowest = tdist.max_over_ranks(float(rank + 1), "cpu")
    np.savez(os.path.join(result_dir, "rank%d.npz" % rank), out=out, d_feat=d_feat,
             d_wf=g[0].numpy(), mask=mask, slowest=slowest, cells=cells.numpy(),
             own_cells=np.asarray(own, np.int32))
  finally:
    dist.destroy_process_group()


def test_two_rank_allreduce_equals_single_process(tmp_path):
  world, port = 2, 29000 + os.getpid() % 2000
  mp.start_processes(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True,
                     start_method="spawn")
  clouds, pts, bid, feat, d_out, w1, b1, wf = make_case()
  ref_out, ref_dfeat, ref_dwf = layer_grads(pts, bid, feat, d_out, w1, b1, wf, clouds, 0.25)
  outs = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
  full_out = np.zeros_like(ref_out); full_df = np.zeros_like(ref_dfeat)
  from oracle import pylib_ref as pr
  batch_cells = np.asarray(pr.Grid(pts, bid, clouds, 0.25).num_cells)
  assert np.array_equal(np.maximum(outs[0]["own_cells"], outs[1]["own_cells"]), batch_cells)
  for o in outs:
    assert np.array_equal(o["cells"], batch_cells)
    full_out[o["mask"]] = o["out"]
    full_df[o["mask"]] = o["d_feat"]
    assert o["slowest"] == float(world)
    # every rank holds the same, complete weight gradient after the all-reduce
    np.testing.assert_allclose(o["d_wf"], ref_dwf, rtol=1e-4, atol=1e-4 * np.abs(ref_dwf).max())
  # shard concatenation equals the single-process result (clouds are independent)
  np.testing.assert_allclose(full_out, ref_out, rtol=1e-5, atol=1e-5)
  np.testing.assert_allclose(full_df, ref_dfeat, rtol=1e-5, atol=1e-5)


def test_bench_shards_concatenate_to_the_batch():
  """bench.py --gpus N shards ONE batch by cloud: the shards of all ranks, put one
  after the other, are the batch (batch ids re-based per shard)."""
  import argparse
  import bench
  args = argparse.Namespace(clouds=8, points=64, cin=8, cout=16, hidden=8)
  full = bench.make_inputs(args, 0)
  for world in (1, 2, 3, 8):
    parts = [bench.shard_inputs(full, args, r, world) for r in range(world)]
    assert sum(c for _, c, _ in parts) == args.clouds
    for idx, name in ((0, "points"), (2, "features"), (3, "gradients")):
      assert np.array_equal(np.concatenate([p[0][idx] for p in parts]), full[idx]), name
    first = 0
    for (inp, clouds, lo) in parts:
      assert lo == first
      assert inp[1].min() == 0 and inp[1].max() == clouds - 1
      first += len(inp[0])
