"""Benchmark of the MCConv hot path: one Monte-Carlo convolution layer, forward
and backward, from raw points (grid build, neighbor search, density estimate,
kernel basis, basis projection + weight GEMM, and all gradients).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # CPU port of the reference path

Workload (synthetic, seeded): ONE batch of 32 clouds x 16384 points uniform in
[0,1)^3, radius 0.079 (about 32 neighbors per point), C_in = 128, one kernel MLP
with 16 hidden units (K = 16), C_out = 256, fp32.  With N GPUs the batch is
sharded by cloud (32 / N clouds per rank, strong scaling) and the weight
gradients are all-reduced; before timing, every rank checks its shard's results
against the whole batch computed on its own GPU.  `--scaling weak` gives every
rank its own 32 clouds instead; a strong run on several GPUs also times the weak
variant and reports it under "weak_scaling".
Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

F32 = np.float32
METRIC = "mcconv_fwd_bwd_points_per_s"
UNIT = "points/s"


def parse_args():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-kernels"],
                  help="ours: this library; reference: the CPU port of the reference path (the "
                       "reference has no CPU kernels of its own); reference-kernels: the "
                       "reference's own CUDA kernels recompiled for sm_100a (oracle/_ref), op by "
                       "op beside this library's on the same inputs")
  ap.add_argument("--clouds", type=int, default=32)
  ap.add_argument("--points", type=int, default=16384)
  ap.add_argument("--radius", type=float, default=0.079)
  ap.add_argument("--cin", type=int, default=128)
  ap.add_argument("--cout", type=int, default=256)
  ap.add_argument("--hidden", type=int, default=16)
  ap.add_argument("--cpu-sample-clouds", type=int, default=1)
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--classifier-preset", default="three_level", choices=["three_level", "script"],
                  help="classifier workload: three levels with radii 0.1 / 0.2 / sqrt(3), widths "
                       "128 / 256 / 1024 and a 1024 -> 40 head, or the four levels of the "
                       "reference's modelnet40_small.py script")
  ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                  help="strong: one batch of --clouds clouds sharded over the GPUs; "
                       "weak: --clouds clouds per GPU")
  ap.add_argument("--no-shard-check", action="store_true",
                  help="skip the shard == whole-batch comparison of a multi-GPU strong run")
  ap.add_argument("--no-side", action="store_true",
                  help="skip the neighbor-search and sampling-hierarchy side measurements")
  ap.add_argument("--side-steps", type=int, default=5)
  ap.add_argument("--workload", default="mcconv", choices=["mcconv", "neighbors", "hierarchy", "classifier"],
                  help="mcconv: the headline step; neighbors: grid build + neighbor search + pdf "
                       "on 16 surface clouds (radius 0.05); hierarchy: 4-level Poisson-disk and "
                       "cell-average sampling of 8 x 100000 Gaussian-mixture points")
  return ap.parse_args()


def workload_config(args, world, scaling=None):
  scaling = scaling or args.scaling
  total_clouds = args.clouds * (world if scaling == "weak" else 1)
  per_gpu = (args.clouds if scaling == "weak" else
             "%d-%d" % (args.clouds // world, -(-args.clouds // world)) if args.clouds % world
             else args.clouds // world)
  return {
      "workload": "MCConv layer fwd+bwd from raw points, %d clouds x %d points%s, "
                  "uniform in [0,1)^3, radius %.3f (~32 neighbors/point), Cin=%d, K=%d, Cout=%d"
                  % (args.clouds, args.points, " per GPU" if scaling == "weak" else " in all",
                     args.radius, args.cin, args.hidden, args.cout),
      "clouds": total_clouds, "clouds_per_gpu": per_gpu, "points_per_cloud": args.points,
      "radius": args.radius,
      "cin": args.cin, "k": args.hidden, "cout": args.cout, "bandwidth": 0.2,
      "global_points": total_clouds * args.points,
      "parallelism": "clouds sharded over %d GPU(s); weight gradients all-reduced" % world,
      "l2": "inputs and intermediates are far larger than L2 (features 268 MB, projection "
            "4.3 GB per step), so no explicit flush between iterations",
  }


def make_inputs(args, rank):
  """Seeded host inputs of a batch of args.clouds clouds (rank 0: seed 2, the
  batch of the single-GPU and of every strong-scaling run; other ranks: their own
  batch in a weak-scaling run)."""
  from tensorflow_graphics_point_clouds_b200 import synthetic
  pts, bid = synthetic.uniform_clouds(args.clouds, args.points, seed=2 + 1000 * rank)
  rng = np.random.default_rng(12345 + rank)
  n = pts.shape[0]
  feat = rng.standard_normal((n, args.cin), dtype=F32)
  d_out = rng.standard_normal((n, args.cout), dtype=F32)
  w1, b1, wf = synthetic.mcconv_weights(7, 3, args.cin, args.cout, 1, args.hidden)
  return pts, bid, feat, d_out, w1, b1, wf


def shard_inputs(inputs, args, rank, world):
  """The clouds of `rank` out of the whole batch: (inputs of the shard, number of
  its clouds, index of its first point).  Clouds are stored one after the other
  with args.points points each."""
  from tensorflow_graphics_point_clouds_b200 import dist as tdist
  pts, bid, feat, d_out, w1, b1, wf = inputs
  b, e = tdist.shard_clouds(args.clouds, world, rank)
  lo, hi = b * args.points, e * args.points
  return ((pts[lo:hi], (bid[lo:hi] - b).astype(np.int32), feat[lo:hi], d_out[lo:hi], w1, b1, wf),
          e - b, lo)


# ------------------------------------------------------------------ peaks ----

def measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      p = json.load(f)
    return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
            "source": "measured"}
  return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


# Per-launch DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) taken
# from the ncu captures summarised under profiles/, scaled to this workload by
# the units processed; None where no capture exists yet.
NCU_TRAFFIC_BYTES_PER_POINT = {
    # profiles/projection_and_gemm_kernels_16_clouds.md: bytes of one launch / 262144 points
    "basis_proj_split": (1.030125e9 + 2.100271e9) / 262144,
    "basis_proj_split_mma": (1.318681e9 + 2.100419e9) / 262144,
    "basis_proj_grads": (4.091760e9 + 1.135269e9) / 262144,
    "basis_proj_grads_mma": (3.955412e9 + 1.121180e9) / 262144,
    "basis_proj_grads_tc": (3.792681e9 + 0.670124e9) / 262144,
    "gemm_bf16x3_k_mn": (2.176700e9 + 0.255623e9) / 262144,
    "gemm_bf16x3_mn_k_t": (2.172271e9 + 0.255117e9) / 262144,
    "gemm_bf16x3_k_k": (2.150015e9 + 2.098627e9) / 262144,
    "gemm_bf16x3_k_k_image": (2.149690e9 + 2.100168e9) / 262144,
    "gemm_bf16x3_k_mn_image": (2.149690e9 + 2.100168e9) / 262144,
    "gemm_bf16x3_mn_k_image": (0.270630e9 + 2.103353e9) / 262144,
    "gemm_bf16x3_mn_mn": (2.415943e9 + 0.004868e9) / 262144,
    # profiles/grouped_projection_kernels_8_clouds.md: bytes of one launch / 131072 points
    "basis_proj_fwd_tcu": (0.388030e9 + 1.016499e9) / 131072,
    "basis_proj_grads_tcu": (1.529835e9 + 0.318466e9) / 131072,
    "gemm_bf16x3_mn_k_scatter": (1.088718e9 + 0.120507e9) / 131072,
    "kernel_basis": (0.036006e9 + 0.212095e9) / 131072,
}


def kernel_model(name, sizes):
  """Algorithmic work of one launch of a library kernel on this workload:
  (bound, amount) with amount in bytes (hbm) or flops (tensor)."""
  n, m = sizes["n"], sizes["m"]
  c, k, co = sizes["cin"], sizes["k"], sizes["cout"]
  ck = c * k
  if name in ("basis_proj_split", "basis_proj_split_mma", "basis_proj_fwd_tcu"):
    # basis rows + neighbor ids, every feature row once, ranges, the projection
    return "hbm", m * (4 * k + 8) + n * 4 * c + n * 4 + n * ck * 4
  if name in ("basis_proj_grads", "basis_proj_grads_mma", "basis_proj_grads_tc",
              "basis_proj_grads_tcu"):
    return "hbm", n * ck * 4 + m * (4 * k + 8) + n * 4 * c + n * 4 + m * 4 * k + n * 4 * c
  if name in ("gemm_bf16x3_k_mn", "gemm_bf16x3_mn_k_t", "gemm_bf16x3_mn_k_scatter"):  # out = X W
    return "tensor", 2.0 * n * ck * co
  if name in ("gemm_bf16x3_k_k", "gemm_bf16x3_k_k_image", "gemm_bf16x3_k_mn_image",
              "gemm_bf16x3_mn_k_image"):  # dX = dOut W^T (4-byte output dominates)
    return "hbm", n * co * 4 + ck * co * 4 + n * ck * 4
  if name == "gemm_bf16x3_mn_mn":     # dW = X^T dOut
    return "tensor", 2.0 * n * ck * co
  if name == "find_neighbors_fill":
    return "hbm", n * 36 + m * 8
  if name == "find_neighbors_fill_fused":     # both forms of the list
    return "hbm", n * 40 + m * 16
  if name == "find_neighbors_count":
    return "hbm", n * 36
  if name == "compute_pdf":
    return "hbm", n * 20 + m * 8
  if name == "kernel_basis":          # ids, two point gathers, density, the 4K-byte row
    return "hbm", m * (8 + 24 + 4 + 4 * k)
  if name == "kernel_basis_grads":
    return "hbm", m * (8 + 24 + 4 + 4 * k)
  if name == "group_plan":            # both id lists in, one row entry (id + 4 pair slots) per pair out
    return "hbm", m * (8 + 8 + 20) + n * 4
  if name == "original_neighbor_ids":
    return "hbm", m * 20
  return "hbm", None


# ----------------------------------------------------------------- clocks ----

class ClockSampler:
  """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
  FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
            "clocks_event_reasons.sw_power_cap")

  def __init__(self, index):
    self.index = index
    self.proc = None
    self.lines = []

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
           "--format=csv,noheader,nounits", "-lms", "50"],
          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except OSError:
      self.proc = None

  def _read(self):
    for line in self.proc.stdout:
      self.lines.append(line.strip())

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    sm, mx, reasons = [], None, set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.lines:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 6:
        continue
      try:
        sm.append(float(parts[0])); mx = float(parts[1])
      except ValueError:
        continue
      for nm, val in zip(names, parts[2:6]):
        if val.lower().startswith("active"):
          reasons.add(nm)
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
            "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------ CPU baseline ----

def cpu_port_step(args, pts, bid, feat, d_out, w1, b1, wf, clouds):
  """One forward+backward of the layer on `clouds` clouds through the CPU
  oracle (C + NumPy restatement of the reference path).  Returns seconds."""
  import oracle as orc
  from oracle import pylib_ref as pr
  n = clouds * args.points
  pts, bid, feat, d_out = pts[:n], bid[:n], feat[:n], d_out[:n]
  t0 = time.perf_counter()
  grid = pr.Grid(pts, bid, clouds, args.radius)
  neigh = pr.Neighborhood(grid, args.radius, pts, bid)
  pdf = neigh.get_pdf(bandwidth=0.2, mode=0)
  basis, diff, hid = pr.mcconv_basis(pts, pts, neigh, pdf, w1, b1, args.radius)
  out, x = pr.mcconv_forward(feat, basis, neigh, wf)
  d_wf, d_basis, d_feat, _ = pr.mcconv_backward(feat, basis, neigh, wf, x, d_out)
  dpre = d_basis / pdf.reshape(-1, 1) * np.where(hid > 0, 1.0, 0.2)
  _ = diff.T @ dpre
  return time.perf_counter() - t0


def use_all_host_threads():
  """Gives the CPU port every core this process may run on.  Launchers such as
  torchrun export OMP_NUM_THREADS=1, which would otherwise leave the OpenMP loops
  of the oracle and the BLAS behind NumPy on one thread."""
  import oracle as orc
  try:
    cores = len(os.sched_getaffinity(0))
  except AttributeError:
    cores = os.cpu_count() or 1
  orc.set_num_threads(cores)
  try:
    import threadpoolctl
    threadpoolctl.threadpool_limits(limits=cores)
  except Exception:  # BLAS thread count stays what the environment set
    pass
  return cores


def cpu_baseline(args, inputs, reps=1):
  import oracle as orc
  use_all_host_threads()
  clouds = max(1, min(args.cpu_sample_clouds, args.clouds))
  best = min(cpu_port_step(args, *inputs, clouds) for _ in range(reps))
  return {"value": clouds * args.points / best, "unit": UNIT, "cores": orc.num_threads(),
          "kind": "port",
          "sample": "%d of the %d clouds (%d points), one forward+backward through the C/NumPy "
                    "oracle with OpenMP and BLAS on all host threads, %.2f s"
                    % (clouds, args.clouds, clouds * args.points, best)}


def run_reference(args, rank, world):
  """The reference publishes no CPU implementation of its custom ops (they are
  GPU-only TensorFlow kernels and TensorFlow is not installed), so this arm
  times the CPU port of the same path on all host threads."""
  if rank != 0:
    return
  import oracle as orc
  orc.build()
  use_all_host_threads()
  inputs = make_inputs(args, 0)
  clouds = max(1, min(args.cpu_sample_clouds, args.clouds))
  for _ in range(min(args.warmup, 1)):
    cpu_port_step(args, *inputs, clouds)
  times = [cpu_port_step(args, *inputs, clouds) for _ in range(max(1, min(args.steps, 3)))]
  t = statistics.mean(times)
  value = clouds * args.points / t
  line = {
      "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
      "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * t,
      "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
      "data": "synthetic", "config": workload_config(args, world),
      "cpu_baseline": {"value": value, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                       "sample": "each step is %d of the %d clouds (%d points)"
                                 % (clouds, args.clouds, clouds * args.points)},
      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }
  print(json.dumps(line), flush=True)



# ------------------------------------------- the reference's own kernels -----

def run_reference_kernels(args):
  """Times the reference's own CUDA kernels (its *_kernels.cu.cc files compiled
  unchanged for sm_100a into oracle/_ref by oracle/build_ref.py, behind a plain
  CUDA device object) op by op against this library's kernels on the same GPU
  and the same seeded inputs: CUDA-event times around the kernel sequence of each
  op (second call, device buffers recycled, host copies excluded).  Prints one
  JSON line with a row per op.  --clouds / --points set the size (8 clouds fit
  the reference's [N, Cin, K] fp32 projection comfortably)."""
  import torch
  from oracle import ref_kernels as ref
  from tensorflow_graphics_point_clouds_b200 import _lib, custom_ops as ops, pc, synthetic
  if not ref.available():
    print(json.dumps({"impl": "reference-kernels",
                      "unavailable": "oracle/_ref is not built (needs the reference checkout "
                                     "at build time)"}), flush=True)
    return
  clouds, per = args.clouds, args.points

  def ours(fn, name_prefixes, reps=3):
    for _ in range(2):
      fn()
    torch.cuda.synchronize()
    _lib.profile_enable(True)
    for _ in range(reps):
      fn()
    torch.cuda.synchronize()
    rec = _lib.profile_collect()
    _lib.profile_enable(False)
    return sum(ms for n, ms in rec if n.startswith(name_prefixes)) / reps

  radius, cin, k = 0.079, 128, 16
  pts, bid = synthetic.uniform_clouds(clouds, per, seed=2)
  n = len(pts)
  rng = np.random.default_rng(0)
  t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
  cloud = pc.PointCloud(t(pts), t(bid), clouds)
  grid = pc.Grid(cloud, radius)
  neigh = pc.Neighborhood(grid, radius)               # self neighborhood, sorted order
  g_np = dict(sp=grid._sorted_points.cpu().numpy(), sb=grid._sorted_batch_ids.cpu().numpy(),
              sk=grid._sorted_keys.cpu().numpy(), ds=grid.get_DS().cpu().numpy(),
              nc=grid._num_cells.cpu().numpy(), smin=grid._scaled_aabb_min.cpu().numpy(),
              ic=grid._inv_cell_sizes.cpu().numpy())
  inv_r = np.repeat(F32(1) / F32(radius), 3)
  inv_bw = np.repeat(F32(5.0), 3)
  nb = neigh._neighbors.cpu().numpy(); rg = neigh._samples_neigh_ranges.cpu().numpy()
  m = len(nb)
  rows = []

  def twice(fn):     # the second call reuses the harness' device buffers: kernels only
    fn()
    return fn()

  _, ms = twice(lambda: ref.compute_keys(pts, bid, g_np["smin"], g_np["nc"], g_np["ic"]))
  mine = ours(lambda: ops.compute_keys(cloud._points, cloud._batch_ids, grid._scaled_aabb_min,
                                       grid._num_cells, grid._inv_cell_sizes), ("compute_keys",))
  rows.append(("ComputeKeys", ms, mine))
  _, ms = twice(lambda: ref.build_grid_ds(g_np["sk"], g_np["nc"], clouds))
  mine = ours(lambda: ops.build_grid_ds(grid._sorted_keys, grid._num_cells, grid._num_cells_host,
                                        clouds), ("build_grid_ds",))
  rows.append(("BuildGridDs", ms, mine))
  _, _, ms = twice(lambda: ref.find_neighbors(g_np["sp"], g_np["sb"], g_np["sp"], g_np["sk"],
                                              g_np["ds"], g_np["nc"], g_np["smin"], g_np["ic"],
                                              inv_r, capacity=m + 16))
  mine = ours(lambda: pc.Neighborhood(grid, radius)._neighbors, ("find_neighbors", "scan_i32"))
  rows.append(("FindNeighbors", ms, mine))
  _, _, ms = twice(lambda: ref.compute_pdf(g_np["sp"], nb, rg, inv_bw, inv_r, 0))
  mine = ours(lambda: ops.compute_pdf(grid._sorted_points, neigh._neighbors,
                                      neigh._samples_neigh_ranges, t(inv_bw), t(inv_r), 0),
              ("compute_pdf",))
  rows.append(("ComputePdf", ms, mine))
  basis = rng.standard_normal((m, k), dtype=F32)
  feat = rng.standard_normal((n, cin), dtype=F32)
  out, _, _, ms = twice(lambda: ref.basis_proj(basis, feat, nb, rg))
  tb, tf = t(basis), t(feat)
  mine = ours(lambda: ops.basis_proj(tb, tf, neigh._neighbors, neigh._samples_neigh_ranges),
              ("basis_proj", "split_features"))
  rows.append(("BasisProj [%d,%d,%d]" % (n, cin, k), ms, mine))
  _, _, _, ms = twice(lambda: ref.sampling(g_np["sp"], g_np["sb"], g_np["sk"], g_np["nc"], nb, rg, 0))
  mine = ours(lambda: pc.sample(neigh, "poisson"), ("sampling", "scan_i32"))
  rows.append(("Sampling (Poisson)", ms, mine))

  line = {"impl": "reference-kernels", "unit": "ms", "data": "synthetic",
          "config": {"workload": "%d clouds x %d points uniform in [0,1)^3, radius %.3f, Cin %d, "
                                 "K %d" % (clouds, per, radius, cin, k), "neighbor_pairs": int(m)},
          "ops": [{"op": name, "reference_kernels_ms": r, "this_library_ms": o,
                   "ratio": (r / o if o > 0 else None)} for name, r, o in rows]}
  print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- our arm ----

class LayerRun:
  """One rank's inputs on the device and the step that runs on them."""

  def __init__(self, args, inputs, clouds, dev, world):
    import torch
    from tensorflow_graphics_point_clouds_b200 import mcconv
    pts, bid, feat, d_out, w1, b1, wf = inputs
    self.args, self.clouds, self.dev, self.world = args, clouds, dev, world
    self.n = pts.shape[0]
    self.host = {k: torch.from_numpy(np.ascontiguousarray(v)).pin_memory() for k, v in
                 dict(pts=pts, bid=bid, feat=feat, d_out=d_out).items()}
    self.dev_in = {k: v.to(dev) for k, v in self.host.items()}
    self.layer = mcconv.MCConv(torch.from_numpy(w1).to(dev), torch.from_numpy(b1).to(dev),
                               torch.from_numpy(wf).to(dev), args.cin)
    self.pairs = 0

  def step(self, x, allreduce=True):
    from tensorflow_graphics_point_clouds_b200 import pc
    from tensorflow_graphics_point_clouds_b200 import dist as tdist
    # cell counts are the maximum over the whole batch, i.e. over all shards
    cloud = pc.PointCloud(x["pts"], x["bid"], self.clouds,
                          num_cells_reduce=tdist.allreduce_max_ if self.world > 1 else None)
    out = self.layer.forward(x["feat"], cloud, cloud, self.args.radius)
    self.pairs = int(self.layer._saved[0].num_pairs)
    dfeat, dw1, db1, dwf = self.layer.backward(x["d_out"])
    if allreduce:
      tdist.allreduce_sum_([dwf, dw1, db1])   # the path's only exchange step
    return out, dfeat, dwf, dw1, db1


def shard_check(args, full_inputs, run, first_point, dev, world):
  """Every rank runs the WHOLE batch once on its own GPU and compares its shard's
  results with the matching slices: neighbor ranges and lists (re-based) bit for
  bit, output rows and feature gradients within 1e-4 of max(|ref|, rms), and the
  all-reduced weight gradients with those of the whole batch.  Returns the list
  of mismatches (empty = ok)."""
  import torch
  from tensorflow_graphics_point_clouds_b200 import dist as tdist
  whole = LayerRun(args, full_inputs, args.clouds, dev, 1)
  ref = whole.step(whole.dev_in, allreduce=False)
  ref_nb = whole.layer._saved[0]
  got = run.step(run.dev_in, allreduce=True)
  nb = run.layer._saved[0]
  lo, hi = first_point, first_point + run.n
  bad = []

  def rel(a, b):
    a, b = a.double(), b.double()
    scale = torch.maximum(b.abs(), b.pow(2).mean().sqrt())
    return float(((a - b).abs() / scale).max())

  ref_ranges = ref_nb._samples_neigh_ranges
  pair_lo = int(ref_ranges[lo - 1]) if lo > 0 else 0
  pair_hi = int(ref_ranges[hi - 1])
  if not torch.equal(nb._samples_neigh_ranges, ref_ranges[lo:hi] - pair_lo):
    bad.append("ranges")
  ids = ref_nb._original_neigh_ids[pair_lo:pair_hi] - lo
  if nb._original_neigh_ids.shape != ids.shape or not torch.equal(nb._original_neigh_ids, ids):
    bad.append("neighbor lists")
  for name, a, b in (("out", got[0], ref[0][lo:hi]), ("dfeat", got[1], ref[1][lo:hi]),
                     ("dW", got[2], ref[2]), ("dw1", got[3], ref[3]), ("db1", got[4], ref[4])):
    err = rel(a, b)
    if not err <= (2e-4 if name in ("dw1", "db1") else 1e-4):
      bad.append("%s (rel err %.2e)" % (name, err))
  del whole
  torch.cuda.empty_cache()
  return bad


def timed_steps(run, steps, barrier, collect_kernels):
  """Device-resident timing of `steps` steps: (ms per step on this rank, kernel records)."""
  import torch
  from tensorflow_graphics_point_clouds_b200 import _lib
  barrier()
  if collect_kernels:
    _lib.profile_enable(True)
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(steps):
    run.step(run.dev_in)
  e1.record()
  barrier()
  records = []
  if collect_kernels:
    records = _lib.profile_collect()
    _lib.profile_enable(False)
  return e0.elapsed_time(e1) / steps, records


def bind_near_gpu(index):
  """Restricts this process to the host cores NVML lists as nearest to GPU `index`
  (its NUMA node), so that the pinned buffers of the end-to-end variant are first
  touched there instead of wherever the launcher happened to start the rank.
  Reads NVML only.  Returns the number of cores kept, or None if nothing changed
  (no NVML, no NUMA information, or the cores lie outside this process's set)."""
  try:
    import pynvml
    pynvml.nvmlInit()
    handle = pynvml.nvmlDeviceGetHandleByIndex(index)
    n = max(os.cpu_count() or 1, max(os.sched_getaffinity(0)) + 1)
    words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n + 63) // 64)
    near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
    allowed = os.sched_getaffinity(0)
    keep = near & allowed
    if keep and keep != allowed:
      os.sched_setaffinity(0, keep)
      return len(keep)
  except Exception:
    pass
  return None


def e2e_steps(run, steps, barrier):
  """End to end: every step copies its inputs from pinned host memory and its
  results back to pinned host memory.  The copies run on two copy streams so that
  the upload of step i+1 and the download of step i-1 overlap the kernels of step i
  (two sets of device input buffers and of host output buffers).
  Returns (ms per step on this rank, bytes up per step, bytes down per step)."""
  import torch
  host, dev = run.host, run.dev
  h2d = sum(v.numel() * v.element_size() for v in host.values())
  main = torch.cuda.current_stream()
  s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
  dev_bufs = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(2)]
  ev_in = [torch.cuda.Event() for _ in range(2)]
  ev_free = [torch.cuda.Event() for _ in range(2)]   # step that used the buffer set has finished
  ev_out = [torch.cuda.Event() for _ in range(2)]    # download into the host set has finished
  out_host = [None, None]
  d2h = [0]

  def upload(i):
    b = i % 2
    with torch.cuda.stream(s_in):
      s_in.wait_event(ev_free[b])
      for k, v in host.items():
        dev_bufs[b][k].copy_(v, non_blocking=True)
      ev_in[b].record(s_in)

  def run_one(i):
    b = i % 2
    main.wait_event(ev_in[b])
    res = run.step(dev_bufs[b])
    ev_free[b].record(main)
    done = torch.cuda.Event()
    done.record(main)
    if out_host[b] is None:
      out_host[b] = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res]
      d2h[0] = sum(r.numel() * r.element_size() for r in res)
    with torch.cuda.stream(s_out):
      s_out.wait_event(done)
      s_out.wait_event(ev_out[b])
      for h, r in zip(out_host[b], res):
        r.record_stream(s_out)
        h.copy_(r, non_blocking=True)
      ev_out[b].record(s_out)

  def loop(count):
    upload(0)
    for i in range(count):
      if i + 1 < count:
        upload(i + 1)
      run_one(i)
    main.wait_stream(s_out)

  for b in range(2):
    ev_free[b].record(main)
    ev_out[b].record(main)
  loop(2)
  barrier()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  loop(steps)
  e1.record()
  barrier()
  return e0.elapsed_time(e1) / steps, h2d, d2h[0]


def run_ours(args, rank, local_rank, world):
  import torch
  import torch.distributed as dist
  from tensorflow_graphics_point_clouds_b200 import build
  from tensorflow_graphics_point_clouds_b200 import dist as tdist

  if not torch.cuda.is_available():
    raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
  build.build()
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)

  def barrier():
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
      torch.cuda.synchronize()

  # several ranks on one host: keep each near its own GPU before any pinned buffer exists
  near_cores = bind_near_gpu(local_rank) if world > 1 else None
  strong = args.scaling == "strong"
  full_inputs = make_inputs(args, 0 if strong else rank)
  if strong:
    inputs, clouds, first_point = shard_inputs(full_inputs, args, rank, world)
  else:
    inputs, clouds, first_point = full_inputs, args.clouds, 0
  run = LayerRun(args, inputs, clouds, dev, world)
  n_global = args.clouds * args.points * (1 if strong else world)
  sizes = {"n": run.n, "m": 0, "cin": args.cin, "k": args.hidden, "cout": args.cout}

  # nvidia-smi needs a few hundred ms to deliver its first sample: start it
  # before the warm-up so that it is sampling (under the same load) throughout
  # the timed region
  sampler = ClockSampler(local_rank)
  sampler.start()
  check = None
  if strong and world > 1 and not args.no_shard_check:
    bad = shard_check(args, full_inputs, run, first_point, dev, world)
    flag = torch.tensor([0 if bad else 1], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    check = "ok" if int(flag.item()) == 1 else "FAILED"
    if bad:
      sys.stderr.write("shard_check rank %d: mismatch in %s\n" % (rank, ", ".join(bad)))
    if rank == 0:
      sys.stderr.write("shard_check: %s\n" % check)
  for _ in range(max(args.warmup, 3)):
    run.step(run.dev_in)
  run.layer._op.check_status()

  # ---- device-resident timing
  ms_rank, records = timed_steps(run, args.steps, barrier, True)
  clocks = sampler.stop()
  run.layer._op.check_status()
  sizes["m"] = run.pairs
  ms_per_step = tdist.max_over_ranks(ms_rank, dev)
  pairs_global = run.pairs
  if world > 1:
    t = torch.tensor([run.pairs], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    pairs_global = int(t.item())

  # ---- end to end: host buffers in, host buffers out, every step
  e2e = None
  if not args.no_e2e:
    e2e_rank, h2d, d2h = e2e_steps(run, args.steps, barrier)
    e2e_ms = tdist.max_over_ranks(e2e_rank, dev)
    per_rank = torch.tensor([h2d / (e2e_rank * 1e-3) / 1e9, d2h / (e2e_rank * 1e-3) / 1e9],
                            dtype=torch.float64, device=dev)
    if world > 1:
      gathered = [torch.zeros_like(per_rank) for _ in range(world)]
      dist.all_gather(gathered, per_rank)
    else:
      gathered = [per_rank]
    e2e = {"value": n_global / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "h2d_gbs_per_rank": [round(float(g[0]), 2) for g in gathered],
           "d2h_gbs_per_rank": [round(float(g[1]), 2) for g in gathered],
           "host_cores_near_gpu": near_cores,
           "note": "bytes per step are this rank's; GB/s = bytes / the rank's own step time, both "
                   "directions in flight at once with the kernels; host_cores_near_gpu: cores "
                   "rank 0 was bound to before its pinned buffers were allocated (null: no "
                   "NUMA information, nothing bound)"}

  # ---- weak scaling beside a strong multi-GPU run: every rank its own batch
  weak = None
  if strong and world > 1:
    del run
    torch.cuda.empty_cache()
    wrun = LayerRun(args, make_inputs(args, rank), args.clouds, dev, world)
    for _ in range(3):
      wrun.step(wrun.dev_in)
    wms, _ = timed_steps(wrun, args.steps, barrier, False)
    wms = tdist.max_over_ranks(wms, dev)
    weak = {"value": args.clouds * args.points * world / (wms * 1e-3), "unit": UNIT,
            "ms_per_step": wms, "clouds_per_gpu": args.clouds, "scaling": "weak"}
    del wrun
    torch.cuda.empty_cache()

  if rank == 0:
    peaks = measured_peaks()
    agg = {}
    for name, kms in records:
      a = agg.setdefault(name, [0, 0.0])
      a[0] += 1; a[1] += kms
    total_kernel_ms = sum(v[1] for v in agg.values())
    kernels = {k: {"launches_per_step": v[0] / args.steps, "ms_per_step": v[1] / args.steps}
               for k, v in sorted(agg.items(), key=lambda kv: -kv[1][1])}
    # the dominant kernel among those with a work model
    modelled = {k: v for k, v in agg.items() if kernel_model(k, sizes)[1] is not None}
    top = max(modelled.items(), key=lambda kv: kv[1][1])[0]
    bound, amount = kernel_model(top, sizes)
    avg_ms = agg[top][1] / agg[top][0]
    if bound == "hbm":
      achieved = amount / (avg_ms * 1e-3) / 1e9
      peak, runit = peaks["hbm_gbs"], "GB/s"
    else:
      achieved = amount / (avg_ms * 1e-3) / 1e12
      peak, runit = peaks["bf16_tflops"], "TFLOP/s"
    roofline = {"kernel": top, "bound": bound, "achieved": achieved, "peak": peak, "unit": runit,
                "frac": achieved / peak, "traffic": (NCU_TRAFFIC_BYTES_PER_POINT[top] * sizes["n"]
                            if top in NCU_TRAFFIC_BYTES_PER_POINT else None),
                "avg_launch_ms": avg_ms, "peak_source": peaks["source"],
                "note": "tensor-bound kernels issue 3 bf16 passes per algorithmic flop"
                        if bound == "tensor" else "algorithmic bytes / launch time"}
    # every modelled kernel against its own bound (rank 0's launches)
    per_kernel = {}
    for name, v in modelled.items():
      kb, amt = kernel_model(name, sizes)
      k_ms = v[1] / v[0]
      if kb == "hbm":
        per_kernel[name] = {"bound": "hbm", "frac": amt / (k_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
      else:
        per_kernel[name] = {"bound": "tensor", "frac_algorithmic":
                            amt / (k_ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                            "frac_issued": 3 * amt / (k_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    line = {
        "metric": METRIC, "value": n_global / (ms_per_step * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, world), "clocks": clocks, "e2e": e2e,
        "gpu_launches": int(sum(v[0] for v in agg.values())),
        "roofline": roofline,
        "kernels": kernels,
        "kernel_roofline_fracs": per_kernel,
        "kernel_ms_per_step": total_kernel_ms / args.steps,
        "neighbor_pairs": pairs_global,
        "neighbor_pairs_per_layer_step_per_s": pairs_global / (ms_per_step * 1e-3),
    }
    if check is not None:
      line["shard_check"] = check
    if weak is not None:
      line["weak_scaling"] = weak
    if world == 1 and not args.no_cpu_baseline:
      import oracle as orc
      orc.build()
      line["cpu_baseline"] = cpu_baseline(args, full_inputs)
    if not args.no_side and args.workload == "mcconv":
      line["side"] = {}
      for wl in ("neighbors", "hierarchy"):
        side_args = argparse.Namespace(**vars(args))
        side_args.workload, side_args.steps, side_args.warmup = wl, args.side_steps, 3
        line["side"][wl] = side_workload_line(side_args, local_rank)
    print(json.dumps(line), flush=True)
  if world > 1:
    barrier()
    dist.destroy_process_group()


# ------------------------------------------------- secondary workloads -------

SIDE_MODELS = {
    # algorithmic bytes per launch: n points / samples, m neighbor pairs, s samples out
    "compute_aabb": lambda n, m, s: n * 16 ,
    "compute_keys": lambda n, m, s: n * 24,
    "sort_radix": lambda n, m, s: n * 36,
    "sort_gather": lambda n, m, s: n * 36,
    "build_grid_ds": lambda n, m, s: n * 8,
    "find_neighbors_count": lambda n, m, s: n * 36,
    "find_neighbors_fill": lambda n, m, s: n * 36 + m * 8,
    "find_neighbors_fill_fused": lambda n, m, s: n * 40 + m * 16,
    "compute_pdf": lambda n, m, s: n * 20 + m * 8,
    "sampling_poisson_pass": lambda n, m, s: (n * 8 + m * 12) / 8.0,
    "sampling_store_poisson": lambda n, m, s: n * 8 + s * 20,
    "sampling_cell_average": lambda n, m, s: n * 20 + s * 16,
}


def run_side_workload(args):
  print(json.dumps(side_workload_line(args, 0)), flush=True)


def side_workload_line(args, device_index):
  """Grid / neighbor / pdf (surface clouds) or the sampling hierarchy (Gaussian
  mixtures) on one GPU: per-kernel time and algorithmic GB/s against the HBM peak."""
  import torch
  from tensorflow_graphics_point_clouds_b200 import _lib, build, pc, synthetic
  if not torch.cuda.is_available():
    raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
  build.build()
  dev = torch.device("cuda", device_index)
  peaks = measured_peaks()
  if args.workload == "neighbors":
    pts, bid = synthetic.surface_clouds(16, seed=1)
    batch, radii = 16, [0.05]
  else:
    pts, bid = synthetic.gaussian_mixture_clouds(8, 100000, seed=3)
    batch, radii = 8, [0.025, 0.05, 0.1, 0.2]
  tp, tb = torch.from_numpy(pts).to(dev), torch.from_numpy(bid).to(dev)
  sizes = []   # (n, m, s) per level, in launch order

  def step(record):
    cloud = pc.PointCloud(tp, tb, batch)
    if args.workload == "neighbors":
      neigh = pc.grid_neighborhood(cloud, radii[0])
      neigh.compute_pdf(bandwidth=0.2, mode=0)
      if record:
        sizes.append((tp.shape[0], neigh._neighbors.shape[0], 0))
      return neigh._neighbors.shape[0]
    pairs = 0
    for mode in ("poisson", "average"):
      cur = cloud
      for r in radii:
        neigh = pc.grid_neighborhood(cur, r)
        nxt, _ = pc.sample(neigh, mode)
        if record:
          sizes.append((cur._points.shape[0], neigh._neighbors.shape[0], nxt._points.shape[0]))
        pairs += neigh._neighbors.shape[0]
        cur = nxt
    return pairs

  for _ in range(max(args.warmup, 3)):
    step(False)
  torch.cuda.synchronize()
  pairs = step(True)
  sampler = ClockSampler(device_index)
  sampler.start()
  _lib.profile_enable(True)
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(args.steps):
    step(False)
  e1.record()
  torch.cuda.synchronize()
  records = _lib.profile_collect()
  _lib.profile_enable(False)
  clocks = sampler.stop()
  ms = e0.elapsed_time(e1) / args.steps
  per_step = len(records) // args.steps
  # attribute every launch to the level (point count, pair count) it worked on
  agg = {}
  counters = {}
  for idx, (name, kms) in enumerate(records):
    pos_in_step = counters.get(name, 0)
    counters[name] = pos_in_step + 1
    a = agg.setdefault(name, [0, 0.0, 0.0])
    a[0] += 1; a[1] += kms
    model = SIDE_MODELS.get(name)
    if model is not None and sizes:
      launches_per_step = sum(1 for n2, _ in records[:per_step] if n2 == name) or 1
      k = pos_in_step % launches_per_step
      per_level = 8 if name == "sampling_poisson_pass" else 1
      if name in ("sampling_store_poisson",):
        lvl = k                                   # Poisson levels come first
      elif name == "sampling_cell_average":
        lvl = len(radii) + k
      else:
        lvl = min(k // per_level, len(sizes) - 1)
      n, m, so = sizes[min(lvl, len(sizes) - 1)]
      a[2] += model(n, m, so)
  kernels = {}
  for name, (cnt, tot, bytes_) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
    entry = {"launches_per_step": cnt / args.steps, "ms_per_step": tot / args.steps}
    if bytes_ > 0:
      gbs = bytes_ / (tot * 1e-3) / 1e9
      entry["algorithmic_gbs"] = gbs
      entry["frac_of_hbm_peak"] = gbs / peaks["hbm_gbs"]
    kernels[name] = entry
  n_pts = tp.shape[0]
  line = {
      "metric": "neighbor_pairs_per_s", "value": pairs / (ms * 1e-3), "unit": "pairs/s",
      "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
      "higher_is_better": True, "dtype": "f32", "data": "synthetic",
      "config": {"workload": args.workload, "points": int(n_pts), "neighbor_pairs": int(pairs),
                 "radii": radii, "levels": [list(map(int, x)) for x in sizes]},
      "clocks": clocks, "kernels": kernels, "peak_hbm_gbs": peaks["hbm_gbs"],
      "peak_source": peaks["source"],
  }
  return line


def run_classifier_workload(args):
  """Forward pass of the small classification network (MCConv with 4 kernel MLPs
  of 8 units per level; level layout by --classifier-preset) on 32 clouds of 1024
  points on one GPU: time per batch and the kernels it spends it in."""
  import torch
  from tensorflow_graphics_point_clouds_b200 import _lib, build, classifier, synthetic
  if not torch.cuda.is_available():
    raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
  build.build()
  dev = torch.device("cuda", 0)
  clouds, points = 32, 1024
  preset = classifier.PRESETS[args.classifier_preset]
  radii = list(preset["radii"])
  pts, bid = synthetic.unit_sphere_shapes(clouds, points, seed=4)
  tp, tb = torch.from_numpy(pts).to(dev), torch.from_numpy(bid).to(dev)
  feat = torch.ones((len(pts), 1), dtype=torch.float32, device=dev)
  weights = synthetic.small_classifier_weights(40, preset["feature_sizes"],
                                               head_layers=preset["head_layers"])
  net = classifier.SmallClassifier(weights, radii, dev, preset["pool_before_head"])
  sampler = ClockSampler(0)
  sampler.start()
  for _ in range(max(args.warmup, 3)):
    net.forward(tp, tb, clouds, feat)
  torch.cuda.synchronize()
  _lib.profile_enable(True)
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(args.steps):
    net.forward(tp, tb, clouds, feat)
  e1.record()
  torch.cuda.synchronize()
  records = _lib.profile_collect()
  _lib.profile_enable(False)
  clocks = sampler.stop()
  ms = e0.elapsed_time(e1) / args.steps
  agg = {}
  for name, kms in records:
    a = agg.setdefault(name, [0, 0.0])
    a[0] += 1; a[1] += kms
  kernels = {name: {"launches_per_step": c / args.steps, "ms_per_step": t / args.steps}
             for name, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])}
  line = {
      "metric": "classifier_forward_points_per_s", "value": clouds * points / (ms * 1e-3),
      "unit": "points/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
      "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
      "config": {"workload": "classifier", "preset": args.classifier_preset, "clouds": clouds,
                 "points_per_cloud": points, "radii": [float(r) for r in radii],
                 "feature_sizes": list(preset["feature_sizes"])},
      "clocks": clocks, "kernels": kernels,
      "kernel_ms_per_step": sum(v["ms_per_step"] for v in kernels.values()),
  }
  print(json.dumps(line), flush=True)


def main():
  args = parse_args()
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  if args.workload == "classifier":
    if rank == 0:
      run_classifier_workload(args)
  elif args.workload != "mcconv":
    if rank == 0:
      run_side_workload(args)
  elif args.impl == "reference-kernels":
    if rank == 0:
      run_reference_kernels(args)
  elif args.impl == "reference":
    run_reference(args, rank, world)
  else:
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
  main()
