// Poisson-disk and cell-average sampling on the sorted grid.
//
// Both modes start from the runs of equal keys (one run = one occupied cell),
// found with a flag + scan + ordered compaction, so the cells come out in
// ascending first-point index (the reference compacts with atomicAdd and gets
// an arbitrary order, store_unique_keys_kernels.cu.cc:36-56).
//
// Poisson disk (count_sampling_pd_kernels.cu.cc:42-108, 157-180): 2^D passes,
// pass p takes the cells whose coordinate d has parity bit d of p; inside a
// cell the points are visited in sorted order and a point is taken iff none of
// its neighbors is taken.  Here one warp owns a cell and its lanes test 32
// neighbors per step, where the reference walks both loops with one thread.
// The taken points are then compacted in ascending index with a scan (the
// reference: atomicAdd, store_sampled_pts_kernels.cu.cc:42-69).
#include "common.cuh"

namespace tfgpc {

constexpr int kSmpThreads = 256;
constexpr int kCellBits = 4096;  // points of one cell tracked in the per-warp bit set

struct SamplingWs {
  int32_t* flags;      // [n] 1 where a run of equal keys starts
  int32_t* run_idx;    // [n] inclusive scan of flags
  int32_t* starts;     // [n] first index of every run, ascending
  int32_t* used;       // [n] Poisson: 1 if the point is taken
  int32_t* used_scan;  // [n] inclusive scan of used
  int64_t* block_sums;
  int64_t* totals;     // [0] number of runs, [1] number of taken points
};

static size_t sampling_ws_bytes(int64_t n) {
  if (n < 0) n = 0;
  return 5 * align_up((size_t)n * sizeof(int32_t), 256) +
         align_up((size_t)scan_block_sums_elems(n) * sizeof(int64_t), 256) + 256;
}

static SamplingWs carve(void* ws, int64_t n) {
  SamplingWs w;
  char* p = (char*)ws;
  size_t arr = align_up((size_t)(n > 0 ? n : 0) * sizeof(int32_t), 256);
  w.flags = (int32_t*)p; p += arr;
  w.run_idx = (int32_t*)p; p += arr;
  w.starts = (int32_t*)p; p += arr;
  w.used = (int32_t*)p; p += arr;
  w.used_scan = (int32_t*)p; p += arr;
  w.block_sums = (int64_t*)p;
  p += align_up((size_t)scan_block_sums_elems(n) * sizeof(int64_t), 256);
  w.totals = (int64_t*)p;
  return w;
}

__global__ void flag_runs_kernel(int64_t n, const int64_t* __restrict__ keys,
                                 int32_t* __restrict__ flags) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) flags[i] = (i == 0 || __ldg(keys + i) != __ldg(keys + i - 1)) ? 1 : 0;
}

__global__ void compact_runs_kernel(int64_t n, const int32_t* __restrict__ flags,
                                    const int32_t* __restrict__ run_idx,
                                    int32_t* __restrict__ starts) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && flags[i]) starts[run_idx[i] - 1] = (int32_t)i;
}

template <int D>
__global__ void __launch_bounds__(kSmpThreads)
poisson_pass_kernel(int pass, int64_t n, const int64_t* __restrict__ num_runs,
                    const int32_t* __restrict__ starts, const int64_t* __restrict__ keys,
                    const int32_t* __restrict__ num_cells, const int2* __restrict__ neigh,
                    const int32_t* __restrict__ ranges, int32_t* used) {
  __shared__ uint32_t bits_all[(kSmpThreads / 32) * (kCellBits / 32)];
  uint32_t* bits = bits_all + (threadIdx.x >> 5) * (kCellBits / 32);
  const int64_t runs = *num_runs;
  const int lane = lane_id();
  int nc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) nc[d] = __ldg(num_cells + d);
  const int64_t warps = ((int64_t)gridDim.x * kSmpThreads) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * kSmpThreads + threadIdx.x) >> 5; r < runs; r += warps) {
    const int begin = __ldg(starts + r);
    const int end = (r + 1 < runs) ? __ldg(starts + r + 1) : (int)n;
    int64_t aux = __ldg(keys + begin);
    bool mine = true;
#pragma unroll
    for (int d = D - 1; d >= 0; --d) {  // grid_utils.h:110-125
      int c = (int)(aux % nc[d]);
      aux /= nc[d];
      mine = mine && ((c & 1) == ((pass >> d) & 1));
    }
    if (!mine) continue;
    // Flags of points outside this cell cannot change during this pass (cells of
    // equal parity are never neighbors), so they are read through the caches;
    // the flags of the cell's own points are kept in a per-warp bit set in
    // shared memory (cells of up to kCellBits points; larger cells fall back to
    // uncached global reads), which takes the L2 round trip out of the
    // point-after-point dependency chain.
    const bool local = end - begin <= kCellBits;
    if (local)
      for (int i = lane; i < kCellBits / 32; i += 32) bits[i] = 0u;
    __syncwarp();
    for (int q = begin; q < end; ++q) {
      const int a = q ? __ldg(ranges + q - 1) : 0;
      const int e = __ldg(ranges + q);
      bool taken_nb = false;
      for (int base = a; base < e && !taken_nb; base += 32) {
        const int m = base + lane;
        bool hit = false;
        if (m < e) {
          const int j = __ldg(&neigh[m].x);
          if (j >= begin && j < end) {
            hit = local ? ((bits[(j - begin) >> 5] >> ((j - begin) & 31)) & 1u) != 0u
                        : __ldcg(used + j) != 0;
          } else if (j >= 0 && j < n) {
            hit = used[j] != 0;
          }
        }
        taken_nb = __any_sync(0xffffffffu, hit);
      }
      if (!taken_nb && lane == 0) {
        __stcg(used + q, 1);
        if (local) bits[(q - begin) >> 5] |= 1u << ((q - begin) & 31);
      }
      __syncwarp();
    }
  }
}

// The same pass for SYMMETRIC neighbor lists (j is listed for i exactly when i
// is listed for j, as in every self neighborhood found without a neighbor
// limit).  "None of my neighbors is taken" then equals "no taken point lists
// me", so a taken point marks its whole list as blocked and every other point
// costs one flag read instead of a walk over its list: the work drops from the
// sum of all list lengths to the lists of the taken points, and the
// point-after-point chain inside a crowded cell to one flag read per 32 points.
// During a pass only the warp that owns a cell writes flags of that cell's
// points (cells of equal parity are never neighbors), so the flags of the 32
// points in flight are kept in a register mask and patched from the marks the
// warp itself makes.
template <int D>
__global__ void __launch_bounds__(kSmpThreads)
poisson_pass_symmetric_kernel(int pass, int64_t n, const int64_t* __restrict__ num_runs,
                              const int32_t* __restrict__ starts,
                              const int64_t* __restrict__ keys,
                              const int32_t* __restrict__ num_cells,
                              const int2* __restrict__ neigh, const int32_t* __restrict__ ranges,
                              int32_t* __restrict__ used, int32_t* blocked) {
  const int64_t runs = *num_runs;
  const int lane = lane_id();
  int nc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) nc[d] = __ldg(num_cells + d);
  const int64_t warps = ((int64_t)gridDim.x * kSmpThreads) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * kSmpThreads + threadIdx.x) >> 5; r < runs; r += warps) {
    const int begin = __ldg(starts + r);
    const int end = (r + 1 < runs) ? __ldg(starts + r + 1) : (int)n;
    int64_t aux = __ldg(keys + begin);
    bool mine = true;
#pragma unroll
    for (int d = D - 1; d >= 0; --d) {  // grid_utils.h:110-125
      int c = (int)(aux % nc[d]);
      aux /= nc[d];
      mine = mine && ((c & 1) == ((pass >> d) & 1));
    }
    if (!mine) continue;
    for (int q0 = begin; q0 < end; q0 += 32) {
      const int q = q0 + lane;
      unsigned open = __ballot_sync(0xffffffffu, q < end && __ldcg(blocked + q) == 0);
      while (open) {
        const int t = __ffs(open) - 1;
        const int taken = q0 + t;
        open &= open - 1u;
        if (lane == 0) used[taken] = 1;
        const int a = taken ? __ldg(ranges + taken - 1) : 0;
        const int e = __ldg(ranges + taken);
        unsigned marked = 0u;
        for (int m = a + lane; m < e; m += 32) {
          const int j = __ldg(&neigh[m].x);
          if (j >= 0 && j < n && j != taken) {
            __stcg(blocked + j, 1);
            if (j >= q0 && j < q0 + 32) marked |= 1u << (j - q0);
          }
        }
        open &= ~__reduce_or_sync(0xffffffffu, marked);
      }
      __syncwarp();  // the marks of this group are visible to the next group's reads
    }
  }
}

template <int D>
__global__ void store_poisson_kernel(int64_t n, const int32_t* __restrict__ used,
                                     const int32_t* __restrict__ used_scan,
                                     const float* __restrict__ pts,
                                     const int32_t* __restrict__ batch_ids,
                                     float* __restrict__ pts_out, int32_t* __restrict__ batch_out,
                                     int32_t* __restrict__ idx_out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n || !used[i]) return;
  const int64_t o = used_scan[i] - 1;
#pragma unroll
  for (int d = 0; d < D; ++d) pts_out[o * D + d] = __ldg(pts + i * D + d);
  batch_out[o] = __ldg(batch_ids + i);
  idx_out[o] = (int32_t)i;
}

// One thread per occupied cell: sequential fp32 sum of its points / count and
// batch = key / prod(num_cells) (sampling_avg_kernels.cu.cc:43-88).
template <int D>
__global__ void cell_average_kernel(int64_t n, int64_t runs, const int32_t* __restrict__ starts,
                                    const float* __restrict__ pts,
                                    const int64_t* __restrict__ keys,
                                    const int32_t* __restrict__ num_cells,
                                    float* __restrict__ pts_out, int32_t* __restrict__ batch_out) {
  int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= runs) return;
  const int begin = __ldg(starts + r);
  const int end = (r + 1 < runs) ? __ldg(starts + r + 1) : (int)n;
  int64_t total_cells = 1;
#pragma unroll
  for (int d = 0; d < D; ++d) total_cells *= __ldg(num_cells + d);
  float acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.0f;
  for (int q = begin; q < end; ++q)
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] += __ldg(pts + (int64_t)q * D + d);
  const float cnt = (float)(end - begin);
#pragma unroll
  for (int d = 0; d < D; ++d) pts_out[r * D + d] = acc[d] / cnt;
  batch_out[r] = (int32_t)(__ldg(keys + begin) / total_cells);
}

static int check_smp_args(int D, int mode, int64_t n, int64_t M) {
  TFGPC_REQUIRE(valid_dims(D), "SamplingOp expects a valid number of dimension (got %d)", D);
  TFGPC_REQUIRE(mode == 0 || mode == 1, "SamplingOp expects mode 0 (poisson) or 1 (average)");
  TFGPC_REQUIRE(n >= 0 && n < (int64_t)INT32_MAX && M >= 0 && M <= (int64_t)INT32_MAX,
                "SamplingOp expects 0 <= n, M < 2^31");
  return TFGPC_OK;
}

}  // namespace tfgpc

using namespace tfgpc;

extern "C" size_t tfgpc_sampling_workspace_bytes(int64_t n) { return sampling_ws_bytes(n); }

static int sampling_count_impl(bool symmetric, void* stream, int D, int mode, int64_t n,
                               const float* points, const int32_t* batch_ids,
                               const int64_t* point_keys, const int32_t* num_cells,
                               const int32_t* neighbors, int64_t M, const int32_t* ranges,
                               void* ws, size_t ws_bytes, int64_t* num_samples_out) {
  int rc = check_smp_args(D, mode, n, M);
  if (rc) return rc;
  TFGPC_REQUIRE(num_samples_out, "SamplingOp got a null pointer");
  *num_samples_out = 0;
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && batch_ids && point_keys && num_cells && ws,
                "SamplingOp got a null pointer");
  TFGPC_REQUIRE(mode == 1 || (ranges && (M == 0 || neighbors)), "SamplingOp got a null pointer");
  if (ws_bytes < sampling_ws_bytes(n))
    return fail(TFGPC_ENOMEM, "SamplingOp workspace too small: %zu < %zu", ws_bytes,
                sampling_ws_bytes(n));
  cudaStream_t st = (cudaStream_t)stream;
  SamplingWs w = carve(ws, n);
  {
    ProfScope prof(st, "sampling_flag_runs");
    flag_runs_kernel<<<blocks_for(n, 256), 256, 0, st>>>(n, point_keys, w.flags);
  }
  TFGPC_LAUNCH_CHECK();
  rc = inclusive_scan_i32(st, w.flags, w.run_idx, n, w.block_sums, w.totals);
  if (rc) return rc;
  {
    ProfScope prof(st, "sampling_compact_runs");
    compact_runs_kernel<<<blocks_for(n, 256), 256, 0, st>>>(n, w.flags, w.run_idx, w.starts);
  }
  TFGPC_LAUNCH_CHECK();
  if (mode == 0) {
    TFGPC_CUDA(cudaMemsetAsync(w.used, 0, sizeof(int32_t) * (size_t)n, st));
    unsigned grid = min(blocks_for(n, kSmpThreads / 32), (unsigned)(sm_count() * 32));
    // the blocked flags of the symmetric variant live in used_scan, which
    // nothing else touches before the scan below overwrites it
    if (symmetric) TFGPC_CUDA(cudaMemsetAsync(w.used_scan, 0, sizeof(int32_t) * (size_t)n, st));
    for (int pass = 0; pass < (1 << D); ++pass) {
      ProfScope prof(st, "sampling_poisson_pass");
      if (symmetric) {
        TFGPC_DIM_SWITCH(D, poisson_pass_symmetric_kernel<kD><<<grid, kSmpThreads, 0, st>>>(
            pass, n, w.totals, w.starts, point_keys, num_cells, (const int2*)neighbors, ranges,
            w.used, w.used_scan));
      } else {
        TFGPC_DIM_SWITCH(D, poisson_pass_kernel<kD><<<grid, kSmpThreads, 0, st>>>(
            pass, n, w.totals, w.starts, point_keys, num_cells, (const int2*)neighbors, ranges,
            w.used));
      }
      TFGPC_LAUNCH_CHECK();
    }
    rc = inclusive_scan_i32(st, w.used, w.used_scan, n, w.block_sums, w.totals + 1);
    if (rc) return rc;
  }
  int64_t totals[2] = {0, 0};
  rc = read_small(st, w.totals, sizeof(totals), totals);
  if (rc) return rc;
  *num_samples_out = mode == 0 ? totals[1] : totals[0];
  return TFGPC_OK;
}

extern "C" int tfgpc_sampling_count(void* stream, int D, int mode, int64_t n, const float* points,
                                    const int32_t* batch_ids, const int64_t* point_keys,
                                    const int32_t* num_cells, const int32_t* neighbors, int64_t M,
                                    const int32_t* ranges, void* ws, size_t ws_bytes,
                                    int64_t* num_samples_out) {
  return sampling_count_impl(false, stream, D, mode, n, points, batch_ids, point_keys, num_cells,
                             neighbors, M, ranges, ws, ws_bytes, num_samples_out);
}

extern "C" int tfgpc_sampling_count_symmetric(void* stream, int D, int mode, int64_t n,
                                              const float* points, const int32_t* batch_ids,
                                              const int64_t* point_keys,
                                              const int32_t* num_cells, const int32_t* neighbors,
                                              int64_t M, const int32_t* ranges, void* ws,
                                              size_t ws_bytes, int64_t* num_samples_out) {
  return sampling_count_impl(true, stream, D, mode, n, points, batch_ids, point_keys, num_cells,
                             neighbors, M, ranges, ws, ws_bytes, num_samples_out);
}

extern "C" int tfgpc_sampling_store(void* stream, int D, int mode, int64_t n, const float* points,
                                    const int32_t* batch_ids, const int64_t* point_keys,
                                    const int32_t* num_cells, int64_t num_samples, void* ws,
                                    size_t ws_bytes, float* sample_pts_out,
                                    int32_t* sample_batch_ids_out, int32_t* sample_indices_out) {
  int rc = check_smp_args(D, mode, n, 0);
  if (rc) return rc;
  TFGPC_REQUIRE(num_samples >= 0 && num_samples <= n, "SamplingOp expects 0 <= num_samples <= n");
  if (n == 0 || num_samples == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && batch_ids && point_keys && num_cells && ws && sample_pts_out &&
                sample_batch_ids_out && (mode == 1 || sample_indices_out),
                "SamplingOp got a null pointer");
  if (ws_bytes < sampling_ws_bytes(n))
    return fail(TFGPC_ENOMEM, "SamplingOp workspace too small: %zu < %zu", ws_bytes,
                sampling_ws_bytes(n));
  cudaStream_t st = (cudaStream_t)stream;
  SamplingWs w = carve(ws, n);
  ProfScope prof(st, mode == 0 ? "sampling_store_poisson" : "sampling_cell_average");
  if (mode == 0) {
    TFGPC_DIM_SWITCH(D, store_poisson_kernel<kD><<<blocks_for(n, 256), 256, 0, st>>>(
        n, w.used, w.used_scan, points, batch_ids, sample_pts_out, sample_batch_ids_out,
        sample_indices_out));
  } else {
    TFGPC_DIM_SWITCH(D, cell_average_kernel<kD><<<blocks_for(num_samples, 128), 128, 0, st>>>(
        n, num_samples, w.starts, points, point_keys, num_cells, sample_pts_out,
        sample_batch_ids_out));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
