// Radius neighbor search on the regular grid: a count pass, a device-wide scan
// and a fill pass that writes CSR neighbor lists in canonical order (ascending
// point index inside every sample).
//
// One warp owns one sample.  Its lanes first resolve, in parallel, the
// candidate index range of every neighboring cell column (the reference spends
// one thread per (sample, offset) in a separate kernel with two interleaved
// binary searches, find_ranges_grid_ds_kernels.cu.cc:49-169); then the warp
// walks the ranges from the highest cell key to the lowest -- keys are sorted
// descending, so this is ascending point index -- testing 32 candidates per
// step and compacting the hits with a ballot, which gives the canonical order
// without atomics (the reference: atomicAdd per hit, count_neighbors_kernels.
// cu.cc:84-87 and store_neighbors_kernels.cu.cc:160-166).
#include <mutex>

#include "common.cuh"

namespace tfgpc {

constexpr int kFnThreads = 256;
constexpr int kFnSpan = 8;  // consecutive samples one warp takes at a time

template <int D>
__host__ __device__ constexpr int num_offsets() {
  int n = 1;
  for (int d = 0; d < (D == 2 ? 2 : D - 1); ++d) n *= 3;
  return n;
}

// First index in [lo, hi) of the descending key array with key <= v.
__device__ __forceinline__ int lower_bound_desc(const int64_t* __restrict__ keys, int lo, int hi,
                                                int64_t v) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (__ldg(keys + mid) > v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Candidate range [a, e) of offset code `code` around `cell`.  For D >= 3 the
// code enumerates the leading D-1 coordinates (most significant first) and the
// last coordinate's +-1 range is cut out of the (batch, c0, c1) tube by key;
// for D == 2 the code enumerates both coordinates and the tube is the cell.
template <int D>
__device__ __forceinline__ int2 candidate_range(int code, const int* cell, int batch,
                                                const Grid<D>& g,
                                                const int64_t* __restrict__ keys,
                                                const int2* __restrict__ ds) {
  constexpr int kDigits = (D == 2) ? 2 : D - 1;
  int cp[D];
  bool ok = true;
  int rem = code;
#pragma unroll
  for (int d = kDigits - 1; d >= 0; --d) {
    cp[d] = cell[d] + (rem % 3) - 1;
    rem /= 3;
    ok = ok && cp[d] >= 0 && cp[d] < g.nc[d];
  }
  if (!ok) return make_int2(0, 0);
  int2 tube = __ldg(ds + ((int64_t)batch * g.nc[0] + cp[0]) * g.nc[1] + cp[1]);
  if (D == 2 || tube.y <= tube.x) return tube.y > tube.x ? tube : make_int2(0, 0);
  int lo_l = max(cell[D - 1] - 1, 0);
  int hi_l = min(cell[D - 1] + 1, g.nc[D - 1] - 1);
  cp[D - 1] = hi_l;
  int64_t k_hi = key_of<D>(cp, g, batch);
  cp[D - 1] = lo_l;
  int64_t k_lo = key_of<D>(cp, g, batch);
  int a = lower_bound_desc(keys, tube.x, tube.y, k_hi);
  int e = lower_bound_desc(keys, a, tube.y, k_lo - 1);
  return make_int2(a, e);
}

// t_d = (s_d - p_d) * inv_r_d, d2 = fma chain from t_0*t_0, sqrtf(d2) < 1
// (count_neighbors_kernels.cu.cc:84-85, math_helper.h:311-327).  The square
// root is not evaluated: a correctly rounded sqrtf maps every float below 1
// to a float below 1 (the largest, 1 - 2^-24, goes to 1 - 2^-24) and every
// float >= 1 to a float >= 1, so `sqrtf(d2) < 1.0f` and `d2 < 1.0f` decide
// identically, NaN included.
template <int D>
__device__ __forceinline__ bool within_radius(const float* s, const float* __restrict__ p,
                                              const float* inv_r) {
  float t = __fmul_rn(__fsub_rn(s[0], __ldg(p)), inv_r[0]);
  float d2 = __fmul_rn(t, t);
#pragma unroll
  for (int d = 1; d < D; ++d) {
    t = __fmul_rn(__fsub_rn(s[d], __ldg(p + d)), inv_r[d]);
    d2 = __fmaf_rn(t, t, d2);
  }
  return d2 < 1.0f;
}

// What the fused fill pass adds to the neighbor list: the same pairs with the
// neighbor's index in the UNSORTED point order (Neighborhood.py:246-250) and the
// (optionally) the Gaussian density estimate at every sample over its neighbors,
// i.e. ComputePdf (compute_pdf_kernels.cu.cc:107-128) evaluated where the
// candidate's coordinates are already in registers.  The ids cost two
// instructions per hit; the densities cost more than a separate pass over the
// finished lists does (here one lane in six holds a hit, there every lane works),
// so the callers of this library ask for the ids only.
struct FillExtras {
  const int32_t* sorted_indices;   // [n] original index of sorted point j
  int2* ids_out;                   // [M] (original neighbor index, sample)
  const float* inv_bw;             // [D]
  int pdf_mode;                    // 0: inv_bw as given, 1: sqrt(n_bw)
  int64_t n_bw;
  float* sample_pdf;               // [ns]
};

// MODE 0: count, 1: fill, 2: fill with FillExtras
template <int D, int MODE>
__global__ void __launch_bounds__(kFnThreads)
find_neighbors_kernel(int64_t ns, const int32_t* __restrict__ order,
                      const float* __restrict__ samples,
                      const int32_t* __restrict__ sbatch, const float* __restrict__ pts,
                      const int64_t* __restrict__ keys, const int2* __restrict__ ds,
                      int batch_size, const int32_t* __restrict__ num_cells,
                      const float* __restrict__ smin_all, const float* __restrict__ inv_cell,
                      const float* __restrict__ inv_radii, int max_neighs,
                      int32_t* __restrict__ counts, const int32_t* __restrict__ ranges,
                      int2* __restrict__ neigh_out, FillExtras ex) {
  constexpr bool FILL = MODE != 0;
  constexpr int kOff = num_offsets<D>();
  constexpr int kChunks = (kOff + 31) / 32;
  const Grid<D> g = load_grid<D>(num_cells, inv_cell);
  float inv_r[D], bw[D];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    inv_r[d] = __ldg(inv_radii + d);
    bw[d] = 0.0f;
    // (inv_bw is only given, and only read, when densities are asked for)
    if (MODE == 2 && ex.sample_pdf)
      bw[d] = ex.pdf_mode == 1 ? sqrtf((float)ex.n_bw) : __ldg(ex.inv_bw + d);
  }
  const int lane = lane_id();
  const unsigned lt_mask = (1u << lane) - 1u;
  const int64_t warps = ((int64_t)gridDim.x * kFnThreads) >> 5;
  // A warp takes kFnSpan consecutive samples at a time.  Samples that follow one
  // another in memory mostly share their cell (always, when the samples are
  // the sorted points themselves), and then the candidate ranges of the
  // previous sample are kept instead of being searched again.
  int prev_cell[D], prev_b = -1;
  int2 my_range[kChunks];
  for (int64_t v = (((int64_t)blockIdx.x * kFnThreads + threadIdx.x) >> 5) * kFnSpan; v < ns;
       v += ((v + 1) % kFnSpan) ? 1 : (warps - 1) * kFnSpan + 1) {
    // `order` lists the samples in the sequence to visit them in (one that keeps
    // spatial neighbors together); what is written for a sample does not depend on it
    const int64_t s = order ? (int64_t)__ldg(order + v) : v;
    if (s < 0 || s >= ns) continue;
    float sp[D], smin[D];
    int cell[D];
    const int b = __ldg(sbatch + s);
    const bool b_ok = b >= 0 && b < batch_size;
    const int bs = b_ok ? b : 0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      sp[d] = __ldg(samples + s * D + d);
      smin[d] = __ldg(smin_all + (int64_t)bs * D + d);
    }
    cell_of<D>(sp, smin, g, cell);
    bool same = b_ok && b == prev_b;
#pragma unroll
    for (int d = 0; d < D; ++d) same = same && cell[d] == prev_cell[d];
    if (!same) {
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        int code = c * 32 + lane;
        my_range[c] = (b_ok && code < kOff) ? candidate_range<D>(code, cell, b, g, keys, ds)
                                            : make_int2(0, 0);
      }
      prev_b = b_ok ? b : -1;
#pragma unroll
      for (int d = 0; d < D; ++d) prev_cell[d] = cell[d];
    }
    int count = 0;
    float density = 0.0f;
    int64_t out_base = 0;
    if (FILL) out_base = s ? (int64_t)__ldg(ranges + s - 1) : 0;
    const int limit = max_neighs > 0 ? max_neighs : INT32_MAX;
#pragma unroll
    for (int c = kChunks - 1; c >= 0; --c) {
      const int top = min(kOff - c * 32, 32) - 1;
      for (int o = top; o >= 0; --o) {
        const int a = __shfl_sync(0xffffffffu, my_range[c].x, o);
        const int e = __shfl_sync(0xffffffffu, my_range[c].y, o);
        for (int base = a; base < e && count < limit; base += 32) {
          const int j = base + lane;
          const bool hit = j < e && within_radius<D>(sp, pts + (int64_t)j * D, inv_r);
          const unsigned m = __ballot_sync(0xffffffffu, hit);
          if (FILL && hit) {
            int pos = count + __popc(m & lt_mask);
            if (pos < limit) {
              neigh_out[out_base + pos] = make_int2(j, (int)s);
              if (MODE == 2)
                ex.ids_out[out_base + pos] = make_int2(__ldg(ex.sorted_indices + j), (int)s);
              if (MODE == 2 && ex.sample_pdf) {
                float local = 1.0f;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                  const float t = (__ldg(pts + (int64_t)j * D + d) - sp[d]) * bw[d] * inv_r[d];
                  local *= bw[d] * expf(t * t * (-0.5f)) * 0.39894228f;
                }
                density += local;
              }
            }
          }
          count += __popc(m);
        }
      }
    }
    if (!FILL && lane == 0) counts[s] = min(count, limit);
    if (MODE == 2 && ex.sample_pdf) {
      density = warp_sum(density);
      if (lane == 0) ex.sample_pdf[s] = density;
    }
  }
}

static int check_fn_args(int D, int64_t ns, int64_t n, int64_t batch_size, int max_neighs) {
  TFGPC_REQUIRE(valid_dims(D), "FindNeighbors expects a valid number of dimension (got %d)", D);
  TFGPC_REQUIRE(ns >= 0 && ns < (int64_t)INT32_MAX && n >= 0 && n < (int64_t)INT32_MAX,
                "FindNeighbors expects 0 <= ns, n < 2^31");
  TFGPC_REQUIRE(batch_size > 0 && batch_size < (int64_t)INT32_MAX,
                "FindNeighbors expects a positive batch size");
  TFGPC_REQUIRE(max_neighs >= 0, "FindNeighbors expects max_neighs >= 0");
  return TFGPC_OK;
}

}  // namespace tfgpc

using namespace tfgpc;

extern "C" size_t tfgpc_find_neighbors_workspace_bytes(int64_t ns) {
  if (ns < 0) ns = 0;
  return align_up((size_t)(scan_block_sums_elems(ns) + 1) * sizeof(int64_t), 256) + 256;
}

// read_mode 0: plain copy of the total (allocates nothing), 1: read through the
// mapped page, 2: no read -- *total_dev_out receives the device address of the
// 64-bit total and the call does not block
static int find_neighbors_count_impl(int read_mode, const int32_t* order,
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    int64_t n, const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs, int32_t* ranges_out,
    void* ws, size_t ws_bytes, int64_t* total_out, int64_t** total_dev_out = nullptr) {
  int rc = check_fn_args(D, ns, n, batch_size, max_neighs);
  if (rc) return rc;
  TFGPC_REQUIRE(total_out, "FindNeighbors got a null pointer");
  *total_out = 0;
  if (ns == 0) return TFGPC_OK;   // (read_mode 2: the caller treats ns == 0 itself)
  TFGPC_REQUIRE(samples && samples_batch_ids && ds && num_cells && scaled_aabb_min &&
                inv_cell_sizes && inv_radii && ranges_out && ws && (n == 0 || (points && point_keys)),
                "FindNeighbors got a null pointer");
  if (ws_bytes < tfgpc_find_neighbors_workspace_bytes(ns))
    return fail(TFGPC_ENOMEM, "FindNeighbors workspace too small: %zu < %zu", ws_bytes,
                tfgpc_find_neighbors_workspace_bytes(ns));
  cudaStream_t st = (cudaStream_t)stream;
  int64_t* block_sums = (int64_t*)ws;
  int64_t* total_dev = block_sums + scan_block_sums_elems(ns);
  unsigned grid = min(blocks_for((ns + kFnSpan - 1) / kFnSpan, kFnThreads / 32),
                      (unsigned)(sm_count() * 32));
  // an order that is not a permutation leaves samples unvisited: they count zero
  if (order) TFGPC_CUDA(cudaMemsetAsync(ranges_out, 0, sizeof(int32_t) * (size_t)ns, st));
  {
  ProfScope prof(st, "find_neighbors_count");
  TFGPC_DIM_SWITCH(D, find_neighbors_kernel<kD, 0><<<grid, kFnThreads, 0, st>>>(
      ns, order, samples, samples_batch_ids, points, point_keys, (const int2*)ds, (int)batch_size,
      num_cells, scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs, ranges_out, nullptr,
      nullptr, FillExtras{}));
  }
  TFGPC_LAUNCH_CHECK();
  rc = inclusive_scan_i32(st, ranges_out, ranges_out, ns, block_sums, total_dev);
  if (rc) return rc;
  if (read_mode == 2) {
    *total_dev_out = total_dev;
    return TFGPC_OK;
  }
  int64_t total = 0;
  if (read_mode == 1) {
    rc = read_small(st, total_dev, sizeof(int64_t), &total);
    if (rc) return rc;
  } else {
    // the entry that must not allocate: a plain copy, which may queue behind
    // bulk transfers of other streams
    TFGPC_CUDA(cudaMemcpyAsync(&total, total_dev, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
    TFGPC_CUDA(cudaStreamSynchronize(st));
  }
  if (total > (int64_t)INT32_MAX)
    return fail(TFGPC_EINVAL, "FindNeighbors found %lld pairs; the int32 ranges of the op "
                "contract hold at most 2^31-1", (long long)total);
  *total_out = total;
  return TFGPC_OK;
}

namespace tfgpc {
// The count pass without its blocking read (grid_neighborhood.cu reads the total
// together with the cell counts).
int find_neighbors_count_async(const int32_t* order, void* stream, int D, int64_t ns,
                               const float* samples, const int32_t* samples_batch_ids, int64_t n,
                               const float* points, const int64_t* point_keys, const int32_t* ds,
                               int64_t batch_size, const int32_t* num_cells,
                               const float* scaled_aabb_min, const float* inv_cell_sizes,
                               const float* inv_radii, int max_neighs, int32_t* ranges_out, void* ws,
                               size_t ws_bytes, int64_t** total_dev_out) {
  int64_t unused = 0;
  return find_neighbors_count_impl(2, order, stream, D, ns, samples, samples_batch_ids, n, points,
                                   point_keys, ds, batch_size, num_cells, scaled_aabb_min,
                                   inv_cell_sizes, inv_radii, max_neighs, ranges_out, ws, ws_bytes,
                                   &unused, total_dev_out);
}
}  // namespace tfgpc

extern "C" int tfgpc_find_neighbors_count(
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    int64_t n, const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs, int32_t* ranges_out,
    void* ws, size_t ws_bytes, int64_t* total_out) {
  return find_neighbors_count_impl(1, nullptr, stream, D, ns, samples, samples_batch_ids, n, points,
                                  point_keys, ds, batch_size, num_cells, scaled_aabb_min,
                                  inv_cell_sizes, inv_radii, max_neighs, ranges_out, ws, ws_bytes,
                                  total_out);
}

static int find_neighbors_fill_impl(const int32_t* order,
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    int64_t n, const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs, const int32_t* ranges,
    int64_t total, int32_t* neigh_out, const FillExtras* extras = nullptr) {
  int rc = check_fn_args(D, ns, n, batch_size, max_neighs);
  if (rc) return rc;
  TFGPC_REQUIRE(total >= 0 && total <= (int64_t)INT32_MAX, "FindNeighbors expects 0 <= total < 2^31");
  cudaStream_t st = (cudaStream_t)stream;
  if (extras && extras->sample_pdf && ns > 0 && total == 0)   // no pair at all: every density is zero
    TFGPC_CUDA(cudaMemsetAsync(extras->sample_pdf, 0, sizeof(float) * (size_t)ns, st));
  if (ns == 0 || total == 0) return TFGPC_OK;
  TFGPC_REQUIRE(samples && samples_batch_ids && points && point_keys && ds && num_cells &&
                scaled_aabb_min && inv_cell_sizes && inv_radii && ranges && neigh_out,
                "FindNeighbors got a null pointer");
  unsigned grid = min(blocks_for((ns + kFnSpan - 1) / kFnSpan, kFnThreads / 32),
                      (unsigned)(sm_count() * 32));
  if (extras) {
    // samples the order leaves unvisited keep a density of zero
    if (order && extras->sample_pdf)
      TFGPC_CUDA(cudaMemsetAsync(extras->sample_pdf, 0, sizeof(float) * (size_t)ns, st));
    ProfScope prof(st, "find_neighbors_fill_fused");
    TFGPC_DIM_SWITCH(D, find_neighbors_kernel<kD, 2><<<grid, kFnThreads, 0, st>>>(
        ns, order, samples, samples_batch_ids, points, point_keys, (const int2*)ds, (int)batch_size,
        num_cells, scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs, nullptr, ranges,
        (int2*)neigh_out, *extras));
  } else {
    ProfScope prof(st, "find_neighbors_fill");
    TFGPC_DIM_SWITCH(D, find_neighbors_kernel<kD, 1><<<grid, kFnThreads, 0, st>>>(
        ns, order, samples, samples_batch_ids, points, point_keys, (const int2*)ds, (int)batch_size,
        num_cells, scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs, nullptr, ranges,
        (int2*)neigh_out, FillExtras{}));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

// The fill pass that also writes the neighbor ids in the unsorted point order and
// the density estimate at every sample (see FillExtras).
extern "C" int tfgpc_find_neighbors_fill_fused(
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    const int32_t* sample_order, int64_t n, const float* points, const int64_t* point_keys,
    const int32_t* ds, int64_t batch_size, const int32_t* num_cells,
    const float* scaled_aabb_min, const float* inv_cell_sizes, const float* inv_radii,
    int max_neighs, const int32_t* ranges, int64_t total, const int32_t* sorted_indices,
    const float* inv_bandwidth, int pdf_mode, int32_t* neigh_out, int32_t* ids_out,
    float* sample_pdf_out) {
  TFGPC_REQUIRE(pdf_mode == 0 || pdf_mode == 1, "FindNeighbors expects density mode 0 or 1");
  TFGPC_REQUIRE(total == 0 || (sorted_indices && ids_out &&
                               (!sample_pdf_out || pdf_mode == 1 || inv_bandwidth)),
                "FindNeighbors got a null pointer");
  FillExtras ex{sorted_indices, (int2*)ids_out, inv_bandwidth, pdf_mode, n, sample_pdf_out};
  return find_neighbors_fill_impl(sample_order, stream, D, ns, samples, samples_batch_ids, n,
                                  points, point_keys, ds, batch_size, num_cells, scaled_aabb_min,
                                  inv_cell_sizes, inv_radii, max_neighs, ranges, total, neigh_out,
                                  &ex);
}

extern "C" int tfgpc_find_neighbors_fill(
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    int64_t n, const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs, const int32_t* ranges,
    int64_t total, int32_t* neigh_out) {
  return find_neighbors_fill_impl(nullptr, stream, D, ns, samples, samples_batch_ids, n, points,
                                  point_keys, ds, batch_size, num_cells, scaled_aabb_min,
                                  inv_cell_sizes, inv_radii, max_neighs, ranges, total, neigh_out);
}

extern "C" int tfgpc_find_neighbors_count_ordered(
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    const int32_t* sample_order, int64_t n, const float* points, const int64_t* point_keys,
    const int32_t* ds, int64_t batch_size, const int32_t* num_cells,
    const float* scaled_aabb_min, const float* inv_cell_sizes, const float* inv_radii,
    int max_neighs, int32_t* ranges_out, void* ws, size_t ws_bytes, int64_t* total_out) {
  return find_neighbors_count_impl(1, sample_order, stream, D, ns, samples, samples_batch_ids,
                                   n, points, point_keys, ds, batch_size, num_cells,
                                   scaled_aabb_min, inv_cell_sizes, inv_radii, max_neighs,
                                   ranges_out, ws, ws_bytes, total_out);
}

extern "C" int tfgpc_find_neighbors_fill_ordered(
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    const int32_t* sample_order, int64_t n, const float* points, const int64_t* point_keys,
    const int32_t* ds, int64_t batch_size, const int32_t* num_cells,
    const float* scaled_aabb_min, const float* inv_cell_sizes, const float* inv_radii,
    int max_neighs, const int32_t* ranges, int64_t total, int32_t* neigh_out) {
  return find_neighbors_fill_impl(sample_order, stream, D, ns, samples, samples_batch_ids, n,
                                  points, point_keys, ds, batch_size, num_cells, scaled_aabb_min,
                                  inv_cell_sizes, inv_radii, max_neighs, ranges, total, neigh_out);
}

// ---- neighbor ids in the unsorted point order, per-pair densities -----------------
//
// pylib maps the sorted neighbor ids back to the original point order with a
// gather and a concat (pylib/pc/Neighborhood.py:246-250) and gathers the
// per-point density per neighbor pair (:287); both are one pass over the pairs.
namespace tfgpc {
__global__ void original_ids_kernel(int64_t m, const int2* __restrict__ neigh,
                                    const int32_t* __restrict__ sorted_indices,
                                    const float* __restrict__ pdf_by_original, int64_t n,
                                    int2* __restrict__ out_ids, float* __restrict__ out_pdf) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int2 nb = __ldg(neigh + i);
    int orig = 0;
    if (nb.x >= 0 && nb.x < n) orig = __ldg(sorted_indices + nb.x);
    out_ids[i] = make_int2(orig, nb.y);
    if (out_pdf) out_pdf[i] = __ldg(pdf_by_original + orig);
  }
}
}  // namespace tfgpc

extern "C" int tfgpc_original_neighbor_ids(void* stream, int64_t M, const int32_t* neighbors,
                                           int64_t n, const int32_t* sorted_indices,
                                           const float* pdf_by_original, int32_t* ids_out,
                                           float* pdf_out) {
  TFGPC_REQUIRE(M >= 0 && M <= (int64_t)INT32_MAX && n >= 0 && n < (int64_t)INT32_MAX,
                "original_neighbor_ids expects 0 <= M, n < 2^31");
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(neighbors && sorted_indices && ids_out, "original_neighbor_ids got a null pointer");
  TFGPC_REQUIRE((pdf_out == nullptr) == (pdf_by_original == nullptr),
                "original_neighbor_ids expects both density pointers or none");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "original_neighbor_ids");
  unsigned grid = min(blocks_for(M, 256), (unsigned)(sm_count() * 32));
  original_ids_kernel<<<grid, 256, 0, st>>>(M, (const int2*)neighbors, sorted_indices,
                                            pdf_by_original, n, (int2*)ids_out, pdf_out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

// ---- FindNeighbors count pass without caller scratch ---------------------------
//
// Scratch of tfgpc_find_neighbors_count_static: the tile sums of the device-wide
// scan plus its 64-bit total, for up to kStaticMaxSamples samples.  The array
// lives in the library image, so every GPU that loads the library keeps these
// bytes resident until the process exits.
namespace tfgpc {
namespace {

constexpr int64_t kStaticMaxSamples = int64_t(1) << 24;                   // 16,777,216 samples
constexpr size_t kStaticScratchBytes = ((size_t(1) << 24) / 4096 + 2) * 8 + 256 + 256;  // ~33 KB

static __device__ __align__(256) unsigned char g_fn_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device.  The array's name
// is only a host-side handle in host code, so the address is looked up once
// per device (with that device current) and cached for the life of the process:
// it does not survive a cudaDeviceReset of that device.
int static_scratch_ptr(void** out) {
  int dev = -1;
  TFGPC_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(TFGPC_EINVAL, "device ordinal %d outside the supported range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_fn_static_scratch);
    if (e != cudaSuccess || !p)
      return fail(TFGPC_ECUDA, "cudaGetSymbolAddress(static scratch) failed: %s",
                  cudaGetErrorString(e));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return TFGPC_OK;
}

}  // namespace
}  // namespace tfgpc

extern "C" int64_t tfgpc_find_neighbors_static_max_samples(void) {
  return tfgpc::kStaticMaxSamples;
}

extern "C" int tfgpc_find_neighbors_count_static(
    void* stream, int D, int64_t ns, const float* samples, const int32_t* samples_batch_ids,
    int64_t n, const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs, int32_t* ranges_out,
    int64_t* total_out) {
  if (ns > kStaticMaxSamples)
    return fail(TFGPC_EINVAL, "find_neighbors_count_static handles at most %lld samples per call "
                "(got %lld); use tfgpc_find_neighbors_count with a caller workspace for more",
                (long long)kStaticMaxSamples, (long long)ns);
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc) return rc;
  // per-launch timing would create CUDA events and grow a host table
  ProfPause no_timing;
  if (tfgpc_find_neighbors_workspace_bytes(ns) > kStaticScratchBytes)
    return fail(TFGPC_ENOMEM, "static scratch of %zu bytes is too small for %lld samples",
                kStaticScratchBytes, (long long)ns);
  // Nothing in the scratch has to start at zero: the scan overwrites every tile
  // sum and the total before it reads them, so stale contents are harmless.
  return find_neighbors_count_impl(0, nullptr, stream, D, ns, samples, samples_batch_ids, n, points,
                                  point_keys, ds, batch_size, num_cells, scaled_aabb_min,
                                  inv_cell_sizes, inv_radii, max_neighs, ranges_out, scratch,
                                  kStaticScratchBytes, total_out);
}
