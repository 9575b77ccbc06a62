// Regular-grid construction: cell keys, descending key sort with the gathers
// that follow it, and the (batch, c0, c1) tube ranges.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace tfgpc {

constexpr int kKeyThreads = 256;

// One point per thread.  The block's kKeyThreads*D coordinates are contiguous
// in memory, so they are staged through shared memory with fully coalesced
// 128-byte warp loads instead of D strided loads per thread.
template <int D>
__global__ void __launch_bounds__(kKeyThreads)
compute_keys_kernel(int64_t n, const float* __restrict__ pts, const int32_t* __restrict__ batch_ids,
                    int64_t batch_size, const float* __restrict__ smin_all,
                    const int32_t* __restrict__ num_cells, const float* __restrict__ inv_cell,
                    int64_t* __restrict__ keys_out) {
  __shared__ float stage[kKeyThreads * D];
  const Grid<D> g = load_grid<D>(num_cells, inv_cell);
  for (int64_t base = (int64_t)blockIdx.x * kKeyThreads; base < n;
       base += (int64_t)gridDim.x * kKeyThreads) {
    int64_t cnt = min((int64_t)kKeyThreads, n - base);
    const float* src = pts + base * D;
#pragma unroll
    for (int i = 0; i < D; ++i) {
      int e = i * kKeyThreads + threadIdx.x;
      if (e < cnt * D) stage[e] = __ldg(src + e);
    }
    __syncthreads();
    if (threadIdx.x < cnt) {
      int64_t idx = base + threadIdx.x;
      int b = __ldg(batch_ids + idx);
      // A batch id outside [0, batch_size) would index past scaled_aabb_min;
      // clamp the lookup (the key still carries the id that was passed in).
      int bs = min(max(b, 0), (int)batch_size - 1);
      float p[D], smin[D];
      int cell[D];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        p[d] = stage[threadIdx.x * D + d];
        smin[d] = __ldg(smin_all + (int64_t)bs * D + d);
      }
      cell_of<D>(p, smin, g, cell);
      keys_out[idx] = key_of<D>(cell, g, b);
    }
    __syncthreads();
  }
}

__global__ void iota_kernel(int32_t* out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (int32_t)i;
}

// sorted_points[i, d] = points[perm[i], d]; one thread per output float so the
// stores are coalesced (the reads are a permutation and cannot be).
template <int D>
__global__ void gather_sorted_kernel(int64_t n, const int32_t* __restrict__ perm,
                                     const float* __restrict__ pts,
                                     const int32_t* __restrict__ batch_ids,
                                     float* __restrict__ pts_out,
                                     int32_t* __restrict__ batch_out) {
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n * D) return;
  int64_t i = e / D;
  int d = (int)(e - i * D);
  int64_t src = __ldg(perm + i);
  pts_out[e] = __ldg(pts + src * D + d);
  if (d == 0) batch_out[i] = __ldg(batch_ids + src);
}

// One sorted key per thread: a tube starts where the tube index differs from
// the previous key's and ends where it differs from the next key's.
template <int D>
__global__ void build_grid_ds_kernel(int64_t n, const int64_t* __restrict__ keys,
                                     const int32_t* __restrict__ num_cells, int64_t n_ds,
                                     int2* __restrict__ ds) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t div = 1;
#pragma unroll
  for (int d = 2; d < D; ++d) div *= __ldg(num_cells + d);
  int64_t cur = __ldg(keys + i) / div;
  if (cur < 0 || cur >= n_ds) return;  // key from another grid: skip, never write outside
  if (i > 0 && __ldg(keys + i - 1) / div != cur) ds[cur].x = (int)i;
  if (i + 1 == n || __ldg(keys + i + 1) / div != cur) ds[cur].y = (int)(i + 1);
}

// Per-cloud axis-aligned bounding box (the unsorted_segment_min / _max of
// pylib/pc/PointCloud.py:38-43).  Floats are ordered through their bit
// patterns: non-negative values compare like signed ints, negative values like
// reversed unsigned ints, so one integer atomic per value is enough.  -0.0f
// compares equal to 0.0f but carries the bit pattern of the most negative int:
// it is turned into +0.0f first (x + 0.0f does that in round-to-nearest), else
// it would overwrite a negative minimum and never raise a negative maximum.
__device__ __forceinline__ void atomic_min_float(float* addr, float v) {
  v = __fadd_rn(v, 0.0f);
  if (v >= 0.0f) atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned*>(addr), __float_as_uint(v));
}

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  v = __fadd_rn(v, 0.0f);
  if (v >= 0.0f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned*>(addr), __float_as_uint(v));
}

__global__ void fill_kernel(float* out, int64_t n, float v) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = v;
}

// Each thread folds a run of consecutive points that share a batch id in
// registers and issues atomics only when the id changes, so clouds stored
// contiguously cost a handful of atomics per thread.
template <int D>
__global__ void __launch_bounds__(256)
aabb_kernel(int64_t n, const float* __restrict__ pts, const int32_t* __restrict__ batch_ids,
            int batch_size, float* __restrict__ mn, float* __restrict__ mx) {
  constexpr int kPer = 16;
  const int64_t begin = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * kPer;
  if (begin >= n) return;
  const int64_t end = min(begin + kPer, n);
  int cur = -1;
  float lo[D], hi[D];
  for (int64_t i = begin; i < end; ++i) {
    const int b = __ldg(batch_ids + i);
    if (b != cur) {
      if (cur >= 0 && cur < batch_size) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
          atomic_min_float(mn + (int64_t)cur * D + d, lo[d]);
          atomic_max_float(mx + (int64_t)cur * D + d, hi[d]);
        }
      }
      cur = b;
#pragma unroll
      for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; }
    }
#pragma unroll
    for (int d = 0; d < D; ++d) {
      const float v = __ldg(pts + i * D + d);
      lo[d] = fminf(lo[d], v);
      hi[d] = fmaxf(hi[d], v);
    }
  }
  // The common case, a whole warp inside one cloud: fold the 32 boxes with
  // shuffles and let one lane issue the atomics (min and max are exact and
  // order-independent, so the result is the same).
  const unsigned active = __activemask();
  const int cur0 = __shfl_sync(active, cur, __ffs(active) - 1);
  if (active == 0xffffffffu && __all_sync(active, cur == cur0)) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
        hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
      }
    }
    if ((threadIdx.x & 31) != 0) return;
  }
  if (cur >= 0 && cur < batch_size) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
      atomic_min_float(mn + (int64_t)cur * D + d, lo[d]);
      atomic_max_float(mx + (int64_t)cur * D + d, hi[d]);
    }
  }
}

}  // namespace tfgpc

using namespace tfgpc;

extern "C" int tfgpc_compute_keys(void* stream, int D, int64_t n, const float* points,
                                  const int32_t* batch_ids, int64_t batch_size,
                                  const float* scaled_aabb_min, const int32_t* num_cells,
                                  const float* inv_cell_sizes, int64_t* keys_out) {
  TFGPC_REQUIRE(valid_dims(D), "ComputeKeys expects a valid number of dimension (got %d)", D);
  TFGPC_REQUIRE(n >= 0 && batch_size > 0, "ComputeKeys expects n >= 0 and batch_size > 0");
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && batch_ids && scaled_aabb_min && num_cells && inv_cell_sizes && keys_out,
                "ComputeKeys got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(n, kKeyThreads), (unsigned)(sm_count() * 16));
  ProfScope prof(st, "compute_keys");
  TFGPC_DIM_SWITCH(D, compute_keys_kernel<kD><<<grid, kKeyThreads, 0, st>>>(
      n, points, batch_ids, batch_size, scaled_aabb_min, num_cells, inv_cell_sizes, keys_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

static size_t cub_sort_temp_bytes(int64_t n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairsDescending(nullptr, bytes, (const int64_t*)nullptr,
                                            (int64_t*)nullptr, (const int32_t*)nullptr,
                                            (int32_t*)nullptr, n, 0, 64, (cudaStream_t)0);
  return bytes;
}

extern "C" size_t tfgpc_sort_keys_workspace_bytes(int64_t n) {
  if (n <= 0) return 256;
  return align_up((size_t)n * sizeof(int32_t), 256) + align_up(cub_sort_temp_bytes(n), 256) + 256;
}

extern "C" int tfgpc_sort_keys_desc(void* stream, int D, int64_t n, int key_bits,
                                    const int64_t* keys, const float* points,
                                    const int32_t* batch_ids, int32_t* perm_out,
                                    int64_t* sorted_keys_out, float* sorted_points_out,
                                    int32_t* sorted_batch_ids_out, void* ws, size_t ws_bytes) {
  TFGPC_REQUIRE(n >= 0 && n < (int64_t)INT32_MAX, "sort_keys expects 0 <= n < 2^31");
  TFGPC_REQUIRE(key_bits >= 0 && key_bits <= 64, "sort_keys expects key_bits in [0, 64]");
  bool do_gather = sorted_points_out != nullptr || sorted_batch_ids_out != nullptr;
  if (do_gather) {
    TFGPC_REQUIRE(valid_dims(D), "sort_keys expects a valid number of dimension (got %d)", D);
    TFGPC_REQUIRE(sorted_points_out && sorted_batch_ids_out && points && batch_ids,
                  "sort_keys gathers points and batch ids together: pass all four pointers");
  }
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(keys && perm_out && sorted_keys_out && ws, "sort_keys got a null pointer");
  if (ws_bytes < tfgpc_sort_keys_workspace_bytes(n))
    return fail(TFGPC_ENOMEM, "sort_keys workspace too small: %zu < %zu", ws_bytes,
                tfgpc_sort_keys_workspace_bytes(n));
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* iota = (int32_t*)ws;
  void* cub_ws = (char*)ws + align_up((size_t)n * sizeof(int32_t), 256);
  size_t cub_bytes = cub_sort_temp_bytes(n);
  {
    ProfScope prof(st, "sort_iota");
    iota_kernel<<<blocks_for(n, 256), 256, 0, st>>>(iota, n);
  }
  TFGPC_LAUNCH_CHECK();
  int end_bit = key_bits == 0 ? 64 : key_bits;
  // LSD radix sort: stable, so equal keys keep ascending original index.
  {
    ProfScope prof(st, "sort_radix");
    TFGPC_CUDA(cub::DeviceRadixSort::SortPairsDescending(cub_ws, cub_bytes, keys, sorted_keys_out,
                                                         (const int32_t*)iota, perm_out, n, 0,
                                                         end_bit, st));
  }
  if (do_gather) {
    ProfScope prof(st, "sort_gather");
    TFGPC_DIM_SWITCH(D, gather_sorted_kernel<kD><<<blocks_for(n * kD, 256), 256, 0, st>>>(
        n, perm_out, points, batch_ids, sorted_points_out, sorted_batch_ids_out));
    TFGPC_LAUNCH_CHECK();
  }
  return TFGPC_OK;
}

extern "C" int tfgpc_build_grid_ds(void* stream, int D, int64_t n, const int64_t* sorted_keys,
                                   const int32_t* num_cells, const int32_t* num_cells_host,
                                   int64_t batch_size, int32_t* ds_out) {
  TFGPC_REQUIRE(valid_dims(D), "BuildGridDs expects a valid number of dimension (got %d)", D);
  TFGPC_REQUIRE(batch_size > 0, "BuildGridDs expects a positive batch size");
  TFGPC_REQUIRE(num_cells && num_cells_host && ds_out, "BuildGridDs got a null pointer");
  TFGPC_REQUIRE(num_cells_host[0] > 0 && num_cells_host[1] > 0,
                "BuildGridDs expects positive cell counts");
  TFGPC_REQUIRE(n >= 0 && n < (int64_t)INT32_MAX, "BuildGridDs expects 0 <= n < 2^31");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t n_ds = batch_size * num_cells_host[0] * num_cells_host[1];
  TFGPC_CUDA(cudaMemsetAsync(ds_out, 0, sizeof(int32_t) * 2 * (size_t)n_ds, st));
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(sorted_keys, "BuildGridDs got a null pointer");
  ProfScope prof(st, "build_grid_ds");
  TFGPC_DIM_SWITCH(D, build_grid_ds_kernel<kD><<<blocks_for(n, 256), 256, 0, st>>>(
      n, sorted_keys, num_cells, n_ds, (int2*)ds_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

namespace tfgpc {
// BuildGridDs into an array sized for `capacity` tubes, without the cell counts
// on the host (grid_neighborhood.cu): the tubes occupy the first batch * C0 * C1
// entries, whatever C0 and C1 turn out to be.
int build_grid_ds_capacity(cudaStream_t st, int D, int64_t n, const int64_t* sorted_keys,
                           const int32_t* num_cells, int64_t capacity, int32_t* ds_out) {
  TFGPC_CUDA(cudaMemsetAsync(ds_out, 0, sizeof(int32_t) * 2 * (size_t)capacity, st));
  if (n == 0) return TFGPC_OK;
  ProfScope prof(st, "build_grid_ds");
  TFGPC_DIM_SWITCH(D, build_grid_ds_kernel<kD><<<blocks_for(n, 256), 256, 0, st>>>(
      n, sorted_keys, num_cells, capacity, (int2*)ds_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
}  // namespace tfgpc

extern "C" int tfgpc_compute_aabb(void* stream, int D, int64_t n, const float* points,
                                  const int32_t* batch_ids, int64_t batch_size, float* aabb_min_out,
                                  float* aabb_max_out) {
  TFGPC_REQUIRE(valid_dims(D), "ComputeAabb expects a valid number of dimension (got %d)", D);
  TFGPC_REQUIRE(n >= 0 && batch_size > 0 && batch_size < (int64_t)INT32_MAX,
                "ComputeAabb expects n >= 0 and a positive batch size");
  TFGPC_REQUIRE(aabb_min_out && aabb_max_out, "ComputeAabb got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "compute_aabb");
  const int64_t cells = batch_size * D;
  fill_kernel<<<blocks_for(cells, 256), 256, 0, st>>>(aabb_min_out, cells, INFINITY);
  fill_kernel<<<blocks_for(cells, 256), 256, 0, st>>>(aabb_max_out, cells, -INFINITY);
  TFGPC_LAUNCH_CHECK();
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && batch_ids, "ComputeAabb got a null pointer");
  TFGPC_DIM_SWITCH(D, aabb_kernel<kD><<<blocks_for((n + 15) / 16, 256), 256, 0, st>>>(
      n, points, batch_ids, (int)batch_size, aabb_min_out, aabb_max_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
