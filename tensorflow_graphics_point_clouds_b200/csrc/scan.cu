// Device-wide inclusive scan of int32 counts (reduce, scan of tile sums, scan).
// Takes the place of the reference's recursive Blelloch scan with its host
// loop (find_neighbors/cc/kernels/scan_alg_kernels.cu.cc:41-266): three
// launches (one for inputs of a single tile), no host synchronisation, 64-bit
// tile sums so that totals beyond 2^31 are detected by the caller instead of
// wrapping silently.
#include "common.cuh"

namespace tfgpc {

constexpr int kScanThreads = 512;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

int64_t scan_block_sums_elems(int64_t n) { return (n + kScanTile - 1) / kScanTile + 1; }

__device__ __forceinline__ int64_t block_reduce_i64(int64_t v, int64_t* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int w = threadIdx.x >> 5;
  if (lane_id() == 0) smem[w] = v;
  __syncthreads();
  int nw = blockDim.x >> 5;
  v = (threadIdx.x < nw) ? smem[threadIdx.x] : 0;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  return v;  // valid in thread 0
}

__global__ void __launch_bounds__(kScanThreads)
scan_reduce_kernel(const int32_t* __restrict__ in, int64_t n, int64_t* __restrict__ tile_sums) {
  __shared__ int64_t smem[32];
  int64_t base = (int64_t)blockIdx.x * kScanTile;
  int64_t v = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    int64_t idx = base + (int64_t)i * kScanThreads + threadIdx.x;
    if (idx < n) v += in[idx];
  }
  v = block_reduce_i64(v, smem);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = v;
}

// Exclusive scan of the tile sums by one block; writes the grand total.
__global__ void __launch_bounds__(1024)
scan_tile_sums_kernel(int64_t* __restrict__ tile_sums, int64_t tiles, int64_t* __restrict__ total) {
  __shared__ int64_t warp_tot[32];
  __shared__ int64_t carry_s;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < tiles; base += blockDim.x) {
    int64_t idx = base + threadIdx.x;
    int64_t v = idx < tiles ? tile_sums[idx] : 0;
    int64_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int64_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane_id() >= o) x += y;
    }
    int w = threadIdx.x >> 5;
    if (lane_id() == 31) warp_tot[w] = x;
    __syncthreads();
    if (w == 0) {
      int64_t t = warp_tot[lane_id()];
      int64_t s = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int64_t y = __shfl_up_sync(0xffffffffu, s, o);
        if (lane_id() >= o) s += y;
      }
      warp_tot[lane_id()] = s - t;  // exclusive warp offsets
    }
    __syncthreads();
    int64_t carry = carry_s;
    int64_t incl = carry + warp_tot[w] + x;
    if (idx < tiles) tile_sums[idx] = incl - v;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry_s;
}

__global__ void __launch_bounds__(kScanThreads)
scan_tiles_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out, int64_t n,
                  const int64_t* __restrict__ tile_offsets, int64_t* __restrict__ total) {
  __shared__ int64_t warp_tot[kScanThreads / 32];
  int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  int32_t item[kScanItems];
  int64_t local = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    item[i] = (base + i < n) ? in[base + i] : 0;
    local += item[i];
  }
  int64_t x = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int64_t y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane_id() >= o) x += y;
  }
  int w = threadIdx.x >> 5;
  if (lane_id() == 31) warp_tot[w] = x;
  __syncthreads();
  if (w == 0) {
    int64_t t = lane_id() < kScanThreads / 32 ? warp_tot[lane_id()] : 0;
    int64_t s = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int64_t y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane_id() >= o) s += y;
    }
    if (lane_id() < kScanThreads / 32) warp_tot[lane_id()] = s - t;
  }
  __syncthreads();
  // tile_offsets == nullptr: the input is a single tile, scanned by this one
  // launch, which then also writes the grand total
  int64_t run = (tile_offsets ? tile_offsets[blockIdx.x] : 0) + warp_tot[w] + (x - local);
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    run += item[i];
    if (base + i < n) out[base + i] = (int32_t)run;
  }
  if (!tile_offsets && threadIdx.x == kScanThreads - 1) *total = run;
}

int inclusive_scan_i32(cudaStream_t stream, const int32_t* in, int32_t* out, int64_t n,
                       int64_t* block_sums, int64_t* total) {
  if (n <= 0) {
    TFGPC_CUDA(cudaMemsetAsync(total, 0, sizeof(int64_t), stream));
    return TFGPC_OK;
  }
  int64_t tiles = (n + kScanTile - 1) / kScanTile;
  ProfScope prof(stream, "scan_i32");
  if (tiles == 1) {
    scan_tiles_kernel<<<1, kScanThreads, 0, stream>>>(in, out, n, nullptr, total);
    TFGPC_LAUNCH_CHECK();
    return TFGPC_OK;
  }
  scan_reduce_kernel<<<(unsigned)tiles, kScanThreads, 0, stream>>>(in, n, block_sums);
  TFGPC_LAUNCH_CHECK();
  scan_tile_sums_kernel<<<1, 1024, 0, stream>>>(block_sums, tiles, total);
  TFGPC_LAUNCH_CHECK();
  scan_tiles_kernel<<<(unsigned)tiles, kScanThreads, 0, stream>>>(in, out, n, block_sums,
                                                                  nullptr);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

}  // namespace tfgpc
