// Shared host/device helpers of the tfgpc library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tfgpc.h"

namespace tfgpc {

// ---- status handling -------------------------------------------------------
// Stores a printf-formatted message for tfgpc_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

#define TFGPC_REQUIRE(cond, ...)                          \
  do {                                                    \
    if (!(cond)) return ::tfgpc::fail(TFGPC_EINVAL, __VA_ARGS__); \
  } while (0)

#define TFGPC_CUDA(expr)                                                      \
  do {                                                                        \
    cudaError_t e__ = (expr);                                                 \
    if (e__ != cudaSuccess)                                                   \
      return ::tfgpc::fail(TFGPC_ECUDA, "%s failed: %s (%s:%d)", #expr,       \
                           cudaGetErrorString(e__), __FILE__, __LINE__);      \
  } while (0)

#define TFGPC_LAUNCH_CHECK() TFGPC_CUDA(cudaGetLastError())

// Dispatch on the point dimension, D in [2, 6] (the reference's
// DIMENSION_SWITCH_CALL, shared/cc/kernels/defines.hpp:42-49).
#define TFGPC_DIM_SWITCH(D, ...)                         \
  switch (D) {                                           \
    case 2: { constexpr int kD = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int kD = 3; __VA_ARGS__; } break; \
    case 4: { constexpr int kD = 4; __VA_ARGS__; } break; \
    case 5: { constexpr int kD = 5; __VA_ARGS__; } break; \
    case 6: { constexpr int kD = 6; __VA_ARGS__; } break; \
    default: break;                                      \
  }

inline bool valid_dims(int D) { return D >= TFGPC_MIN_DIMS && D <= TFGPC_MAX_DIMS; }

// Optional per-launch timing (tfgpc_profile_enable): when on, a ProfScope
// brackets the launches made inside its lifetime with two CUDA events on the
// launching stream; tfgpc_profile_collect returns name and duration of every
// scope.  When off it costs one thread-local load.
struct ProfScope {
  ProfScope(cudaStream_t st, const char* name);
  ~ProfScope();
  int slot;
  cudaStream_t st;
};

// While one of these lives, the ProfScopes of this host thread record nothing
// (and so create no events and grow no record table): for entry points that
// promise to allocate nothing.
struct ProfPause {
  ProfPause();
  ~ProfPause();
  bool was_on;
};

// Number of SMs of the current device (cached per device).
int sm_count();

// Blocking read of a few values (4 .. 4096 bytes, a multiple of 4) from device
// memory, through mapped pinned host memory instead of a copy engine: it does
// not queue behind bulk transfers on other streams.
int read_small(cudaStream_t st, const void* dev_src, size_t bytes, void* host_dst);

inline unsigned blocks_for(int64_t work, int per_block) {
  int64_t b = (work + per_block - 1) / per_block;
  return (unsigned)(b < 1 ? 1 : b);
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- device helpers --------------------------------------------------------

template <int D>
struct Grid {
  int nc[D];      // cells per dimension
  float inv[D];   // inverse cell size
};

// Loads the D cell counts / inverse cell sizes that the reference keeps in
// device tensors (they are op inputs, so the host never reads them).
template <int D>
__device__ __forceinline__ Grid<D> load_grid(const int32_t* __restrict__ num_cells,
                                             const float* __restrict__ inv_cell) {
  Grid<D> g;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    g.nc[d] = __ldg(num_cells + d);
    g.inv[d] = __ldg(inv_cell + d);
  }
  return g;
}

// Cell of a point: clamp(floor(fma(p, inv_cell, -scaled_min)), 0, cells-1).
// The explicit fma is what the reference's `p*inv - min` compiles to under
// nvcc's default -fmad=true (shared/cc/kernels/grid_utils.h:63-74).
template <int D>
__device__ __forceinline__ void cell_of(const float* p, const float* smin,
                                        const Grid<D>& g, int* cell) {
#pragma unroll
  for (int d = 0; d < D; ++d) {
    float rel = __fmaf_rn(p[d], g.inv[d], -smin[d]);
    int c = (int)floorf(rel);
    c = max(c, 0);
    c = min(c, g.nc[d] - 1);
    cell[d] = c;
  }
}

// Key of a cell (shared/cc/kernels/grid_utils.h:85-100).
template <int D>
__device__ __forceinline__ int64_t key_of(const int* cell, const Grid<D>& g,
                                          int batch) {
  int64_t key = 0, acc = 1;
#pragma unroll
  for (int d = D - 1; d >= 0; --d) {
    key += (int64_t)cell[d] * acc;
    acc *= g.nc[d];
  }
  return key + acc * (int64_t)batch;
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- device-wide inclusive scan of int32 (scan.cu) -------------------------
// out[i] = sum_{j<=i} in[i] (int32, as the reference's ranges are), and the
// 64-bit total is written to *total (device).  `in` may alias `out`.
// block_sums needs scan_block_sums_elems(n) int64 elements.
int64_t scan_block_sums_elems(int64_t n);
int inclusive_scan_i32(cudaStream_t stream, const int32_t* in, int32_t* out,
                       int64_t n, int64_t* block_sums, int64_t* total);

}  // namespace tfgpc
