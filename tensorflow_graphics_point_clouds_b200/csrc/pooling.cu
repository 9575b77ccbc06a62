// Pooling layers and the bias of the 1x1 convolution.
//
// The reference runs these as TensorFlow segment ops: a gather of the
// neighbors' feature rows into an [M, C] tensor followed by
// unsorted_segment_max / _mean over the sample index (Pooling.py:148-162), and
// unsorted_segment_max / _mean over the batch ids for the global variants
// (Pooling.py:51-57, 90-96).  Here the rows of a sample are read in place (its
// pairs are contiguous, ranges holds their end), one thread per (sample,
// channel), so the [M, C] tensor is never written; the global variants
// accumulate per cloud with atomics on the [B, C] result.
// An empty segment gives the lowest float for max (what TensorFlow's
// unsorted_segment_max writes) and 0 for mean.
#include <cfloat>

#include "common.cuh"

namespace tfgpc {
namespace {

constexpr int kPoolThreads = 256;

__global__ void __launch_bounds__(kPoolThreads)
neighborhood_pool_kernel(int mode, int C, int64_t ns, const float* __restrict__ features,
                         const int2* __restrict__ neigh, const int32_t* __restrict__ ranges,
                         float* __restrict__ out) {
  const int64_t total = ns * C;
  for (int64_t i = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * kPoolThreads) {
    const int64_t s = i / C;
    const int c = (int)(i - s * C);
    const int a = s ? __ldg(ranges + s - 1) : 0;
    const int e = __ldg(ranges + s);
    float acc = mode == 0 ? -FLT_MAX : 0.0f;
    for (int m = a; m < e; ++m) {
      const float v = __ldg(features + (int64_t)__ldg(&neigh[m].x) * C + c);
      acc = mode == 0 ? fmaxf(acc, v) : acc + v;
    }
    if (mode == 1 && e > a) acc /= (float)(e - a);
    out[i] = acc;
  }
}

// Order-preserving map between floats and unsigned integers, so that the
// maximum of floats is an atomicMax of integers.
__device__ __forceinline__ unsigned float_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void pool_init_kernel(int mode, int64_t n, float* out, float* counts, int64_t b) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = mode == 0 ? __uint_as_float(float_key(-FLT_MAX)) : 0.0f;
  if (i < b) counts[i] = 0.0f;
}

__global__ void __launch_bounds__(kPoolThreads)
global_pool_kernel(int mode, int C, int64_t n, int64_t batch_size,
                   const float* __restrict__ features, const int32_t* __restrict__ batch_ids,
                   float* out, float* counts) {
  const int64_t total = n * C;
  for (int64_t i = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * kPoolThreads) {
    const int64_t p = i / C;
    const int c = (int)(i - p * C);
    const int b = __ldg(batch_ids + p);
    if (b < 0 || b >= batch_size) continue;
    const float v = __ldg(features + i);
    if (mode == 0) {
      atomicMax(reinterpret_cast<unsigned*>(out) + (int64_t)b * C + c, float_key(v));
    } else {
      atomicAdd(out + (int64_t)b * C + c, v);
      if (c == 0) atomicAdd(counts + b, 1.0f);
    }
  }
}

__global__ void pool_finish_kernel(int mode, int C, int64_t n, float* out,
                                   const float* __restrict__ counts) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (mode == 0) {
    out[i] = key_float(reinterpret_cast<unsigned*>(out)[i]);
  } else {
    const float cnt = counts[i / C];
    out[i] = cnt > 0.0f ? out[i] / cnt : 0.0f;
  }
}

__global__ void add_bias_kernel(int64_t n, int C, float* x, const float* __restrict__ bias) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n * C) x[i] += __ldg(bias + (i % C));
}

// x = act(x * scale + bias): inference batch normalisation with stored
// statistics folded into scale and bias, followed by the activation
// (modelnet40_small.py:236-243).  act 0: none, 1: leaky ReLU with slope alpha.
__global__ void scale_bias_act_kernel(int64_t total, int C, float* x, float scale,
                                      const float* __restrict__ bias, int act, float alpha) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (bias) v += __ldg(bias + (i % C));
    if (act == 1) v = v > 0.0f ? v : v * alpha;
    x[i] = v;
  }
}

}  // namespace
}  // namespace tfgpc

using namespace tfgpc;

extern "C" int tfgpc_neighborhood_pool(void* stream, int mode, int C, int64_t ns, int64_t n_in,
                                       int64_t M, const float* features,
                                       const int32_t* neighbors, const int32_t* ranges,
                                       float* out) {
  TFGPC_REQUIRE(mode == 0 || mode == 1, "Pooling expects mode 0 (max) or 1 (average)");
  TFGPC_REQUIRE(C > 0 && ns >= 0 && n_in >= 0 && M >= 0 && ns < (int64_t)INT32_MAX &&
                M <= (int64_t)INT32_MAX, "Pooling expects 0 <= ns, M < 2^31 and C > 0");
  if (ns == 0) return TFGPC_OK;
  TFGPC_REQUIRE(ranges && out && (M == 0 || (features && neighbors)),
                "Pooling got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "neighborhood_pool");
  unsigned grid = min(blocks_for(ns * C, kPoolThreads), (unsigned)(sm_count() * 32));
  neighborhood_pool_kernel<<<grid, kPoolThreads, 0, st>>>(mode, C, ns, features,
                                                          (const int2*)neighbors, ranges, out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" size_t tfgpc_global_pool_workspace_bytes(int64_t batch_size) {
  return align_up((size_t)(batch_size > 0 ? batch_size : 0) * sizeof(float), 256) + 256;
}

extern "C" int tfgpc_global_pool(void* stream, int mode, int C, int64_t n, int64_t batch_size,
                                 const float* features, const int32_t* batch_ids, float* out,
                                 void* ws, size_t ws_bytes) {
  TFGPC_REQUIRE(mode == 0 || mode == 1, "Pooling expects mode 0 (max) or 1 (average)");
  TFGPC_REQUIRE(C > 0 && n >= 0 && batch_size > 0 && n < (int64_t)INT32_MAX,
                "Pooling expects C > 0, a positive batch size and 0 <= n < 2^31");
  TFGPC_REQUIRE(out && ws && (n == 0 || (features && batch_ids)), "Pooling got a null pointer");
  if (ws_bytes < tfgpc_global_pool_workspace_bytes(batch_size))
    return fail(TFGPC_ENOMEM, "Pooling workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "global_pool");
  float* counts = (float*)ws;
  const int64_t cells = batch_size * C;
  const int64_t init = cells > batch_size ? cells : batch_size;
  pool_init_kernel<<<blocks_for(init, 256), 256, 0, st>>>(mode, cells, out, counts, batch_size);
  TFGPC_LAUNCH_CHECK();
  if (n > 0) {
    unsigned grid = min(blocks_for(n * C, kPoolThreads), (unsigned)(sm_count() * 32));
    global_pool_kernel<<<grid, kPoolThreads, 0, st>>>(mode, C, n, batch_size, features, batch_ids,
                                                      out, counts);
    TFGPC_LAUNCH_CHECK();
  }
  pool_finish_kernel<<<blocks_for(cells, 256), 256, 0, st>>>(mode, C, cells, out, counts);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_add_bias(void* stream, int64_t n, int C, float* x, const float* bias) {
  TFGPC_REQUIRE(n >= 0 && C > 0, "AddBias expects n >= 0 and C > 0");
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(x && bias, "AddBias got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "add_bias");
  add_bias_kernel<<<blocks_for(n * C, 256), 256, 0, st>>>(n, C, x, bias);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_scale_bias_activation(void* stream, int64_t n, int C, float* x, float scale,
                                           const float* bias, int activation, float alpha) {
  TFGPC_REQUIRE(n >= 0 && C > 0, "ScaleBiasActivation expects n >= 0 and C > 0");
  TFGPC_REQUIRE(activation == 0 || activation == 1,
                "ScaleBiasActivation expects activation 0 (none) or 1 (leaky ReLU)");
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(x, "ScaleBiasActivation got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "scale_bias_activation");
  unsigned grid = min(blocks_for(n * C, 256), (unsigned)(sm_count() * 16));
  scale_bias_act_kernel<<<grid, 256, 0, st>>>(n * C, C, x, scale, bias, activation, alpha);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
