// Kernel-MLP basis of the Monte-Carlo convolution and its weight gradients.
//
// Forward, per neighbor pair m = (point j, sample s):
//   diff = (p_in[j] - p_out[s]) * inv_radius                (MCConv.py:264-269)
//   basis[m, k] = act(sum_d diff_d * w1[d, k] + b1[k]) / pdf[m]   (:163-171)
// which the reference runs as a chain of TensorFlow ops (two gathers, subtract,
// divide, tile, matmul, add, leaky_relu, transpose/reshape, divide), each a full
// pass over [M, K] memory.  Here one thread owns one pair and the only traffic
// is the pair's indices, two point gathers, its density and the 4*K-byte row
// it writes.
// Backward: dpre = dbasis / pdf * act'(pre); dw1[d, k] = sum_m diff_d * dpre_k,
// db1[k] = sum_m dpre_k, accumulated in registers over a grid-stride loop,
// reduced through shuffles and shared memory, one atomic per block and value.
#include "common.cuh"

namespace tfgpc {
namespace {

constexpr int kKbThreads = 256;
constexpr int kKTile = 16;  // basis functions handled per thread in the backward pass

__device__ __forceinline__ float act_fwd(float x, int act, float alpha) {
  if (act == 1) return x > 0.0f ? x : expm1f(x);       // ELU
  return x > 0.0f ? x : x * alpha;                      // leaky ReLU (alpha 0: ReLU)
}

__device__ __forceinline__ float act_bwd(float x, int act, float alpha) {
  if (act == 1) return x > 0.0f ? 1.0f : expf(x);
  return x > 0.0f ? 1.0f : alpha;
}

// 256-bit accesses to global memory (sm_100): a thread that owns a 64-byte row
// then reads or writes whole 32-byte sectors instead of halves of them.
__device__ __forceinline__ void st_global_256(float* p, const float* v) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]),
                 "f"(v[6]), "f"(v[7]) : "memory");
}

__device__ __forceinline__ void ld_global_256(const float* p, float* v) {
  asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]),
                 "=f"(v[6]), "=f"(v[7]) : "l"(p));
}

template <int D>
__device__ __forceinline__ void pair_diff(const float* __restrict__ p_in,
                                          const float* __restrict__ p_out, int2 nb,
                                          float inv_radius, float* diff) {
#pragma unroll
  for (int d = 0; d < D; ++d)
    diff[d] = (__ldg(p_in + (int64_t)nb.x * D + d) - __ldg(p_out + (int64_t)nb.y * D + d)) * inv_radius;
}

// WIDE: rows are 32-byte aligned, 256-bit accesses are allowed.
template <int D, int K, bool WIDE>
__global__ void __launch_bounds__(kKbThreads)
kernel_basis_kernel(int64_t M, const float* __restrict__ p_in, const float* __restrict__ p_out,
                    const int2* __restrict__ neigh, const float* __restrict__ pdf,
                    const float* __restrict__ w1, const float* __restrict__ b1, float inv_radius,
                    int act, float alpha, float* __restrict__ basis) {
  __shared__ float w_s[D * K + K];
  for (int i = threadIdx.x; i < D * K + K; i += kKbThreads)
    w_s[i] = i < D * K ? __ldg(w1 + i) : __ldg(b1 + i - D * K);
  __syncthreads();
  for (int64_t m = (int64_t)blockIdx.x * kKbThreads + threadIdx.x; m < M;
       m += (int64_t)gridDim.x * kKbThreads) {
    const int2 nb = __ldg(neigh + m);
    float diff[D];
    pair_diff<D>(p_in, p_out, nb, inv_radius, diff);
    const float inv_pdf = 1.0f / __ldg(pdf + m);
    float* dst = basis + m * K;
#pragma unroll
    for (int q = 0; q < K / 8; ++q) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int k = 8 * q + i;
        float pre = w_s[D * K + k];
#pragma unroll
        for (int d = 0; d < D; ++d) pre = fmaf(diff[d], w_s[d * K + k], pre);
        v[i] = act_fwd(pre, act, alpha) * inv_pdf;
      }
      if (WIDE) {
        st_global_256(dst + 8 * q, v);
      } else {
        reinterpret_cast<float4*>(dst)[2 * q] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[2 * q + 1] = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
  }
}

template <int D, int K, bool WIDE>
__global__ void __launch_bounds__(kKbThreads)
kernel_basis_grads_kernel(int64_t M, const float* __restrict__ p_in,
                          const float* __restrict__ p_out, const int2* __restrict__ neigh,
                          const float* __restrict__ pdf, const float* __restrict__ w1,
                          const float* __restrict__ b1, float inv_radius, int act, float alpha,
                          const float* __restrict__ dbasis, float* __restrict__ dw1,
                          float* __restrict__ db1) {
  constexpr int KT = K < kKTile ? K : kKTile;
  __shared__ float w_s[D * K + K];
  __shared__ float red[(D + 1) * KT];
  for (int i = threadIdx.x; i < D * K + K; i += kKbThreads)
    w_s[i] = i < D * K ? __ldg(w1 + i) : __ldg(b1 + i - D * K);
  for (int i = threadIdx.x; i < (D + 1) * KT; i += kKbThreads) red[i] = 0.0f;
  __syncthreads();
  const int k0 = blockIdx.y * KT;
  float acc_w[D][KT], acc_b[KT];
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    acc_b[k] = 0.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) acc_w[d][k] = 0.0f;
  }
  for (int64_t m = (int64_t)blockIdx.x * kKbThreads + threadIdx.x; m < M;
       m += (int64_t)gridDim.x * kKbThreads) {
    const int2 nb = __ldg(neigh + m);
    float diff[D];
    pair_diff<D>(p_in, p_out, nb, inv_radius, diff);
    const float inv_pdf = 1.0f / __ldg(pdf + m);
    const float* src = dbasis + m * K + k0;
#pragma unroll
    for (int q = 0; q < KT / 8; ++q) {
      float g[8];
      if (WIDE) {
        ld_global_256(src + 8 * q, g);
      } else {
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(src) + 2 * q);
        const float4 g1 = __ldg(reinterpret_cast<const float4*>(src) + 2 * q + 1);
        g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w;
        g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int k = 8 * q + i;
        float pre = w_s[D * K + k0 + k];
#pragma unroll
        for (int d = 0; d < D; ++d) pre = fmaf(diff[d], w_s[d * K + k0 + k], pre);
        const float dpre = g[i] * inv_pdf * act_bwd(pre, act, alpha);
        acc_b[k] += dpre;
#pragma unroll
        for (int d = 0; d < D; ++d) acc_w[d][k] = fmaf(diff[d], dpre, acc_w[d][k]);
      }
    }
  }
  // warp reduction, then one shared-memory atomic per warp and value
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    float v = warp_sum(acc_b[k]);
    if (lane_id() == 0) atomicAdd(&red[D * KT + k], v);
#pragma unroll
    for (int d = 0; d < D; ++d) {
      v = warp_sum(acc_w[d][k]);
      if (lane_id() == 0) atomicAdd(&red[d * KT + k], v);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < (D + 1) * KT; i += kKbThreads) {
    const int d = i / KT, k = i % KT;
    if (d < D) atomicAdd(dw1 + d * K + k0 + k, red[i]);
    else atomicAdd(db1 + k0 + k, red[i]);
  }
}

int check_kb_args(const char* op, int D, int K, int64_t M, int act) {
  TFGPC_REQUIRE(valid_dims(D), "%s expects a valid number of dimension (got %d)", op, D);
  TFGPC_REQUIRE(K == 8 || K == 16 || K == 32 || K == 64,
                "%s expects a valid number of basis functions.", op);
  TFGPC_REQUIRE(M >= 0 && M <= (int64_t)INT32_MAX, "%s expects 0 <= M < 2^31", op);
  TFGPC_REQUIRE(act == 0 || act == 1, "%s expects activation 0 (leaky ReLU) or 1 (ELU)", op);
  return TFGPC_OK;
}

#define TFGPC_K_SWITCH(K, ...)                              \
  switch (K) {                                              \
    case 8: { constexpr int kK = 8; __VA_ARGS__; } break;   \
    case 16: { constexpr int kK = 16; __VA_ARGS__; } break; \
    case 32: { constexpr int kK = 32; __VA_ARGS__; } break; \
    default: { constexpr int kK = 64; __VA_ARGS__; } break; \
  }

}  // namespace
}  // namespace tfgpc

using namespace tfgpc;

extern "C" int tfgpc_kernel_basis(void* stream, int D, int K, int64_t M, const float* points_in,
                                  const float* points_out, const int32_t* neighbors,
                                  const float* pdf, const float* w1, const float* b1,
                                  float inv_radius, int activation, float alpha,
                                  float* basis_out) {
  int rc = check_kb_args("KernelBasis", D, K, M, activation);
  if (rc) return rc;
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && pdf && w1 && b1 && basis_out,
                "KernelBasis got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis_out % 16 == 0, "KernelBasis expects a 16-byte aligned output");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(M, kKbThreads), (unsigned)(sm_count() * 16));
  ProfScope prof(st, "kernel_basis");
  if ((uintptr_t)basis_out % 32 == 0) {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_kernel<kD, kK, true><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_out)));
  } else {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_kernel<kD, kK, false><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_out)));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_kernel_basis_grads(void* stream, int D, int K, int64_t M,
                                        const float* points_in, const float* points_out,
                                        const int32_t* neighbors, const float* pdf,
                                        const float* w1, const float* b1, float inv_radius,
                                        int activation, float alpha, const float* basis_grads,
                                        float* dw1_out, float* db1_out) {
  int rc = check_kb_args("KernelBasisGrads", D, K, M, activation);
  if (rc) return rc;
  TFGPC_REQUIRE(dw1_out && db1_out, "KernelBasisGrads got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  TFGPC_CUDA(cudaMemsetAsync(dw1_out, 0, sizeof(float) * (size_t)D * K, st));
  TFGPC_CUDA(cudaMemsetAsync(db1_out, 0, sizeof(float) * (size_t)K, st));
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && pdf && w1 && b1 && basis_grads,
                "KernelBasisGrads got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis_grads % 16 == 0,
                "KernelBasisGrads expects 16-byte aligned gradients");
  const int kt = K < kKTile ? K : kKTile;
  dim3 grid(min(blocks_for(M, kKbThreads), (unsigned)(sm_count() * 8)), (unsigned)(K / kt));
  ProfScope prof(st, "kernel_basis_grads");
  if ((uintptr_t)basis_grads % 32 == 0) {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_grads_kernel<kD, kK, true><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_grads, dw1_out, db1_out)));
  } else {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_grads_kernel<kD, kK, false><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_grads, dw1_out, db1_out)));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
