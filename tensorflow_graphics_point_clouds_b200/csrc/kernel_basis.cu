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
#include "basis_proj.cuh"

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

// diff and 1 / density of pair m.  pdf_mode 0: density per pair, 1: a table with
// one density per point of p_in, 2 (D == 3): p_in is the packed table of
// pack_points_density_kernel, (x, y, z, 1 / density) per point -- ONE 16-byte
// gather per pair in place of three coordinate loads and a density load, which
// matters because these kernels are bound by the number of scattered loads a warp
// issues, not by bytes.
template <int D>
__device__ __forceinline__ float pair_inputs(const float* __restrict__ p_in,
                                             const float* __restrict__ p_out,
                                             const float* __restrict__ pdf, int2 nb, int64_t m,
                                             float inv_radius, int pdf_mode, float* diff) {
  if (D == 3 && pdf_mode == 2) {
    const float4 pp = __ldg(reinterpret_cast<const float4*>(p_in) + nb.x);
    const float* q = p_out + (int64_t)nb.y * 3;
    diff[0] = (pp.x - __ldg(q)) * inv_radius;
    diff[1] = (pp.y - __ldg(q + 1)) * inv_radius;
    diff[2] = (pp.z - __ldg(q + 2)) * inv_radius;
    return pp.w;
  }
  pair_diff<D>(p_in, p_out, nb, inv_radius, diff);
  return 1.0f / __ldg(pdf + (pdf_mode ? (int64_t)nb.x : m));
}

__global__ void pack_points_density_kernel(int64_t n, const float* __restrict__ pts,
                                           const float* __restrict__ pdf,
                                           float4* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[i] = make_float4(__ldg(pts + 3 * i), __ldg(pts + 3 * i + 1), __ldg(pts + 3 * i + 2),
                       1.0f / __ldg(pdf + i));
}

// WIDE: rows are 32-byte aligned, 256-bit accesses are allowed.
template <int D, int K, bool WIDE>
__global__ void __launch_bounds__(kKbThreads)
kernel_basis_kernel(int64_t M, const float* __restrict__ p_in, const float* __restrict__ p_out,
                    const int2* __restrict__ neigh, const float* __restrict__ pdf,
                    const float* __restrict__ w1, const float* __restrict__ b1, float inv_radius,
                    int act, float alpha, float* __restrict__ basis,
                    __nv_bfloat16* __restrict__ pair, int pdf_by_nbr) {
  __shared__ float w_s[D * K + K];
  for (int i = threadIdx.x; i < D * K + K; i += kKbThreads)
    w_s[i] = i < D * K ? __ldg(w1 + i) : __ldg(b1 + i - D * K);
  __syncthreads();
  for (int64_t m = (int64_t)blockIdx.x * kKbThreads + threadIdx.x; m < M;
       m += (int64_t)gridDim.x * kKbThreads) {
    const int2 nb = __ldg(neigh + m);
    float diff[D];
    const float inv_pdf = pair_inputs<D>(p_in, p_out, pdf, nb, m, inv_radius, pdf_by_nbr, diff);
    float* dst = basis + m * K;
    uint4 pr[K / 4];   // hi chunks, then mid chunks, of the bf16 pair
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
      if (!basis) {
      } else if (WIDE) {
        st_global_256(dst + 8 * q, v);
      } else {
        reinterpret_cast<float4*>(dst)[2 * q] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[2 * q + 1] = make_float4(v[4], v[5], v[6], v[7]);
      }
      if (pair) {
        // the same row as bf16 hi / mid terms: [m][hi K | mid K]
        split2_bf16(v[0], v[1], pr[q].x, pr[K / 8 + q].x);
        split2_bf16(v[2], v[3], pr[q].y, pr[K / 8 + q].y);
        split2_bf16(v[4], v[5], pr[q].z, pr[K / 8 + q].z);
        split2_bf16(v[6], v[7], pr[q].w, pr[K / 8 + q].w);
      }
    }
    if (pair) {
      // whole 32-byte sectors per store
      uint8_t* prow = reinterpret_cast<uint8_t*>(pair + m * (2 * K));
#pragma unroll
      for (int i = 0; i < K / 8; ++i)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"l"(prow + 32 * i), "r"(pr[2 * i].x), "r"(pr[2 * i].y), "r"(pr[2 * i].z),
                       "r"(pr[2 * i].w), "r"(pr[2 * i + 1].x), "r"(pr[2 * i + 1].y),
                       "r"(pr[2 * i + 1].z), "r"(pr[2 * i + 1].w) : "memory");
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
                          float* __restrict__ db1, int pdf_by_nbr) {
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
    const float inv_pdf = pair_inputs<D>(p_in, p_out, pdf, nb, m, inv_radius, pdf_by_nbr, diff);
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

// Kernel-point correlation of KPConv (KPConv.py:194-212): per neighbor pair
//   basis[m, k] = weighting(|diff - kp[k]|, sigma)   for k < num_kp, 0 above
// with weighting = max(0, 1 - dist / sigma) (linear, KPConv.py:28-40) or
// exp(-(dist / (sigma / 3))^2) (gaussian, :43-56).  The columns from num_kp up to
// K are the zero padding the reference adds with tf.pad to reach a basis count
// the projection accepts.
constexpr int kMaxKernelPoints = 64;

template <int D, int K, bool WIDE>
__global__ void __launch_bounds__(kKbThreads)
kp_basis_kernel(int64_t M, int num_kp, const float* __restrict__ p_in,
                const float* __restrict__ p_out, const int2* __restrict__ neigh,
                const float* __restrict__ kernel_points, float inv_radius, float sigma,
                int interpolation, float* __restrict__ basis) {
  __shared__ float kp_s[kMaxKernelPoints * D];
  for (int i = threadIdx.x; i < num_kp * D; i += kKbThreads) kp_s[i] = __ldg(kernel_points + i);
  __syncthreads();
  const float gauss_sigma = sigma / 3.0f;
  for (int64_t m = (int64_t)blockIdx.x * kKbThreads + threadIdx.x; m < M;
       m += (int64_t)gridDim.x * kKbThreads) {
    const int2 nb = __ldg(neigh + m);
    float diff[D];
    pair_diff<D>(p_in, p_out, nb, inv_radius, diff);
    float* dst = basis + m * K;
#pragma unroll
    for (int q = 0; q < K / 8; ++q) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int k = 8 * q + i;
        float w = 0.0f;
        if (k < num_kp) {
          float d2 = 0.0f;
#pragma unroll
          for (int d = 0; d < D; ++d) {
            const float t = diff[d] - kp_s[k * D + d];
            d2 = fmaf(t, t, d2);
          }
          const float dist = sqrtf(d2);
          if (interpolation == 0) {
            w = fmaxf(1.0f - dist / sigma, 0.0f);
          } else {
            const float r = dist / gauss_sigma;
            w = expf(-(r * r));
          }
        }
        v[i] = w;
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

// Density transform of PointConv (PointConv.py:168-183): per sample the largest
// density among its neighbor pairs, then per pair
//   out[m] = sum_j relu(pdf[m] / max * w1[j] + b1[j]) * w2[j] + b2      (j < 16)
// One warp owns one sample; its pairs are contiguous (ranges holds their end).
constexpr int kPdfHidden = 16;

__global__ void __launch_bounds__(kKbThreads)
pointconv_pdf_kernel(int64_t ns, const int32_t* __restrict__ ranges,
                     const float* __restrict__ pdf, const float* __restrict__ w1,
                     const float* __restrict__ b1, const float* __restrict__ w2,
                     const float* __restrict__ b2, float* __restrict__ out) {
  __shared__ float par[3 * kPdfHidden + 1];
  for (int i = threadIdx.x; i < 3 * kPdfHidden + 1; i += kKbThreads)
    par[i] = i < kPdfHidden ? __ldg(w1 + i)
             : i < 2 * kPdfHidden ? __ldg(b1 + i - kPdfHidden)
             : i < 3 * kPdfHidden ? __ldg(w2 + i - 2 * kPdfHidden) : __ldg(b2);
  __syncthreads();
  const int lane = lane_id();
  const int64_t warps = ((int64_t)gridDim.x * kKbThreads) >> 5;
  for (int64_t s = ((int64_t)blockIdx.x * kKbThreads + threadIdx.x) >> 5; s < ns; s += warps) {
    const int a = s ? __ldg(ranges + s - 1) : 0;
    const int e = __ldg(ranges + s);
    float mx = -INFINITY;
    for (int m = a + lane; m < e; m += 32) mx = fmaxf(mx, __ldg(pdf + m));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int m = a + lane; m < e; m += 32) {
      const float x = __ldg(pdf + m) / mx;
      float acc = 0.0f;
#pragma unroll
      for (int j = 0; j < kPdfHidden; ++j)
        acc = fmaf(fmaxf(fmaf(x, par[j], par[kPdfHidden + j]), 0.0f), par[2 * kPdfHidden + j], acc);
      out[m] = acc + par[3 * kPdfHidden];
    }
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

static int check_pdf_mode(const char* op, int D, int mode, const float* points_in) {
  TFGPC_REQUIRE(mode >= 0 && mode <= 2, "%s expects pdf_by_neighbor 0, 1 or 2", op);
  TFGPC_REQUIRE(mode != 2 || (D == 3 && (uintptr_t)points_in % 16 == 0),
                "%s: the packed point table (pdf_by_neighbor 2) needs D == 3 and 16-byte alignment",
                op);
  return TFGPC_OK;
}

extern "C" int tfgpc_pack_points_density(void* stream, int64_t n, const float* points,
                                         const float* pdf, float* packed_out) {
  TFGPC_REQUIRE(n >= 0 && n < (int64_t)INT32_MAX, "PackPointsDensity expects 0 <= n < 2^31");
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && pdf && packed_out, "PackPointsDensity got a null pointer");
  TFGPC_REQUIRE((uintptr_t)packed_out % 16 == 0, "PackPointsDensity expects a 16-byte aligned output");
  cudaStream_t st = (cudaStream_t)stream;
  ProfScope prof(st, "pack_points_density");
  pack_points_density_kernel<<<blocks_for(n, 256), 256, 0, st>>>(n, points, pdf,
                                                               (float4*)packed_out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

static int kernel_basis_impl(void* stream, int D, int K, int64_t M, const float* points_in,
                             const float* points_out, const int32_t* neighbors, const float* pdf,
                             const float* w1, const float* b1, float inv_radius, int activation,
                             float alpha, float* basis_out, __nv_bfloat16* pair_out,
                             int pdf_by_nbr) {
  int rc = check_kb_args("KernelBasis", D, K, M, activation);
  if (rc) return rc;
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && (pdf || pdf_by_nbr == 2) && w1 && b1 &&
                (basis_out || pair_out), "KernelBasis got a null pointer");
  rc = check_pdf_mode("KernelBasis", D, pdf_by_nbr, points_in);
  if (rc) return rc;
  TFGPC_REQUIRE((uintptr_t)basis_out % 16 == 0 && (uintptr_t)pair_out % 32 == 0,
                "KernelBasis expects 16-byte aligned outputs (32 for the bf16 pair)");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(M, kKbThreads), (unsigned)(sm_count() * 16));
  ProfScope prof(st, "kernel_basis");
  if ((uintptr_t)basis_out % 32 == 0) {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_kernel<kD, kK, true><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_out, pair_out, pdf_by_nbr)));
  } else {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_kernel<kD, kK, false><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_out, pair_out, pdf_by_nbr)));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_kernel_basis(void* stream, int D, int K, int64_t M, const float* points_in,
                                  const float* points_out, const int32_t* neighbors,
                                  const float* pdf, const float* w1, const float* b1,
                                  float inv_radius, int activation, float alpha,
                                  int pdf_by_neighbor, float* basis_out) {
  return kernel_basis_impl(stream, D, K, M, points_in, points_out, neighbors, pdf, w1, b1,
                           inv_radius, activation, alpha, basis_out, nullptr, pdf_by_neighbor);
}

extern "C" int tfgpc_kernel_basis_split(void* stream, int D, int K, int64_t M,
                                        const float* points_in, const float* points_out,
                                        const int32_t* neighbors, const float* pdf,
                                        const float* w1, const float* b1, float inv_radius,
                                        int activation, float alpha, int pdf_by_neighbor,
                                        float* basis_out, void* basis_pair_out) {
  TFGPC_REQUIRE(M == 0 || basis_pair_out, "KernelBasis got a null pointer");
  return kernel_basis_impl(stream, D, K, M, points_in, points_out, neighbors, pdf, w1, b1,
                           inv_radius, activation, alpha, basis_out,
                           (__nv_bfloat16*)basis_pair_out, pdf_by_neighbor);
}

extern "C" int tfgpc_kernel_basis_grads(void* stream, int D, int K, int64_t M,
                                        const float* points_in, const float* points_out,
                                        const int32_t* neighbors, const float* pdf,
                                        const float* w1, const float* b1, float inv_radius,
                                        int activation, float alpha, int pdf_by_neighbor,
                                        const float* basis_grads, float* dw1_out,
                                        float* db1_out) {
  int rc = check_kb_args("KernelBasisGrads", D, K, M, activation);
  if (rc) return rc;
  TFGPC_REQUIRE(dw1_out && db1_out, "KernelBasisGrads got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  TFGPC_CUDA(cudaMemsetAsync(dw1_out, 0, sizeof(float) * (size_t)D * K, st));
  TFGPC_CUDA(cudaMemsetAsync(db1_out, 0, sizeof(float) * (size_t)K, st));
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && (pdf || pdf_by_neighbor == 2) && w1 &&
                b1 && basis_grads, "KernelBasisGrads got a null pointer");
  rc = check_pdf_mode("KernelBasisGrads", D, pdf_by_neighbor, points_in);
  if (rc) return rc;
  TFGPC_REQUIRE((uintptr_t)basis_grads % 16 == 0,
                "KernelBasisGrads expects 16-byte aligned gradients");
  const int kt = K < kKTile ? K : kKTile;
  dim3 grid(min(blocks_for(M, kKbThreads), (unsigned)(sm_count() * 8)), (unsigned)(K / kt));
  ProfScope prof(st, "kernel_basis_grads");
  if ((uintptr_t)basis_grads % 32 == 0) {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_grads_kernel<kD, kK, true><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_grads, dw1_out, db1_out, pdf_by_neighbor)));
  } else {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kernel_basis_grads_kernel<kD, kK, false><<<grid, kKbThreads, 0, st>>>(
        M, points_in, points_out, (const int2*)neighbors, pdf, w1, b1, inv_radius, activation,
        alpha, basis_grads, dw1_out, db1_out, pdf_by_neighbor)));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_kp_basis(void* stream, int D, int K, int num_kernel_points, int64_t M,
                              const float* points_in, const float* points_out,
                              const int32_t* neighbors, const float* kernel_points,
                              float inv_radius, float sigma, int interpolation,
                              float* basis_out) {
  int rc = check_kb_args("KPBasis", D, K, M, 0);
  if (rc) return rc;
  TFGPC_REQUIRE(num_kernel_points >= 1 && num_kernel_points <= K,
                "KPBasis expects 1 <= kernel points <= basis functions");
  TFGPC_REQUIRE(interpolation == 0 || interpolation == 1,
                "KPBasis expects interpolation 0 (linear) or 1 (gaussian)");
  TFGPC_REQUIRE(sigma > 0.0f && inv_radius > 0.0f, "KPBasis expects a positive sigma and radius");
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && kernel_points && basis_out,
                "KPBasis got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis_out % 16 == 0, "KPBasis expects a 16-byte aligned output");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(M, kKbThreads), (unsigned)(sm_count() * 16));
  ProfScope prof(st, "kp_basis");
  if ((uintptr_t)basis_out % 32 == 0) {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kp_basis_kernel<kD, kK, true><<<grid, kKbThreads, 0, st>>>(
        M, num_kernel_points, points_in, points_out, (const int2*)neighbors, kernel_points,
        inv_radius, sigma, interpolation, basis_out)));
  } else {
    TFGPC_DIM_SWITCH(D, TFGPC_K_SWITCH(K, kp_basis_kernel<kD, kK, false><<<grid, kKbThreads, 0, st>>>(
        M, num_kernel_points, points_in, points_out, (const int2*)neighbors, kernel_points,
        inv_radius, sigma, interpolation, basis_out)));
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_pointconv_pdf(void* stream, int64_t ns, int64_t M, const int32_t* ranges,
                                   const float* pdf, const float* w1, const float* b1,
                                   const float* w2, const float* b2, float* pdf_out) {
  TFGPC_REQUIRE(ns >= 0 && ns < (int64_t)INT32_MAX && M >= 0 && M <= (int64_t)INT32_MAX,
                "PointConvPdf expects 0 <= ns, M < 2^31");
  if (ns == 0 || M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(ranges && pdf && w1 && b1 && w2 && b2 && pdf_out,
                "PointConvPdf got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(ns, kKbThreads / 32), (unsigned)(sm_count() * 16));
  ProfScope prof(st, "pointconv_pdf");
  pointconv_pdf_kernel<<<grid, kKbThreads, 0, st>>>(ns, ranges, pdf, w1, b1, w2, b2, pdf_out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
