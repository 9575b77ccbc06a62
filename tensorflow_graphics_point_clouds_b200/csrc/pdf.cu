// Gaussian kernel density estimate per point over its neighbor list, and the
// gradient of a loss on those densities with respect to the point positions.
//
// One warp owns one point: the lanes stride over the neighbor list (coalesced
// 8-byte index loads, neighbor coordinates gathered from a list that is
// ascending in point index, so mostly from the same cache lines), and the
// partial sums are combined with shuffles.  The reference walks each list with
// a single thread (compute_pdf_kernels.cu.cc:73-130).
#include "common.cuh"

namespace tfgpc {

constexpr int kPdfThreads = 256;
constexpr float kInvSqrt2Pi = 0.39894228f;  // compute_pdf_kernels.cu.cc:111

template <int D>
__device__ __forceinline__ void load_bandwidth(int mode, int64_t n, const float* __restrict__ inv_bw,
                                               const float* __restrict__ inv_r, float* bw, float* ir) {
#pragma unroll
  for (int d = 0; d < D; ++d) {
    // mode 1 uses sqrt(number of points) as the inverse bandwidth
    // (compute_pdf_kernels.cu.cc:47-56, applied with numSamples at :102).
    bw[d] = mode == 1 ? sqrtf((float)n) : __ldg(inv_bw + d);
    ir[d] = __ldg(inv_r + d);
  }
}

template <int D>
__global__ void __launch_bounds__(kPdfThreads)
compute_pdf_kernel(int mode, int64_t n, int64_t n_bw, const float* __restrict__ centers,
                   const float* __restrict__ pts,
                   const int2* __restrict__ neigh, const int32_t* __restrict__ ranges,
                   const float* __restrict__ inv_bw, const float* __restrict__ inv_r,
                   float* __restrict__ pdf_out) {
  float bw[D], ir[D];
  load_bandwidth<D>(mode, n_bw, inv_bw, inv_r, bw, ir);
  const int lane = lane_id();
  const int64_t warps = ((int64_t)gridDim.x * kPdfThreads) >> 5;
  for (int64_t i = ((int64_t)blockIdx.x * kPdfThreads + threadIdx.x) >> 5; i < n; i += warps) {
    const int a = i ? __ldg(ranges + i - 1) : 0;
    const int e = __ldg(ranges + i);
    float p[D];
#pragma unroll
    for (int d = 0; d < D; ++d) p[d] = __ldg(centers + i * D + d);
    float acc = 0.0f;
    for (int m = a + lane; m < e; m += 32) {
      const int j = __ldg(&neigh[m].x);
      float local = 1.0f;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        float t = (__ldg(pts + (int64_t)j * D + d) - p[d]) * bw[d] * ir[d];
        local *= bw[d] * expf(t * t * (-0.5f)) * kInvSqrt2Pi;
      }
      acc += local;
    }
    acc = warp_sum(acc);
    if (lane == 0) pdf_out[i] = acc;
  }
}

// grad[i] += sum_j t_ij * c * w_ij ; grad[j] -= t_ij * c * w_ij with
// w_ij = g_i * prod_d(bw_d * exp(-t_d^2/2) / sqrt(2 pi)), c = bw * inv_r
// (compute_pdf_kernels.cu.cc:187-213).  The point's own sum is reduced in the
// warp and written with one atomic per coordinate; the neighbor terms are
// scattered with fp32 atomics like the reference does.
template <int D>
__global__ void __launch_bounds__(kPdfThreads)
compute_pdf_grads_kernel(int mode, int64_t n, const float* __restrict__ pts,
                         const int2* __restrict__ neigh, const int32_t* __restrict__ ranges,
                         const float* __restrict__ inv_bw, const float* __restrict__ inv_r,
                         const float* __restrict__ pdf_grads, float* __restrict__ grads_out) {
  float bw[D], ir[D];
  load_bandwidth<D>(mode, n, inv_bw, inv_r, bw, ir);
  const int lane = lane_id();
  const int64_t warps = ((int64_t)gridDim.x * kPdfThreads) >> 5;
  for (int64_t i = ((int64_t)blockIdx.x * kPdfThreads + threadIdx.x) >> 5; i < n; i += warps) {
    const int a = i ? __ldg(ranges + i - 1) : 0;
    const int e = __ldg(ranges + i);
    const float g = __ldg(pdf_grads + i);
    float p[D], own[D];
#pragma unroll
    for (int d = 0; d < D; ++d) { p[d] = __ldg(pts + i * D + d); own[d] = 0.0f; }
    for (int m = a + lane; m < e; m += 32) {
      const int j = __ldg(&neigh[m].x);
      float t[D];
      float local = g;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        t[d] = (__ldg(pts + (int64_t)j * D + d) - p[d]) * bw[d] * ir[d];
        local *= bw[d] * expf(t[d] * t[d] * (-0.5f)) * kInvSqrt2Pi;
      }
      if (j != i) {  // the self pair has t == 0: it adds +0 and -0
#pragma unroll
        for (int d = 0; d < D; ++d) {
          float v = t[d] * bw[d] * ir[d] * local;
          own[d] += v;
          atomicAdd(grads_out + (int64_t)j * D + d, -v);
        }
      }
    }
#pragma unroll
    for (int d = 0; d < D; ++d) {
      float v = warp_sum(own[d]);
      if (lane == 0 && v != 0.0f) atomicAdd(grads_out + i * D + d, v);
    }
  }
}

static int check_pdf_args(const char* op, int D, int mode, int64_t n, int64_t M) {
  TFGPC_REQUIRE(valid_dims(D), "%s expects a valid number of dimension (got %d)", op, D);
  TFGPC_REQUIRE(mode == 0 || mode == 1, "%s expects mode 0 or 1 (got %d)", op, mode);
  TFGPC_REQUIRE(n >= 0 && n < (int64_t)INT32_MAX && M >= 0 && M <= (int64_t)INT32_MAX,
                "%s expects 0 <= n, M < 2^31", op);
  return TFGPC_OK;
}

}  // namespace tfgpc

using namespace tfgpc;

extern "C" int tfgpc_compute_pdf(void* stream, int D, int mode, int64_t n, const float* points,
                                 const int32_t* neighbors, int64_t M, const int32_t* ranges,
                                 const float* inv_bandwidth, const float* inv_radii,
                                 float* pdf_out) {
  int rc = check_pdf_args("ComputePdf", D, mode, n, M);
  if (rc) return rc;
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && ranges && inv_bandwidth && inv_radii && pdf_out && (M == 0 || neighbors),
                "ComputePdf got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(n, kPdfThreads / 32), (unsigned)(sm_count() * 32));
  ProfScope prof(st, "compute_pdf");
  TFGPC_DIM_SWITCH(D, compute_pdf_kernel<kD><<<grid, kPdfThreads, 0, st>>>(
      mode, n, n, points, points, (const int2*)neighbors, ranges, inv_bandwidth, inv_radii,
      pdf_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_compute_pdf_at_samples(void* stream, int D, int mode, int64_t ns,
                                            const float* samples, int64_t n, const float* points,
                                            const int32_t* neighbors, int64_t M,
                                            const int32_t* ranges, const float* inv_bandwidth,
                                            const float* inv_radii, float* pdf_out) {
  int rc = check_pdf_args("ComputePdfAtSamples", D, mode, ns, M);
  if (rc) return rc;
  TFGPC_REQUIRE(n >= 0 && n < (int64_t)INT32_MAX, "ComputePdfAtSamples expects 0 <= n < 2^31");
  if (ns == 0) return TFGPC_OK;
  TFGPC_REQUIRE(samples && points && ranges && inv_bandwidth && inv_radii && pdf_out &&
                (M == 0 || neighbors), "ComputePdfAtSamples got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(ns, kPdfThreads / 32), (unsigned)(sm_count() * 32));
  ProfScope prof(st, "compute_pdf");
  TFGPC_DIM_SWITCH(D, compute_pdf_kernel<kD><<<grid, kPdfThreads, 0, st>>>(
      mode, ns, n, samples, points, (const int2*)neighbors, ranges, inv_bandwidth, inv_radii,
      pdf_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_compute_pdf_pt_grads(void* stream, int D, int mode, int64_t n,
                                          const float* points, const int32_t* neighbors,
                                          int64_t M, const int32_t* ranges,
                                          const float* inv_bandwidth, const float* inv_radii,
                                          const float* pdf_grads, float* pt_grads_out) {
  int rc = check_pdf_args("ComputePdfPtGrads", D, mode, n, M);
  if (rc) return rc;
  if (n == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points && ranges && inv_bandwidth && inv_radii && pdf_grads && pt_grads_out &&
                (M == 0 || neighbors), "ComputePdfPtGrads got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  TFGPC_CUDA(cudaMemsetAsync(pt_grads_out, 0, sizeof(float) * (size_t)n * D, st));
  unsigned grid = min(blocks_for(n, kPdfThreads / 32), (unsigned)(sm_count() * 32));
  ProfScope prof(st, "compute_pdf_grads");
  TFGPC_DIM_SWITCH(D, compute_pdf_grads_kernel<kD><<<grid, kPdfThreads, 0, st>>>(
      mode, n, points, (const int2*)neighbors, ranges, inv_bandwidth, inv_radii, pdf_grads,
      pt_grads_out));
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
