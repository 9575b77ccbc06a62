// Kernel MLP of the Monte-Carlo convolution with any number of hidden layers,
// and ALL of its gradients (weights, biases, point coordinates, densities).
//
// MCConv.py:163-171 runs num_mlps independent MLPs on the relative neighbor
// position: layer l of MLP g maps H_{l-1} values to H_l values (H_0 = D), every
// layer is followed by the activation, the last layer's outputs of all MLPs are
// concatenated (column g * H_last + h) and divided by the pair's density:
//   diff = (p_in[j] - p_out[s]) * inv_radius                      (MCConv.py:264-269)
//   a_0 = diff, a_l = act(a_{l-1} W_l[g] + b_l[g]), basis[m, g H + h] = a_L[h] / pdf[m]
// kernel_basis.cu holds the fast path for one hidden layer and the weight
// gradients only; this file is the general path: one thread per pair walks the
// MLPs with its activations in local arrays.  The backward pass recomputes the
// activations, back-propagates dbasis, and adds
//   * the weight and bias gradients: reduced over the warp by shuffles, then over
//     the block in shared memory, one global atomic per value and block;
//   * the gradient of the point coordinates (MCConv's inputs are the positions:
//     monte_carlo_conv_test.py:182-219 checks this jacobian): +d_diff / radius to
//     the neighbor's row of points_in, -d_diff / radius to the sample's row of
//     points_out, by atomics;
//   * the gradient of the density, d_pdf[m] = -sum_k dbasis[m,k] basis[m,k] / pdf[m],
//     which the caller carries on through ComputePdfPtGrads.
#include "common.cuh"

namespace tfgpc {
namespace {

constexpr int kMlpThreads = 128;
constexpr int kMaxLayers = 4;
constexpr int kMaxWidth = 64;
constexpr int kMaxParams = 8192;     // floats of all weights and biases (32 KB of shared memory)

struct MlpShape {
  int D, G, L;
  int h[kMaxLayers + 1];       // h[0] = D, h[l] = width of layer l
  int w_off[kMaxLayers];       // offset of layer l's weights [G][h[l-1]][h[l]] in the parameter block
  int b_off[kMaxLayers];       // offset of layer l's biases [G][h[l]]
  int params;                  // floats in the parameter block (weights of all layers, then biases)
};

__device__ __forceinline__ float act_fwd(float x, int act, float alpha) {
  if (act == 1) return x > 0.0f ? x : expm1f(x);
  return x > 0.0f ? x : x * alpha;
}

__device__ __forceinline__ float act_bwd(float x, int act, float alpha) {
  if (act == 1) return x > 0.0f ? 1.0f : expf(x);
  return x > 0.0f ? 1.0f : alpha;
}

__device__ __forceinline__ void load_params(const MlpShape& s, const float* __restrict__ weights,
                                            const float* __restrict__ biases, float* par) {
  const int nw = s.b_off[0];   // biases follow the weights
  for (int i = threadIdx.x; i < s.params; i += kMlpThreads)
    par[i] = i < nw ? __ldg(weights + i) : __ldg(biases + i - nw);
}

__global__ void __launch_bounds__(kMlpThreads)
kernel_mlp_basis_kernel(MlpShape s, int64_t M, const float* __restrict__ p_in,
                        const float* __restrict__ p_out, const int2* __restrict__ neigh,
                        const float* __restrict__ pdf, const float* __restrict__ weights,
                        const float* __restrict__ biases, float inv_radius, int act, float alpha,
                        int pdf_by_nbr, float* __restrict__ basis) {
  extern __shared__ float par[];
  load_params(s, weights, biases, par);
  __syncthreads();
  const int k_total = s.G * s.h[s.L];
  for (int64_t m = (int64_t)blockIdx.x * kMlpThreads + threadIdx.x; m < M;
       m += (int64_t)gridDim.x * kMlpThreads) {
    const int2 nb = __ldg(neigh + m);
    float diff[TFGPC_MAX_DIMS];
    for (int d = 0; d < s.D; ++d)
      diff[d] = (__ldg(p_in + (int64_t)nb.x * s.D + d) - __ldg(p_out + (int64_t)nb.y * s.D + d)) *
                inv_radius;
    const float inv_pdf = 1.0f / __ldg(pdf + (pdf_by_nbr ? (int64_t)nb.x : m));
    for (int g = 0; g < s.G; ++g) {
      float a[kMaxWidth], b[kMaxWidth];
      for (int d = 0; d < s.D; ++d) a[d] = diff[d];
      for (int l = 1; l <= s.L; ++l) {
        const int hi = s.h[l - 1], ho = s.h[l];
        const float* w = par + s.w_off[l - 1] + g * hi * ho;
        const float* bb = par + s.b_off[l - 1] + g * ho;
        for (int j = 0; j < ho; ++j) {
          float pre = bb[j];
          for (int i = 0; i < hi; ++i) pre = fmaf(a[i], w[i * ho + j], pre);
          b[j] = act_fwd(pre, act, alpha);
        }
        for (int j = 0; j < ho; ++j) a[j] = b[j];
      }
      float* dst = basis + m * k_total + g * s.h[s.L];
      for (int j = 0; j < s.h[s.L]; ++j) dst[j] = a[j] * inv_pdf;
    }
  }
}

__global__ void __launch_bounds__(kMlpThreads)
kernel_mlp_grads_kernel(MlpShape s, int64_t M, const float* __restrict__ p_in,
                        const float* __restrict__ p_out, const int2* __restrict__ neigh,
                        const float* __restrict__ pdf, const float* __restrict__ weights,
                        const float* __restrict__ biases, float inv_radius, int act, float alpha,
                        int pdf_by_nbr, const float* __restrict__ dbasis,
                        float* __restrict__ dweights,
                        float* __restrict__ dbiases, float* __restrict__ dp_in,
                        float* __restrict__ dp_out, float* __restrict__ dpdf) {
  extern __shared__ float smem[];
  float* par = smem;                 // parameters
  float* acc = smem + s.params;      // their gradients, summed over the block
  load_params(s, weights, biases, par);
  for (int i = threadIdx.x; i < s.params; i += kMlpThreads) acc[i] = 0.0f;
  __syncthreads();
  const int k_total = s.G * s.h[s.L];
  const int lane = threadIdx.x & 31;
  // whole warps iterate together (the shuffles below need all lanes): the loop
  // bound is rounded up to the warp, lanes beyond M contribute zeros
  const int64_t stride = (int64_t)gridDim.x * kMlpThreads;
  for (int64_t m0 = (int64_t)blockIdx.x * kMlpThreads + (threadIdx.x & ~31); m0 < M; m0 += stride) {
    const int64_t m = m0 + lane;
    const bool live = m < M;
    int2 nb = make_int2(0, 0);
    float diff[TFGPC_MAX_DIMS], ddiff[TFGPC_MAX_DIMS];
    float inv_pdf = 0.0f, dpdf_m = 0.0f;
    if (live) {
      nb = __ldg(neigh + m);
      inv_pdf = 1.0f / __ldg(pdf + (pdf_by_nbr ? (int64_t)nb.x : m));
    }
    for (int d = 0; d < s.D; ++d) {
      diff[d] = live ? (__ldg(p_in + (int64_t)nb.x * s.D + d) - __ldg(p_out + (int64_t)nb.y * s.D + d)) *
                           inv_radius : 0.0f;
      ddiff[d] = 0.0f;
    }
    for (int g = 0; g < s.G; ++g) {
      // forward with every layer's input and pre-activation kept
      float a[kMaxLayers + 1][kMaxWidth], pre[kMaxLayers][kMaxWidth];
      for (int d = 0; d < s.D; ++d) a[0][d] = diff[d];
      for (int l = 1; l <= s.L; ++l) {
        const int hi = s.h[l - 1], ho = s.h[l];
        const float* w = par + s.w_off[l - 1] + g * hi * ho;
        const float* bb = par + s.b_off[l - 1] + g * ho;
        for (int j = 0; j < ho; ++j) {
          float p = bb[j];
          for (int i = 0; i < hi; ++i) p = fmaf(a[l - 1][i], w[i * ho + j], p);
          pre[l - 1][j] = p;
          a[l][j] = act_fwd(p, act, alpha);
        }
      }
      // gradient of the last layer's output: dbasis / pdf; the density's own
      // gradient: basis = a_L / pdf  ->  d/dpdf = -a_L / pdf^2
      float grad[kMaxWidth], gprev[kMaxWidth];
      const int hl = s.h[s.L];
      for (int j = 0; j < hl; ++j) {
        const float gb = live ? __ldg(dbasis + m * k_total + g * hl + j) : 0.0f;
        grad[j] = gb * inv_pdf;
        dpdf_m -= gb * a[s.L][j] * inv_pdf * inv_pdf;
      }
      for (int l = s.L; l >= 1; --l) {
        const int hi = s.h[l - 1], ho = s.h[l];
        const float* w = par + s.w_off[l - 1] + g * hi * ho;
        float* dw = acc + s.w_off[l - 1] + g * hi * ho;
        float* db = acc + s.b_off[l - 1] + g * ho;
        for (int j = 0; j < ho; ++j) {
          grad[j] *= act_bwd(pre[l - 1][j], act, alpha);      // now d(pre-activation)
          const float t = warp_sum(grad[j]);
          if (lane == 0) atomicAdd(db + j, t);
        }
        for (int i = 0; i < hi; ++i) {
          float back = 0.0f;
          for (int j = 0; j < ho; ++j) {
            const float t = warp_sum(a[l - 1][i] * grad[j]);
            if (lane == 0) atomicAdd(dw + i * ho + j, t);
            back = fmaf(grad[j], w[i * ho + j], back);
          }
          gprev[i] = back;
        }
        for (int i = 0; i < hi; ++i) grad[i] = gprev[i];
      }
      for (int d = 0; d < s.D; ++d) ddiff[d] += grad[d];
    }
    if (live) {
      if (dpdf) dpdf[m] = dpdf_m;
      for (int d = 0; d < s.D; ++d) {
        const float v = ddiff[d] * inv_radius;
        if (dp_in) atomicAdd(dp_in + (int64_t)nb.x * s.D + d, v);
        if (dp_out) atomicAdd(dp_out + (int64_t)nb.y * s.D + d, -v);
      }
    }
  }
  __syncthreads();
  const int nw = s.b_off[0];
  for (int i = threadIdx.x; i < s.params; i += kMlpThreads) {
    if (i < nw) atomicAdd(dweights + i, acc[i]);
    else atomicAdd(dbiases + i - nw, acc[i]);
  }
}

int make_shape(const char* op, int D, int G, int L, const int32_t* layer_sizes, MlpShape* out) {
  TFGPC_REQUIRE(valid_dims(D), "%s expects a valid number of dimension (got %d)", op, D);
  TFGPC_REQUIRE(G >= 1 && L >= 1 && L <= kMaxLayers && layer_sizes,
                "%s expects 1 to %d hidden layers and at least one MLP", op, kMaxLayers);
  MlpShape s;
  s.D = D; s.G = G; s.L = L; s.h[0] = D;
  int off = 0;
  for (int l = 0; l < L; ++l) {
    TFGPC_REQUIRE(layer_sizes[l] >= 1 && layer_sizes[l] <= kMaxWidth,
                  "%s expects hidden layers of 1 to %d units", op, kMaxWidth);
    s.h[l + 1] = layer_sizes[l];
    s.w_off[l] = off;
    off += G * s.h[l] * s.h[l + 1];
  }
  for (int l = 0; l < L; ++l) {
    s.b_off[l] = off;
    off += G * s.h[l + 1];
  }
  for (int l = L + 1; l <= kMaxLayers; ++l) s.h[l] = 0;
  for (int l = L; l < kMaxLayers; ++l) { s.w_off[l] = 0; s.b_off[l] = 0; }
  s.params = off;
  TFGPC_REQUIRE(off <= kMaxParams, "%s: the kernel MLPs hold %d parameters, at most %d are supported",
                op, off, kMaxParams);
  *out = s;
  return TFGPC_OK;
}

}  // namespace
}  // namespace tfgpc

using namespace tfgpc;

extern "C" int tfgpc_kernel_mlp_basis(void* stream, int D, int num_mlps, int num_layers,
                                      const int32_t* layer_sizes, int64_t M,
                                      const float* points_in, const float* points_out,
                                      const int32_t* neighbors, const float* pdf,
                                      const float* weights, const float* biases, float inv_radius,
                                      int activation, float alpha, int pdf_by_neighbor,
                                      float* basis_out) {
  MlpShape s;
  int rc = make_shape("KernelMlpBasis", D, num_mlps, num_layers, layer_sizes, &s);
  if (rc) return rc;
  TFGPC_REQUIRE(M >= 0 && M <= (int64_t)INT32_MAX, "KernelMlpBasis expects 0 <= M < 2^31");
  TFGPC_REQUIRE(activation == 0 || activation == 1,
                "KernelMlpBasis expects activation 0 (leaky ReLU) or 1 (ELU)");
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && pdf && weights && biases && basis_out,
                "KernelMlpBasis got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = min(blocks_for(M, kMlpThreads), (unsigned)(sm_count() * 16));
  ProfScope prof(st, "kernel_mlp_basis");
  kernel_mlp_basis_kernel<<<grid, kMlpThreads, sizeof(float) * (size_t)s.params, st>>>(
      s, M, points_in, points_out, (const int2*)neighbors, pdf, weights, biases, inv_radius,
      activation, alpha, pdf_by_neighbor, basis_out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

extern "C" int tfgpc_kernel_mlp_grads(void* stream, int D, int num_mlps, int num_layers,
                                      const int32_t* layer_sizes, int64_t M, int64_t n_in,
                                      int64_t ns, const float* points_in, const float* points_out,
                                      const int32_t* neighbors, const float* pdf,
                                      const float* weights, const float* biases, float inv_radius,
                                      int activation, float alpha, int pdf_by_neighbor,
                                      const float* basis_grads, float* dweights_out,
                                      float* dbiases_out,
                                      float* dpoints_in_out, float* dpoints_out_out,
                                      float* dpdf_out) {
  MlpShape s;
  int rc = make_shape("KernelMlpGrads", D, num_mlps, num_layers, layer_sizes, &s);
  if (rc) return rc;
  TFGPC_REQUIRE(M >= 0 && M <= (int64_t)INT32_MAX && n_in >= 0 && ns >= 0,
                "KernelMlpGrads expects 0 <= M < 2^31 and non-negative point counts");
  TFGPC_REQUIRE(activation == 0 || activation == 1,
                "KernelMlpGrads expects activation 0 (leaky ReLU) or 1 (ELU)");
  TFGPC_REQUIRE(dweights_out && dbiases_out, "KernelMlpGrads got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int nw = s.b_off[0];
  TFGPC_CUDA(cudaMemsetAsync(dweights_out, 0, sizeof(float) * (size_t)nw, st));
  TFGPC_CUDA(cudaMemsetAsync(dbiases_out, 0, sizeof(float) * (size_t)(s.params - nw), st));
  // points_in and points_out may be one cloud: its gradient is then one array
  // that both roles add into
  if (dpoints_in_out)
    TFGPC_CUDA(cudaMemsetAsync(dpoints_in_out, 0, sizeof(float) * (size_t)n_in * D, st));
  if (dpoints_out_out && dpoints_out_out != dpoints_in_out)
    TFGPC_CUDA(cudaMemsetAsync(dpoints_out_out, 0, sizeof(float) * (size_t)ns * D, st));
  if (M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(points_in && points_out && neighbors && pdf && weights && biases && basis_grads,
                "KernelMlpGrads got a null pointer");
  const size_t smem = sizeof(float) * 2 * (size_t)s.params;
  TFGPC_CUDA(cudaFuncSetAttribute(kernel_mlp_grads_kernel,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  unsigned grid = min(blocks_for(M, kMlpThreads), (unsigned)(sm_count() * 8));
  ProfScope prof(st, "kernel_mlp_grads");
  kernel_mlp_grads_kernel<<<grid, kMlpThreads, smem, st>>>(
      s, M, points_in, points_out, (const int2*)neighbors, pdf, weights, biases, inv_radius,
      activation, alpha, pdf_by_neighbor, basis_grads, dweights_out, dbiases_out, dpoints_in_out,
      dpoints_out_out, dpdf_out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
