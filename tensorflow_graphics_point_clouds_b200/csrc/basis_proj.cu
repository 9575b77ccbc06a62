// Basis projection: out[s, c, k] = sum over the sample's neighbor range of
// basis[m, k] * features[neighbor(m), c], and its two gradients.
//
// A group of G lanes (G = 32 for wide layers) owns one sample; every lane keeps
// a CPL x K tile of the [C, K] result in registers, so one neighbor costs one
// 16-byte feature load per lane (a coalesced row read for the group), K/4
// broadcast loads of the basis row and CPL*K FMAs, with no shared-memory
// traffic and no barriers in the neighbor loop.  (The reference: one 64-thread
// block per (sample, 8 channels), two __syncthreads per neighbor step,
// basis_proj_kernels.cu.cc:30-127.)
#include "basis_proj.cuh"
#include "basis_proj_wide.cuh"

namespace tfgpc {

constexpr int kBpThreads = 256;

template <int K, bool VEC>
__device__ __forceinline__ void load_features(const float* __restrict__ row, int cbase, int C,
                                              float* f) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  if (VEC) {
    if (cbase < C) {
      float4 v = __ldg(reinterpret_cast<const float4*>(row + cbase));
      f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else {
      f[0] = f[1] = f[2] = f[3] = 0.0f;
    }
  } else {
#pragma unroll
    for (int cc = 0; cc < kCpl; ++cc) f[cc] = (cbase + cc < C) ? __ldg(row + cbase + cc) : 0.0f;
  }
}

template <int K>
__device__ __forceinline__ void load_basis_row(const float* __restrict__ row, float* w) {
#pragma unroll
  for (int q = 0; q < K / 4; ++q) {
    float4 v = __ldg(reinterpret_cast<const float4*>(row) + q);
    w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
  }
}

// OUT = 0: fp32 [ns, C, K] (the op's output).  OUT = 1: the same values split
// into two bf16 arrays [ns, C*K] (left operand of the tensor-core GEMM).
template <int K, bool VEC, int OUT>
__global__ void __launch_bounds__(kBpThreads)
basis_proj_kernel(int C, int64_t ns, int G, const float* __restrict__ basis,
                  const float* __restrict__ feat, const int2* __restrict__ neigh,
                  const int32_t* __restrict__ ranges, float* __restrict__ out,
                  __nv_bfloat16* __restrict__ out_hi, __nv_bfloat16* __restrict__ out_mid) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  constexpr int kAcc = BpCfg<K>::kAcc;
  constexpr int kRow = BpCfg<K>::kRow;
  extern __shared__ __align__(16) float stage_all[];  // used when G == 32
  const int lane = lane_id();
  const int gl = lane & (G - 1);
  const int groups_per_warp = 32 / G;
  const int64_t warp0 = ((int64_t)blockIdx.x * kBpThreads + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * kBpThreads) >> 5;
  float* stage = stage_all + (size_t)(threadIdx.x >> 5) * 32 * kRow;
  const int chunk = G * kCpl;
  for (int64_t s0 = warp0 * groups_per_warp; s0 < ns; s0 += warps * groups_per_warp) {
    const int64_t s = s0 + lane / G;
    const bool active = s < ns;
    const int a = (active && s) ? __ldg(ranges + s - 1) : 0;
    const int e = active ? __ldg(ranges + s) : 0;
    for (int c0 = 0; c0 < C; c0 += chunk) {
      const int cbase = c0 + gl * kCpl;
      float acc[kCpl][K];
#pragma unroll
      for (int cc = 0; cc < kCpl; ++cc)
#pragma unroll
        for (int k = 0; k < K; ++k) acc[cc][k] = 0.0f;
      for (int m = a; m < e; ++m) {
        const int j = __ldg(&neigh[m].x);
        float f[kCpl], w[K];
        load_features<K, VEC>(feat + (int64_t)j * C, cbase, C, f);
        load_basis_row<K>(basis + (int64_t)m * K, w);
#pragma unroll
        for (int cc = 0; cc < kCpl; ++cc)
#pragma unroll
          for (int k = 0; k < K; ++k) acc[cc][k] = fmaf(f[cc], w[k], acc[cc][k]);
      }
      if (G == 32) {
        // Stage the warp's 32 x (CPL*K) tile and write it out with contiguous
        // 512-byte warp stores (a lane's own values are CPL*K*4 bytes apart).
        __syncwarp();
#pragma unroll
        for (int q = 0; q < kAcc / 4; ++q)
          *reinterpret_cast<float4*>(stage + lane * kRow + 4 * q) =
              make_float4(acc[(4 * q) / K][(4 * q) % K], acc[(4 * q + 1) / K][(4 * q + 1) % K],
                          acc[(4 * q + 2) / K][(4 * q + 2) % K], acc[(4 * q + 3) / K][(4 * q + 3) % K]);
        __syncwarp();
        const int valid = min(chunk, C - c0) * K;  // floats of this chunk that exist
        const int64_t obase = s * (int64_t)C * K + (int64_t)c0 * K;
        if (active) {
#pragma unroll 4
          for (int f0 = lane * 4; f0 < valid; f0 += 128) {
            float4 v = *reinterpret_cast<const float4*>(stage + (f0 / kAcc) * kRow + (f0 % kAcc));
            if (OUT == 0) {
              *reinterpret_cast<float4*>(out + obase + f0) = v;
            } else {
              __nv_bfloat16 h[4], l[4];
              split_bf16(v.x, h[0], l[0]); split_bf16(v.y, h[1], l[1]);
              split_bf16(v.z, h[2], l[2]); split_bf16(v.w, h[3], l[3]);
              *reinterpret_cast<uint2*>(out_hi + obase + f0) = *reinterpret_cast<uint2*>(h);
              *reinterpret_cast<uint2*>(out_mid + obase + f0) = *reinterpret_cast<uint2*>(l);
            }
          }
        }
      } else if (active) {
#pragma unroll
        for (int cc = 0; cc < kCpl; ++cc) {
          if (cbase + cc < C) {
            const int64_t o = s * (int64_t)C * K + (int64_t)(cbase + cc) * K;
#pragma unroll
            for (int k = 0; k < K; ++k) {
              if (OUT == 0) {
                out[o + k] = acc[cc][k];
              } else {
                __nv_bfloat16 h, l;
                split_bf16(acc[cc][k], h, l);
                out_hi[o + k] = h;
                out_mid[o + k] = l;
              }
            }
          }
        }
      }
    }
  }
}

// Gradients.  The lane keeps its CPL x K tile of the incoming gradient g[s] in
// registers.  Per neighbor: dfeat[nbr, c] += sum_k g[c,k] * basis[m,k] (one
// vector atomic per lane), and dbasis[m, k] = sum_c g[c,k] * feat[nbr,c],
// reduced over the group's lanes with a halving butterfly (K values -> one
// value per lane in log2 steps) and written once when the sample's channels
// fit one pass, else accumulated with atomics.
template <int K, bool VEC>
__global__ void __launch_bounds__(kBpThreads)
basis_proj_grads_kernel(int C, int64_t ns, int G, const float* __restrict__ basis,
                        const float* __restrict__ feat, const int2* __restrict__ neigh,
                        const int32_t* __restrict__ ranges, const float* __restrict__ in_grads,
                        float* __restrict__ dbasis, float* __restrict__ dfeat) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  const int lane = lane_id();
  const int gl = lane & (G - 1);
  const int groups_per_warp = 32 / G;
  const int64_t warp0 = ((int64_t)blockIdx.x * kBpThreads + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * kBpThreads) >> 5;
  const int chunk = G * kCpl;
  const bool single_pass = C <= chunk;
  for (int64_t s0 = warp0 * groups_per_warp; s0 < ns; s0 += warps * groups_per_warp) {
    const int64_t s = s0 + lane / G;
    const bool active = s < ns;
    const int a = (active && s) ? __ldg(ranges + s - 1) : 0;
    const int e = active ? __ldg(ranges + s) : 0;
    // all lanes of the warp run the same number of steps so that the shuffles
    // below stay convergent
    int steps = e - a;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) steps = max(steps, __shfl_xor_sync(0xffffffffu, steps, o));
    for (int c0 = 0; c0 < C; c0 += chunk) {
      const int cbase = c0 + gl * kCpl;
      float g[kCpl][K];
#pragma unroll
      for (int cc = 0; cc < kCpl; ++cc) {
        const bool ok = active && cbase + cc < C;
        const float* src = in_grads + s * (int64_t)C * K + (int64_t)(cbase + cc) * K;
#pragma unroll
        for (int q = 0; q < K / 4; ++q) {
          float4 v = ok ? __ldg(reinterpret_cast<const float4*>(src) + q)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
          g[cc][4 * q] = v.x; g[cc][4 * q + 1] = v.y; g[cc][4 * q + 2] = v.z; g[cc][4 * q + 3] = v.w;
        }
      }
      for (int it = 0; it < steps; ++it) {
        const int m = a + it;
        const bool live = m < e;
        float f[kCpl], w[K], part[K];
        int j = 0;
        if (live) {
          j = __ldg(&neigh[m].x);
          load_features<K, VEC>(feat + (int64_t)j * C, cbase, C, f);
          load_basis_row<K>(basis + (int64_t)m * K, w);
        } else {
#pragma unroll
          for (int cc = 0; cc < kCpl; ++cc) f[cc] = 0.0f;
#pragma unroll
          for (int k = 0; k < K; ++k) w[k] = 0.0f;
        }
        // feature gradient of this lane's channels
        float df[kCpl];
#pragma unroll
        for (int cc = 0; cc < kCpl; ++cc) {
          float accv = 0.0f;
#pragma unroll
          for (int k = 0; k < K; ++k) accv = fmaf(g[cc][k], w[k], accv);
          df[cc] = accv;
        }
        if (live) {
          float* dst = dfeat + (int64_t)j * C + cbase;
          if (VEC) {
            if (cbase < C) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(df[0]),
                           "f"(df[1]), "f"(df[2]), "f"(df[3]) : "memory");
            }
          } else {
#pragma unroll
            for (int cc = 0; cc < kCpl; ++cc)
              if (cbase + cc < C) atomicAdd(dst + cc, df[cc]);
          }
        }
        // basis gradient: partial sums over this lane's channels ...
#pragma unroll
        for (int k = 0; k < K; ++k) {
          float accv = 0.0f;
#pragma unroll
          for (int cc = 0; cc < kCpl; ++cc) accv = fmaf(g[cc][k], f[cc], accv);
          part[k] = accv;
        }
        // ... reduced across the G lanes of the group by a halving butterfly
        // over xor distances 1, 2, 4, ...: at each step a lane hands half of
        // its values to its partner and keeps the other half (lanes with the
        // distance bit set keep the upper half).  With G <= K a lane ends up
        // with K/G finished values; with G > K the remaining steps are plain
        // all-reduces and the lanes gl < K own one value each.
#pragma unroll
        for (int t = 0; t < 5; ++t) {
          const int half = 1 << t;
          if (half < G) {
            const int width = K >> (t + 1);
            if (width >= 1) {
              const bool upper = (gl & half) != 0;
#pragma unroll
              for (int k = 0; k < K / 2; ++k) {
                if (k < width) {
                  const float send = upper ? part[k] : part[k + width];
                  const float keep = upper ? part[k + width] : part[k];
                  part[k] = keep + __shfl_xor_sync(0xffffffffu, send, half);
                }
              }
            } else {
              part[0] += __shfl_xor_sync(0xffffffffu, part[0], half);
            }
          }
        }
        if (live) {
          int kbase = 0;
#pragma unroll
          for (int t = 0; t < 5; ++t)
            if ((1 << t) < G && (K >> (t + 1)) >= 1 && (gl & (1 << t))) kbase += K >> (t + 1);
          const int cnt = G <= K ? K / G : 1;
          const bool owner = G <= K || gl < K;
          if (owner) {
            float* dst = dbasis + (int64_t)m * K + kbase;
#pragma unroll
            for (int q = 0; q < K; ++q) {
              if (q < cnt) {
                if (single_pass) dst[q] = part[q]; else atomicAdd(dst + q, part[q]);
              }
            }
          }
        }
      }
    }
  }
}

template <int K, int OUT>
static int launch_basis_proj(cudaStream_t st, int C, int64_t ns, const float* basis,
                             const float* feat, const int2* neigh, const int32_t* ranges,
                             float* out, __nv_bfloat16* hi, __nv_bfloat16* mid) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  const int G = bp_group_lanes(C, kCpl);
  const bool vec = kCpl == 4 && C % 4 == 0 && ((uintptr_t)feat % 16 == 0);
  const size_t smem = G == 32 ? (size_t)(kBpThreads / 32) * 32 * BpCfg<K>::kRow * sizeof(float) : 0;
  const int64_t samples_per_block = (int64_t)(kBpThreads / 32) * (32 / G);
  unsigned grid = min(blocks_for(ns, (int)samples_per_block), (unsigned)(sm_count() * 64));
  ProfScope prof(st, OUT == 0 ? "basis_proj" : "basis_proj_split");
  if (G == 32 && C % kCpl == 0 && ((uintptr_t)feat % 16 == 0) && (C * 4) % (kCpl * 4) == 0) {
    auto kern = basis_proj_wide_kernel<K, OUT>;
    const size_t wsmem = (size_t)(kBpwThreads / 32) * bpw_warp_floats<K>() * sizeof(float);
    TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem));
    TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    cudaSharedmemCarveoutMaxShared));
    // exactly one resident wave: all warps then sweep the samples in lock step
    // and the feature rows they gather stay within a few clouds, i.e. in L2
    int per_sm = 1;
    TFGPC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kBpwThreads, wsmem));
    unsigned wgrid = min(blocks_for(ns, kBpwThreads / 32), (unsigned)(sm_count() * max(per_sm, 1)));
    kern<<<wgrid, kBpwThreads, wsmem, st>>>(C, ns, basis, feat, neigh, ranges, out, hi, mid);
    TFGPC_LAUNCH_CHECK();
    return TFGPC_OK;
  }
  if (vec) {
    auto kern = basis_proj_kernel<K, true, OUT>;
    if (smem > 48 * 1024)
      TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kBpThreads, smem, st>>>(C, ns, G, basis, feat, neigh, ranges, out, hi, mid);
  } else {
    auto kern = basis_proj_kernel<K, false, OUT>;
    if (smem > 48 * 1024)
      TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kBpThreads, smem, st>>>(C, ns, G, basis, feat, neigh, ranges, out, hi, mid);
  }
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

// Entry used by the fused MCConv path (mcconv.cu): split bf16 output.
int basis_proj_split(cudaStream_t st, int K, int C, int64_t ns, const float* basis,
                     const float* feat, const int32_t* neigh, const int32_t* ranges,
                     __nv_bfloat16* hi, __nv_bfloat16* mid) {
  switch (K) {
    case 8: return launch_basis_proj<8, 1>(st, C, ns, basis, feat, (const int2*)neigh, ranges, nullptr, hi, mid);
    case 16: return launch_basis_proj<16, 1>(st, C, ns, basis, feat, (const int2*)neigh, ranges, nullptr, hi, mid);
    case 32: return launch_basis_proj<32, 1>(st, C, ns, basis, feat, (const int2*)neigh, ranges, nullptr, hi, mid);
    case 64: return launch_basis_proj<64, 1>(st, C, ns, basis, feat, (const int2*)neigh, ranges, nullptr, hi, mid);
  }
  return fail(TFGPC_EINVAL, "BasisProj expects a valid number of basis functions.");
}

template <int K>
static int launch_basis_proj_grads(cudaStream_t st, int C, int64_t ns, const float* basis,
                                   const float* feat, const int2* neigh, const int32_t* ranges,
                                   const float* in_grads, float* dbasis, float* dfeat) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  const int G = bp_group_lanes(C, kCpl);
  const bool vec = kCpl == 4 && C % 4 == 0 && ((uintptr_t)feat % 16 == 0) &&
                   ((uintptr_t)dfeat % 16 == 0);
  const int64_t samples_per_block = (int64_t)(kBpThreads / 32) * (32 / G);
  unsigned grid = min(blocks_for(ns, (int)samples_per_block), (unsigned)(sm_count() * 64));
  ProfScope prof(st, "basis_proj_grads");
  if (G == 32 && C % kCpl == 0 && ((uintptr_t)feat % 16 == 0) && ((uintptr_t)dfeat % 16 == 0) &&
      ((uintptr_t)dbasis % 16 == 0)) {
    auto kern = basis_proj_grads_wide_kernel<K>;
    const size_t wsmem = (size_t)(kBpwThreads / 32) * bpw_grads_warp_floats<K>() * sizeof(float);
    TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem));
    TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    cudaSharedmemCarveoutMaxShared));
    int per_sm = 1;
    TFGPC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kBpwThreads, wsmem));
    unsigned wgrid = min(blocks_for(ns, kBpwThreads / 32), (unsigned)(sm_count() * max(per_sm, 1)));
    kern<<<wgrid, kBpwThreads, wsmem, st>>>(C, ns, basis, feat, neigh, ranges, in_grads, dbasis,
                                            dfeat);
    TFGPC_LAUNCH_CHECK();
    return TFGPC_OK;
  }
  if (vec)
    basis_proj_grads_kernel<K, true><<<grid, kBpThreads, 0, st>>>(C, ns, G, basis, feat, neigh,
                                                                  ranges, in_grads, dbasis, dfeat);
  else
    basis_proj_grads_kernel<K, false><<<grid, kBpThreads, 0, st>>>(C, ns, G, basis, feat, neigh,
                                                                   ranges, in_grads, dbasis, dfeat);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

// basis_proj_mma.cu: the same contractions on warp-level tensor-core MMAs, over a
// bf16 hi/mid copy of the features kept in caller scratch
bool basis_proj_mma_supported(int K, int C);
int split_features(cudaStream_t st, const float* feat, int64_t n, int C, __nv_bfloat16* fs);
int basis_proj_mma_f32(cudaStream_t st, int K, int C, int64_t ns, const float* basis,
                       const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                       float* out);
int basis_proj_grads_mma(cudaStream_t st, int K, int C, int64_t ns, int64_t M, const float* basis,
                         const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                         const float* in_grads, float* dbasis, float* dfeat);

static int check_bp_args(const char* op, int K, int C, int64_t ns, int64_t n_in, int64_t M) {
  TFGPC_REQUIRE(valid_basis(K), "%s expects a valid number of basis functions.", op);
  TFGPC_REQUIRE(valid_features(C), "%s expects a valid number of input features, between 1 and 8 "
                "or multiple of 8", op);
  TFGPC_REQUIRE(ns >= 0 && ns < (int64_t)INT32_MAX && n_in >= 0 && n_in < (int64_t)INT32_MAX &&
                M >= 0 && M <= (int64_t)INT32_MAX, "%s expects 0 <= ns, n_in, M < 2^31", op);
  return TFGPC_OK;
}

}  // namespace tfgpc

using namespace tfgpc;

extern "C" int tfgpc_basis_proj(void* stream, int K, int C, int64_t ns, int64_t n_in, int64_t M,
                                const float* basis, const float* features,
                                const int32_t* neighbors, const int32_t* ranges, float* out) {
  int rc = check_bp_args("BasisProjOp", K, C, ns, n_in, M);
  if (rc) return rc;
  if (ns == 0) return TFGPC_OK;
  TFGPC_REQUIRE(ranges && out && (M == 0 || (basis && features && neighbors)),
                "BasisProjOp got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis % 16 == 0 && (uintptr_t)out % 16 == 0,
                "BasisProjOp expects 16-byte aligned basis and output buffers");
  cudaStream_t st = (cudaStream_t)stream;
  const int2* nb = (const int2*)neighbors;
  switch (K) {
    case 8: return launch_basis_proj<8, 0>(st, C, ns, basis, features, nb, ranges, out, nullptr, nullptr);
    case 16: return launch_basis_proj<16, 0>(st, C, ns, basis, features, nb, ranges, out, nullptr, nullptr);
    case 32: return launch_basis_proj<32, 0>(st, C, ns, basis, features, nb, ranges, out, nullptr, nullptr);
    default: return launch_basis_proj<64, 0>(st, C, ns, basis, features, nb, ranges, out, nullptr, nullptr);
  }
}

extern "C" int tfgpc_basis_proj_grads(void* stream, int K, int C, int64_t ns, int64_t n_in,
                                      int64_t M, const float* basis, const float* features,
                                      const int32_t* neighbors, const int32_t* ranges,
                                      const float* in_grads, float* dbasis_out, float* dfeat_out) {
  int rc = check_bp_args("BasisProjGradsOp", K, C, ns, n_in, M);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (M > 0) {
    TFGPC_REQUIRE(dbasis_out, "BasisProjGradsOp got a null pointer");
    TFGPC_CUDA(cudaMemsetAsync(dbasis_out, 0, sizeof(float) * (size_t)M * K, st));
  }
  if (n_in > 0) {
    TFGPC_REQUIRE(dfeat_out, "BasisProjGradsOp got a null pointer");
    TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
  }
  if (ns == 0 || M == 0) return TFGPC_OK;
  TFGPC_REQUIRE(basis && features && neighbors && ranges && in_grads,
                "BasisProjGradsOp got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis % 16 == 0 && (uintptr_t)in_grads % 16 == 0,
                "BasisProjGradsOp expects 16-byte aligned basis and gradient buffers");
  const int2* nb = (const int2*)neighbors;
  switch (K) {
    case 8: return launch_basis_proj_grads<8>(st, C, ns, basis, features, nb, ranges, in_grads, dbasis_out, dfeat_out);
    case 16: return launch_basis_proj_grads<16>(st, C, ns, basis, features, nb, ranges, in_grads, dbasis_out, dfeat_out);
    case 32: return launch_basis_proj_grads<32>(st, C, ns, basis, features, nb, ranges, in_grads, dbasis_out, dfeat_out);
    default: return launch_basis_proj_grads<64>(st, C, ns, basis, features, nb, ranges, in_grads, dbasis_out, dfeat_out);
  }
}

extern "C" size_t tfgpc_basis_proj_workspace_bytes(int K, int C, int64_t n_in) {
  if (n_in <= 0 || !basis_proj_mma_supported(K, C)) return 0;
  return (size_t)n_in * C * 4 + 256;
}

// True if `ws` can hold the split features of this call and everything is
// aligned for the tensor-core kernels.
static bool mma_path(int K, int C, int64_t n_in, const void* ws, size_t ws_bytes, const void* a,
                     const void* b, const void* c) {
  const size_t need = tfgpc_basis_proj_workspace_bytes(K, C, n_in);
  return need > 0 && ws && ws_bytes >= need && (uintptr_t)ws % 16 == 0 && (uintptr_t)a % 16 == 0 &&
         (uintptr_t)b % 16 == 0 && (uintptr_t)c % 16 == 0;
}

extern "C" int tfgpc_basis_proj_ws(void* stream, int K, int C, int64_t ns, int64_t n_in, int64_t M,
                                   const float* basis, const float* features,
                                   const int32_t* neighbors, const int32_t* ranges, float* out,
                                   void* ws, size_t ws_bytes) {
  if (ns == 0 || M == 0 || !mma_path(K, C, n_in, ws, ws_bytes, features, basis, out))
    return tfgpc_basis_proj(stream, K, C, ns, n_in, M, basis, features, neighbors, ranges, out);
  int rc = check_bp_args("BasisProjOp", K, C, ns, n_in, M);
  if (rc) return rc;
  TFGPC_REQUIRE(ranges && out && basis && features && neighbors, "BasisProjOp got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  __nv_bfloat16* fs = (__nv_bfloat16*)ws;
  rc = split_features(st, features, n_in, C, fs);
  if (rc) return rc;
  return basis_proj_mma_f32(st, K, C, ns, basis, fs, neighbors, ranges, out);
}

extern "C" int tfgpc_basis_proj_grads_ws(void* stream, int K, int C, int64_t ns, int64_t n_in,
                                         int64_t M, const float* basis, const float* features,
                                         const int32_t* neighbors, const int32_t* ranges,
                                         const float* in_grads, float* dbasis_out,
                                         float* dfeat_out, void* ws, size_t ws_bytes) {
  if (ns == 0 || M == 0 || !mma_path(K, C, n_in, ws, ws_bytes, features, dbasis_out, dfeat_out) ||
      (uintptr_t)basis % 16 != 0 || (uintptr_t)in_grads % 16 != 0)
    return tfgpc_basis_proj_grads(stream, K, C, ns, n_in, M, basis, features, neighbors, ranges,
                                  in_grads, dbasis_out, dfeat_out);
  int rc = check_bp_args("BasisProjGradsOp", K, C, ns, n_in, M);
  if (rc) return rc;
  TFGPC_REQUIRE(basis && features && neighbors && ranges && in_grads && dbasis_out && dfeat_out,
                "BasisProjGradsOp got a null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  __nv_bfloat16* fs = (__nv_bfloat16*)ws;
  rc = split_features(st, features, n_in, C, fs);
  if (rc) return rc;
  TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
  return basis_proj_grads_mma(st, K, C, ns, M, basis, fs, neighbors, ranges, in_grads, dbasis_out,
                              dfeat_out);
}
