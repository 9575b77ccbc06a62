// Wide-layer variants of the basis projection kernels (C_in covers a full
// warp: 32 lanes x CPL channels per pass).  One warp owns one sample and
// walks its neighbor list in chunks of 32:
//   - the 32 neighbor indices are loaded with one coalesced read and handed
//     out by shuffle, so no index load sits on the critical path;
//   - the chunk's basis rows (32 x K floats, contiguous in memory) are staged
//     in the warp's shared-memory tile and read back as broadcast 128-bit
//     loads;
//   - the feature rows, the only scattered traffic, are fetched U at a time
//     before any of them is used, which keeps U independent 512-byte row reads
//     in flight per warp.
#pragma once

#include "basis_proj.cuh"

namespace tfgpc {

constexpr int kBpwThreads = 256;
constexpr int kBpwUnroll = 4;

template <int CPL>
struct FeatVec;
template <>
struct FeatVec<4> {
  typedef float4 type;
  static __device__ __forceinline__ void unpack(const float4& v, float* f) {
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
};
template <>
struct FeatVec<2> {
  typedef float2 type;
  static __device__ __forceinline__ void unpack(const float2& v, float* f) { f[0] = v.x; f[1] = v.y; }
};
template <>
struct FeatVec<1> {
  typedef float type;
  static __device__ __forceinline__ void unpack(const float& v, float* f) { f[0] = v; }
};

// Per-warp shared-memory tile: 32 rows of kRow floats.  During the neighbor
// loop its first 32*K floats hold the staged basis rows; afterwards the whole
// tile stages the warp's output for coalesced stores.
template <int K>
__device__ __forceinline__ void stage_basis_chunk(float* tile, const float* __restrict__ basis,
                                                  int base, int cnt, int lane) {
  const float4* src = reinterpret_cast<const float4*>(basis + (int64_t)base * K);
  float4* dst = reinterpret_cast<float4*>(tile);
  for (int i = lane; i < cnt * (K / 4); i += 32) dst[i] = __ldg(src + i);
}

template <int K, int OUT>
__global__ void __launch_bounds__(kBpwThreads, 2)
basis_proj_wide_kernel(int C, int64_t ns, const float* __restrict__ basis,
                       const float* __restrict__ feat, const int2* __restrict__ neigh,
                       const int32_t* __restrict__ ranges, float* __restrict__ out,
                       __nv_bfloat16* __restrict__ out_hi, __nv_bfloat16* __restrict__ out_mid) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  constexpr int kAcc = BpCfg<K>::kAcc;
  constexpr int kRow = BpCfg<K>::kRow;
  constexpr int kChunk = 32 * kCpl;
  typedef typename FeatVec<kCpl>::type fvec;
  extern __shared__ __align__(16) float smem_all[];
  const int lane = lane_id();
  float* tile = smem_all + (size_t)(threadIdx.x >> 5) * 32 * kRow;
  const int64_t warps = ((int64_t)gridDim.x * kBpwThreads) >> 5;
  for (int64_t s = ((int64_t)blockIdx.x * kBpwThreads + threadIdx.x) >> 5; s < ns; s += warps) {
    const int a = s ? __ldg(ranges + s - 1) : 0;
    const int e = __ldg(ranges + s);
    for (int c0 = 0; c0 < C; c0 += kChunk) {
      const int cbase = c0 + lane * kCpl;
      const bool c_ok = cbase < C;  // C is a multiple of CPL on this path
      float acc[kCpl][K];
#pragma unroll
      for (int cc = 0; cc < kCpl; ++cc)
#pragma unroll
        for (int k = 0; k < K; ++k) acc[cc][k] = 0.0f;
      for (int base = a; base < e; base += 32) {
        const int cnt = min(32, e - base);
        __syncwarp();
        const int my_j = lane < cnt ? __ldg(&neigh[base + lane].x) : 0;
        stage_basis_chunk<K>(tile, basis, base, cnt, lane);
        __syncwarp();
        // Feature rows are fetched one group of U ahead of their use.
        fvec cur[kBpwUnroll], nxt[kBpwUnroll];
        auto fetch = [&](fvec* dst, int it) {
#pragma unroll
          for (int u = 0; u < kBpwUnroll; ++u) {
            const int j = __shfl_sync(0xffffffffu, my_j, (it + u) & 31);
            if (it + u < cnt && c_ok)
              dst[u] = __ldg(reinterpret_cast<const fvec*>(feat + (int64_t)j * C + cbase));
          }
        };
        auto consume = [&](const fvec* src, int it) {
#pragma unroll
          for (int u = 0; u < kBpwUnroll; ++u) {
            if (it + u < cnt) {
              float f[kCpl];
              if (c_ok) FeatVec<kCpl>::unpack(src[u], f);
              else {
#pragma unroll
                for (int cc = 0; cc < kCpl; ++cc) f[cc] = 0.0f;
              }
              const float4* wrow = reinterpret_cast<const float4*>(tile + (it + u) * K);
#pragma unroll
              for (int q = 0; q < K / 4; ++q) {
                const float4 w = wrow[q];
#pragma unroll
                for (int cc = 0; cc < kCpl; ++cc) {
                  acc[cc][4 * q] = fmaf(f[cc], w.x, acc[cc][4 * q]);
                  acc[cc][4 * q + 1] = fmaf(f[cc], w.y, acc[cc][4 * q + 1]);
                  acc[cc][4 * q + 2] = fmaf(f[cc], w.z, acc[cc][4 * q + 2]);
                  acc[cc][4 * q + 3] = fmaf(f[cc], w.w, acc[cc][4 * q + 3]);
                }
              }
            }
          }
        };
        fetch(cur, 0);
        for (int it = 0; it < cnt; it += 2 * kBpwUnroll) {
          fetch(nxt, it + kBpwUnroll);
          consume(cur, it);
          fetch(cur, it + 2 * kBpwUnroll);
          consume(nxt, it + kBpwUnroll);
        }
      }
      // stage the warp's 32 x (CPL*K) results, then store 512 contiguous bytes
      // per warp instruction
      __syncwarp();
#pragma unroll
      for (int q = 0; q < kAcc / 4; ++q)
        *reinterpret_cast<float4*>(tile + lane * kRow + 4 * q) =
            make_float4(acc[(4 * q) / K][(4 * q) % K], acc[(4 * q + 1) / K][(4 * q + 1) % K],
                        acc[(4 * q + 2) / K][(4 * q + 2) % K], acc[(4 * q + 3) / K][(4 * q + 3) % K]);
      __syncwarp();
      const int valid = min(kChunk, C - c0) * K;
      const int64_t obase = s * (int64_t)C * K + (int64_t)c0 * K;
#pragma unroll 4
      for (int f0 = lane * 4; f0 < valid; f0 += 128) {
        const float4 v = *reinterpret_cast<const float4*>(tile + (f0 / kAcc) * kRow + (f0 % kAcc));
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
  }
}

// Gradients, same walk.  Per neighbor: dfeat[nbr, c] += sum_k g[c,k]*basis[m,k]
// (one 128-bit reduction per lane) and dbasis[m,k] = sum_c g[c,k]*feat[nbr,c],
// folded across the 32 lanes by a halving butterfly into the warp's
// shared-memory tile [32 neighbors x K], which is written out with contiguous
// stores once per chunk -- no atomics on dbasis.
template <int K>
__global__ void __launch_bounds__(kBpwThreads, 2)
basis_proj_grads_wide_kernel(int C, int64_t ns, const float* __restrict__ basis,
                             const float* __restrict__ feat, const int2* __restrict__ neigh,
                             const int32_t* __restrict__ ranges,
                             const float* __restrict__ in_grads, float* __restrict__ dbasis,
                             float* __restrict__ dfeat) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  constexpr int kChunk = 32 * kCpl;
  constexpr int kU = 4;
  typedef typename FeatVec<kCpl>::type fvec;
  extern __shared__ __align__(16) float smem_all[];
  const int lane = lane_id();
  float* wtile = smem_all + (size_t)(threadIdx.x >> 5) * 2 * 32 * K;  // staged basis rows
  float* dtile = wtile + 32 * K;                                      // dbasis of the chunk
  const int64_t warps = ((int64_t)gridDim.x * kBpwThreads) >> 5;
  // which basis function this lane holds after the butterfly (see below)
  int kbase = 0;
#pragma unroll
  for (int t = 0; t < 5; ++t)
    if ((K >> (t + 1)) >= 1 && (lane & (1 << t))) kbase += K >> (t + 1);
  const int own_cnt = K >= 32 ? K / 32 : 1;
  const bool owner = K >= 32 || lane < K;
  for (int64_t s = ((int64_t)blockIdx.x * kBpwThreads + threadIdx.x) >> 5; s < ns; s += warps) {
    const int a = s ? __ldg(ranges + s - 1) : 0;
    const int e = __ldg(ranges + s);
    for (int base = a; base < e; base += 32) {
      const int cnt = min(32, e - base);
      __syncwarp();
      const int my_j = lane < cnt ? __ldg(&neigh[base + lane].x) : 0;
      stage_basis_chunk<K>(wtile, basis, base, cnt, lane);
      for (int i = lane; i < 32 * K; i += 32) dtile[i] = 0.0f;
      __syncwarp();
      for (int c0 = 0; c0 < C; c0 += kChunk) {
        const int cbase = c0 + lane * kCpl;
        const bool c_ok = cbase < C;
        float g[kCpl][K];
#pragma unroll
        for (int cc = 0; cc < kCpl; ++cc) {
          const float4* src = reinterpret_cast<const float4*>(
              in_grads + s * (int64_t)C * K + (int64_t)(cbase + cc) * K);
#pragma unroll
          for (int q = 0; q < K / 4; ++q) {
            const float4 v = c_ok ? __ldg(src + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            g[cc][4 * q] = v.x; g[cc][4 * q + 1] = v.y; g[cc][4 * q + 2] = v.z; g[cc][4 * q + 3] = v.w;
          }
        }
        for (int it = 0; it < cnt; it += kU) {
          fvec fv[kU];
          int js[kU];
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            js[u] = __shfl_sync(0xffffffffu, my_j, (it + u) & 31);
            if (it + u < cnt && c_ok)
              fv[u] = __ldg(reinterpret_cast<const fvec*>(feat + (int64_t)js[u] * C + cbase));
          }
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            if (it + u < cnt) {  // warp-uniform
              float f[kCpl], w[K], part[K];
              if (c_ok) FeatVec<kCpl>::unpack(fv[u], f);
              else {
#pragma unroll
                for (int cc = 0; cc < kCpl; ++cc) f[cc] = 0.0f;
              }
              const float4* wrow = reinterpret_cast<const float4*>(wtile + (it + u) * K);
#pragma unroll
              for (int q = 0; q < K / 4; ++q) {
                const float4 v = wrow[q];
                w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
              }
              float df[kCpl];
#pragma unroll
              for (int cc = 0; cc < kCpl; ++cc) {
                float accv = 0.0f;
#pragma unroll
                for (int k = 0; k < K; ++k) accv = fmaf(g[cc][k], w[k], accv);
                df[cc] = accv;
              }
              if (c_ok) {
                float* dst = dfeat + (int64_t)js[u] * C + cbase;
                if (kCpl == 4) {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                               "f"(df[0]), "f"(df[1]), "f"(df[2]), "f"(df[3]) : "memory");
                } else if (kCpl == 2) {
                  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(dst), "f"(df[0]),
                               "f"(df[1 % kCpl]) : "memory");
                } else {
                  atomicAdd(dst, df[0]);
                }
              }
#pragma unroll
              for (int k = 0; k < K; ++k) {
                float accv = 0.0f;
#pragma unroll
                for (int cc = 0; cc < kCpl; ++cc) accv = fmaf(g[cc][k], f[cc], accv);
                part[k] = accv;
              }
              // halving butterfly over xor distances 1, 2, 4, ...: lanes with
              // the distance bit set keep the upper half of their values
#pragma unroll
              for (int t = 0; t < 5; ++t) {
                const int half = 1 << t;
                const int width = K >> (t + 1);
                if (width >= 1) {
                  const bool upper = (lane & half) != 0;
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
              if (owner) {
#pragma unroll
                for (int q = 0; q < K; ++q)
                  if (q < own_cnt) dtile[(it + u) * K + kbase + q] += part[q];
              }
            }
          }
        }
      }
      __syncwarp();
      float4* dst = reinterpret_cast<float4*>(dbasis + (int64_t)base * K);
      const float4* srcd = reinterpret_cast<const float4*>(dtile);
      for (int i = lane; i < cnt * (K / 4); i += 32) dst[i] = srcd[i];
    }
  }
}

}  // namespace tfgpc
