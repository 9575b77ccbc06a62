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

// ---- small PTX helpers ---------------------------------------------------------

// Two fp32 FMAs per instruction (sm_100 packed fp32): d = a * b + c on both
// halves of 64-bit register pairs.  Halves the issue slots of the FMA-bound
// inner loops below.
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b,
                                                    unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}

__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// Asynchronous global -> shared copy of one lane's slice of a feature row.
template <int BYTES>
__device__ __forceinline__ void cp_async_row(float* dst_smem, const float* src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(dst_smem);
  if (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(src), "n"(BYTES)
                 : "memory");
}

__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kBpwRing = 8;  // feature rows in flight per warp

// Floats of shared memory one warp needs: the output staging tile, or the ring
// of in-flight feature rows plus the staged basis rows, whichever is larger.
template <int K>
__host__ __device__ constexpr int bpw_warp_floats() {
  return (32 * BpCfg<K>::kRow > kBpwRing * 32 * BpCfg<K>::kCpl + 32 * K)
             ? 32 * BpCfg<K>::kRow
             : kBpwRing * 32 * BpCfg<K>::kCpl + 32 * K;
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
  constexpr int R = kBpwRing;
  typedef typename FeatVec<kCpl>::type fvec;
  extern __shared__ __align__(16) float smem_all[];
  const int lane = lane_id();
  float* tile = smem_all + (size_t)(threadIdx.x >> 5) * bpw_warp_floats<K>();
  float* ring = tile;                           // [R][32 lanes][CPL]
  float* wtile = tile + R * 32 * kCpl;          // [32 neighbors][K]
  const int64_t warps = ((int64_t)gridDim.x * kBpwThreads) >> 5;
  for (int64_t s = ((int64_t)blockIdx.x * kBpwThreads + threadIdx.x) >> 5; s < ns; s += warps) {
    const int a = s ? __ldg(ranges + s - 1) : 0;
    const int e = __ldg(ranges + s);
    for (int c0 = 0; c0 < C; c0 += kChunk) {
      const int cbase = c0 + lane * kCpl;
      const bool c_ok = cbase < C;  // C is a multiple of CPL on this path
      unsigned long long acc[kCpl][K / 2];
#pragma unroll
      for (int cc = 0; cc < kCpl; ++cc)
#pragma unroll
        for (int k = 0; k < K / 2; ++k) acc[cc][k] = 0ull;
      for (int base = a; base < e; base += 32) {
        const int cnt = min(32, e - base);
        __syncwarp();
        const int my_j = lane < cnt ? __ldg(&neigh[base + lane].x) : 0;
        stage_basis_chunk<K>(wtile, basis, base, cnt, lane);
        // fill the ring: rows 0 .. R-1 of the chunk (one commit group per row)
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int j = __shfl_sync(0xffffffffu, my_j, r);
          if (r < cnt && c_ok)
            cp_async_row<kCpl * 4>(ring + (r * 32 + lane) * kCpl, feat + (int64_t)j * C + cbase);
          cp_async_commit();
        }
        __syncwarp();
        for (int it = 0; it < cnt; ++it) {
          cp_async_wait<R - 1>();  // row `it` has landed (each lane reads only what it copied)
          float f[kCpl];
          if (c_ok) {
            FeatVec<kCpl>::unpack(*reinterpret_cast<const fvec*>(ring + ((it & (R - 1)) * 32 + lane) * kCpl), f);
          } else {
#pragma unroll
            for (int cc = 0; cc < kCpl; ++cc) f[cc] = 0.0f;
          }
          unsigned long long ff[kCpl];
#pragma unroll
          for (int cc = 0; cc < kCpl; ++cc) ff[cc] = pack2(f[cc], f[cc]);
          const ulonglong2* wrow = reinterpret_cast<const ulonglong2*>(wtile + it * K);
#pragma unroll
          for (int q = 0; q < K / 4; ++q) {
            const ulonglong2 w = wrow[q];
#pragma unroll
            for (int cc = 0; cc < kCpl; ++cc) {
              acc[cc][2 * q] = ffma2(ff[cc], w.x, acc[cc][2 * q]);
              acc[cc][2 * q + 1] = ffma2(ff[cc], w.y, acc[cc][2 * q + 1]);
            }
          }
          // refill the slot just consumed with row it + R
          const int nxt = it + R;
          const int jn = __shfl_sync(0xffffffffu, my_j, nxt & 31);
          if (nxt < cnt && c_ok)
            cp_async_row<kCpl * 4>(ring + ((it & (R - 1)) * 32 + lane) * kCpl,
                                   feat + (int64_t)jn * C + cbase);
          cp_async_commit();
        }
        cp_async_wait<0>();
      }
      // stage the warp's 32 x (CPL*K) results, then store 512 contiguous bytes
      // per warp instruction
      __syncwarp();
#pragma unroll
      for (int q = 0; q < kAcc / 4; ++q) {
        float4 v;
        unpack2(acc[(4 * q) / K][((4 * q) % K) / 2], v.x, v.y);
        unpack2(acc[(4 * q) / K][((4 * q) % K) / 2 + 1], v.z, v.w);
        *reinterpret_cast<float4*>(tile + lane * kRow + 4 * q) = v;
      }
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
__host__ __device__ constexpr int bpw_grads_warp_floats() {
  return kBpwRing * 32 * BpCfg<K>::kCpl + 2 * 32 * K;
}

template <int K>
__global__ void __launch_bounds__(kBpwThreads, 2)
basis_proj_grads_wide_kernel(int C, int64_t ns, const float* __restrict__ basis,
                             const float* __restrict__ feat, const int2* __restrict__ neigh,
                             const int32_t* __restrict__ ranges,
                             const float* __restrict__ in_grads, float* __restrict__ dbasis,
                             float* __restrict__ dfeat) {
  constexpr int kCpl = BpCfg<K>::kCpl;
  constexpr int kChunk = 32 * kCpl;
  constexpr int R = kBpwRing;
  typedef typename FeatVec<kCpl>::type fvec;
  extern __shared__ __align__(16) float smem_all[];
  const int lane = lane_id();
  float* ring = smem_all + (size_t)(threadIdx.x >> 5) * bpw_grads_warp_floats<K>();  // [R][32][CPL]
  float* wtile = ring + R * 32 * kCpl;   // staged basis rows [32][K]
  float* dtile = wtile + 32 * K;         // dbasis of the chunk [32][K]
  const int64_t warps = ((int64_t)gridDim.x * kBpwThreads) >> 5;
  // which basis function this lane holds after the butterfly (see below)
  int kbase = 0;
#pragma unroll
  for (int t = 0; t < 5; ++t)
    if ((K >> (t + 1)) >= 1 && (lane & (1 << t))) kbase += K >> (t + 1);
  const int own_cnt = K >= 32 ? K / 32 : 1;
  const bool owner = K >= 32 || lane < K;
  // The first butterfly steps (those that still move whole groups of 4 values)
  // need no selects if every lane keeps its gradient tile and basis row in a
  // lane-dependent order: register r holds basis function r ^ perm, where perm
  // flips, for every such step, the half the lane has to give away.  Partners
  // then always exchange registers [width, 2*width) and keep [0, width).
  constexpr int kFreeSteps = (K == 8) ? 1 : (K == 16) ? 2 : (K == 32) ? 3 : 4;
  int perm = 0;
#pragma unroll
  for (int t = 0; t < kFreeSteps; ++t)
    if (lane & (1 << t)) perm += K >> (t + 1);
  const int permq = perm >> 2;  // in units of 4 values (one 128-bit load)
  for (int64_t s = ((int64_t)blockIdx.x * kBpwThreads + threadIdx.x) >> 5; s < ns; s += warps) {
    const int a = s ? __ldg(ranges + s - 1) : 0;
    const int e = __ldg(ranges + s);
    for (int base = a; base < e; base += 32) {
      const int cnt = min(32, e - base);
      __syncwarp();
      const int my_j = lane < cnt ? __ldg(&neigh[base + lane].x) : 0;
      stage_basis_chunk<K>(wtile, basis, base, cnt, lane);
      for (int i = lane; i < 32 * K; i += 32) dtile[i] = 0.0f;
      for (int c0 = 0; c0 < C; c0 += kChunk) {
        const int cbase = c0 + lane * kCpl;
        const bool c_ok = cbase < C;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int j = __shfl_sync(0xffffffffu, my_j, r);
          if (r < cnt && c_ok)
            cp_async_row<kCpl * 4>(ring + (r * 32 + lane) * kCpl, feat + (int64_t)j * C + cbase);
          cp_async_commit();
        }
        // this lane's CPL x K tile of the incoming gradient, as packed pairs over k
        unsigned long long g[kCpl][K / 2];
#pragma unroll
        for (int cc = 0; cc < kCpl; ++cc) {
          const ulonglong2* src = reinterpret_cast<const ulonglong2*>(
              in_grads + s * (int64_t)C * K + (int64_t)(cbase + cc) * K);
#pragma unroll
          for (int q = 0; q < K / 4; ++q) {
            const ulonglong2 v = c_ok ? __ldg(src + (q ^ permq)) : make_ulonglong2(0ull, 0ull);
            g[cc][2 * q] = v.x; g[cc][2 * q + 1] = v.y;
          }
        }
        __syncwarp();
        for (int it = 0; it < cnt; ++it) {
          cp_async_wait<R - 1>();
          float f[kCpl];
          if (c_ok) {
            FeatVec<kCpl>::unpack(*reinterpret_cast<const fvec*>(ring + ((it & (R - 1)) * 32 + lane) * kCpl), f);
          } else {
#pragma unroll
            for (int cc = 0; cc < kCpl; ++cc) f[cc] = 0.0f;
          }
          const int j = __shfl_sync(0xffffffffu, my_j, it);
          unsigned long long w[K / 2];
          const ulonglong2* wrow = reinterpret_cast<const ulonglong2*>(wtile + it * K);
#pragma unroll
          for (int q = 0; q < K / 4; ++q) {
            const ulonglong2 v = wrow[q ^ permq];
            w[2 * q] = v.x; w[2 * q + 1] = v.y;
          }
          // dfeat[nbr, c] += sum_k g[c,k] * basis[m,k]
          float df[kCpl];
#pragma unroll
          for (int cc = 0; cc < kCpl; ++cc) {
            unsigned long long acc2 = 0ull;
#pragma unroll
            for (int kp = 0; kp < K / 2; ++kp) acc2 = ffma2(g[cc][kp], w[kp], acc2);
            float lo, hi;
            unpack2(acc2, lo, hi);
            df[cc] = lo + hi;
          }
          if (c_ok) {
            float* dst = dfeat + (int64_t)j * C + cbase;
            if (kCpl == 4) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(df[0]),
                           "f"(df[1 % kCpl]), "f"(df[2 % kCpl]), "f"(df[3 % kCpl]) : "memory");
            } else if (kCpl == 2) {
              asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(dst), "f"(df[0]),
                           "f"(df[1 % kCpl]) : "memory");
            } else {
              atomicAdd(dst, df[0]);
            }
          }
          // dbasis[m, k]: partial sums over this lane's channels ...
          float part[K];
#pragma unroll
          for (int kp = 0; kp < K / 2; ++kp) {
            unsigned long long acc2 = 0ull;
#pragma unroll
            for (int cc = 0; cc < kCpl; ++cc) acc2 = ffma2(g[cc][kp], pack2(f[cc], f[cc]), acc2);
            unpack2(acc2, part[2 * kp], part[2 * kp + 1]);
          }
          // ... folded over the 32 lanes by a halving butterfly over xor distances
          // 1, 2, 4, ...: the select-free steps first (see perm above), then the
          // last steps, where lanes with the distance bit set keep the upper half
#pragma unroll
          for (int t = 0; t < 5; ++t) {
            const int half = 1 << t;
            const int width = K >> (t + 1);
            if (t < kFreeSteps) {
#pragma unroll
              for (int k = 0; k < K / 2; ++k)
                if (k < width) part[k] += __shfl_xor_sync(0xffffffffu, part[k + width], half);
            } else if (width >= 1) {
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
              if (q < own_cnt) dtile[it * K + kbase + q] += part[q];
          }
          // refill the ring slot just consumed
          const int nxt = it + R;
          const int jn = __shfl_sync(0xffffffffu, my_j, nxt & 31);
          if (nxt < cnt && c_ok)
            cp_async_row<kCpl * 4>(ring + ((it & (R - 1)) * 32 + lane) * kCpl,
                                   feat + (int64_t)jn * C + cbase);
          cp_async_commit();
        }
        cp_async_wait<0>();
      }
      __syncwarp();
      float4* dst = reinterpret_cast<float4*>(dbasis + (int64_t)base * K);
      const float4* srcd = reinterpret_cast<const float4*>(dtile);
      for (int i = lane; i < cnt * (K / 4); i += 32) dst[i] = srcd[i];
    }
  }
}

}  // namespace tfgpc
