// Basis projection and its gradients on warp-level tensor-core MMAs.
//
// Per sample the projection is a small ragged matrix product,
//   X[c, k] = sum_m feat[nbr(m), c] * basis[m, k],      m over the sample's pairs,
// and so are its two gradients,
//   dbasis[m, k]    = sum_c feat[nbr(m), c] * dX[c, k],
//   dfeat[nbr(m), c] += sum_k basis[m, k] * dX[c, k].
// A CTA-wide tcgen05 tile (128 rows) does not fit products with ~32 pairs per
// sample, so these kernels keep the one-warp-per-sample walk of the SIMT
// kernels and issue mma.sync.m16n8k16 on 16-pair chunks instead of FMAs.  fp32
// accuracy comes from the same 3-pass bf16 split as the big GEMMs:
//   x ~= hi + mid,   a*b ~= a_hi*b_mid + a_mid*b_hi + a_hi*b_hi  (fp32 accumulate).
// Features are pre-split once per call into [n, 2, C] bf16 (hi row, mid row), so
// a neighbor's operand row is gathered with one asynchronous 16-byte copy per
// lane and handed to the MMAs by ldmatrix, never touching registers in between.
//
// Shared-memory rows are padded by 16 bytes so that the eight row reads of one
// ldmatrix fall into distinct bank groups.  Basis functions are stored in a
// permuted order inside every group of 16 (position 8*t + 2*a + b holds
// k = 4*a + 2*t + b): the two accumulator tiles of a tile pair then give every
// lane four consecutive k (or channels), i.e. 128-bit stores and reductions.
#pragma once

#include "basis_proj.cuh"

namespace tfgpc {
namespace bpm {

constexpr int kChunk = 16;  // pairs per MMA step (the k or m extent of m16n8k16)

template <int K>
struct Cfg {
  static_assert(K == 16 || K == 32 || K == 64, "MMA projection: K in {16, 32, 64}");
  static constexpr int kCC = K == 16 ? 128 : (K == 32 ? 64 : 32);  // channels per pass
  static constexpr int kMT = kCC / 16;   // 16-channel tiles per pass
  static constexpr int kNT = K / 8;      // 8-wide basis tiles
  static constexpr int kNTP = K / 16;    // tile pairs
  static constexpr int kFeatStride = kCC * 4 + 16;  // bytes: hi[kCC] | mid[kCC] | pad
  static constexpr int kKStride = K * 2 + 16;       // bytes of one bf16 row over k (+ pad)
  static constexpr int kFeatBytes = kChunk * kFeatStride;
  static constexpr int kBasisBytes = 2 * kChunk * kKStride;   // hi rows, then mid rows
  static constexpr int kDxRawBytes = kCC * K * 4;
  static constexpr int kDxBytes = 2 * kCC * kKStride;         // hi rows, then mid rows
  static constexpr int kFwdWarpBytes = 2 * kFeatBytes + 2 * kBasisBytes;
  static constexpr int kGradWarpBytes = kFeatBytes + kBasisBytes + kDxRawBytes + kDxBytes;
  static constexpr int kBasisVecs = K / 8;   // float4 loads per lane for a 16-row basis chunk
};

// ---- PTX helpers -----------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// d += a (16 x 16, row) * b (16 x 8, col), bf16 operands, fp32 accumulators
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// the three passes of the split product
__device__ __forceinline__ void mma3(float* d, const uint32_t* a_hi, const uint32_t* a_mid,
                                     uint32_t bh0, uint32_t bh1, uint32_t bm0, uint32_t bm1) {
  mma16816(d, a_hi, bm0, bm1);
  mma16816(d, a_mid, bh0, bh1);
  mma16816(d, a_hi, bh0, bh1);
}

__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& mid) {
  split2_bf16(x, y, hi, mid);
}

// 16-byte asynchronous copy; copies nothing and writes zeros when !valid
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n)
               : "memory");
}

__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- the walk over samples ---------------------------------------------------------
//
// A warp takes blocks of 32 consecutive samples, strided over all warps of the
// grid.  The 32 range ends of a block are read with one coalesced load (the
// next block's are fetched while this one is processed) and handed out by
// shuffle, so moving from chunk to chunk and sample to sample costs no memory
// access.  A job is one chunk of up to 16 pairs; a sample without pairs still
// yields one empty job so that its (zero) result gets written.
struct Job {
  int64_t s;     // sample, -1 once the walk is over
  int base;      // first pair of the chunk
  int cnt;       // pairs in the chunk (0 .. 16)
  bool first, last;  // first / last chunk of the sample
  __device__ __forceinline__ bool valid() const { return s >= 0; }
};

struct Walker {
  const int32_t* ranges;
  int64_t ns, blk, stride;
  int lane, li, r_end, a0, nr_end, na0, base, e;
  bool started;

  __device__ __forceinline__ void load_block(int64_t b, int& rend, int& first) const {
    const int64_t s0 = b * 32;
    rend = (s0 + lane < ns) ? __ldg(ranges + s0 + lane) : 0;
    first = (s0 > 0 && s0 < ns) ? __ldg(ranges + s0 - 1) : 0;
  }

  __device__ __forceinline__ void init(const int32_t* r, int64_t n, int64_t warp, int64_t warps,
                                       int ln) {
    ranges = r; ns = n; blk = warp; stride = warps; lane = ln;
    li = 0; base = 0; e = 0; started = false;
    load_block(blk, r_end, a0);
    load_block(blk + stride, nr_end, na0);
  }

  __device__ __forceinline__ Job next() {
    Job j;
    if (started && base + kChunk < e) {
      base += kChunk;
      j.s = blk * 32 + li; j.base = base; j.cnt = min(kChunk, e - base);
      j.first = false; j.last = base + kChunk >= e;
      return j;
    }
    if (started) ++li;
    started = true;
    if (li == 32 || blk * 32 + li >= ns) {
      blk += stride; li = 0;
      r_end = nr_end; a0 = na0;
      load_block(blk + stride, nr_end, na0);
    }
    if (blk * 32 >= ns) {
      j.s = -1; j.base = 0; j.cnt = 0; j.first = j.last = false;
      base = 0; e = 0; started = false; blk = ns;  // stay exhausted
      return j;
    }
    const int prev = __shfl_sync(0xffffffffu, r_end, (li + 31) & 31);
    e = __shfl_sync(0xffffffffu, r_end, li);
    base = li ? prev : a0;
    j.s = blk * 32 + li; j.base = base; j.cnt = min(kChunk, e - base);
    j.first = true; j.last = base + kChunk >= e;
    return j;
  }
};

// Sample that follows s in the walk of its warp (>= ns when there is none).
__device__ __forceinline__ int64_t next_sample(int64_t s, int64_t ns, int64_t stride) {
  if ((s & 31) != 31 && s + 1 < ns) return s + 1;
  return ((s >> 5) + stride) << 5;
}

// ---- staging ---------------------------------------------------------------------------

// Neighbor (point) index of pair base + lane of a job, 0 beyond the chunk.
__device__ __forceinline__ int load_idx(const Job& j, const int2* __restrict__ neigh, int lane) {
  return (j.valid() && lane < j.cnt) ? __ldg(&neigh[j.base + lane].x) : 0;
}

// Starts the gather of a chunk's feature rows: row r of the tile receives
// hi[c0 .. c0+w) and mid[c0 .. c0+w) of point idx(r); rows beyond the chunk are
// zero-filled.  One commit group per call is left to the caller.
template <int K>
__device__ __forceinline__ void issue_features(uint32_t tile, const __nv_bfloat16* __restrict__ fs,
                                               int C, int c0, int w, int idx, int cnt, int lane) {
  typedef Cfg<K> cfg;
  constexpr int kLph = cfg::kCC / 8;           // 16-byte segments per half row
  constexpr int kRpi = 32 / (2 * kLph);        // rows per warp instruction
  const int sub = lane % (2 * kLph), rsub = lane / (2 * kLph);
  const int half = sub / kLph, seg = sub % kLph;
  const bool seg_ok = seg * 8 < w;
  const uint32_t dst0 = tile + half * (cfg::kCC * 2) + seg * 16;
  const int64_t src0 = (int64_t)half * C + c0 + seg * 8;
#pragma unroll
  for (int it = 0; it < kChunk / kRpi; ++it) {
    const int row = it * kRpi + rsub;
    const int j = __shfl_sync(0xffffffffu, idx, row);
    if (seg_ok)
      cp_async16_zfill(dst0 + row * cfg::kFeatStride, fs + (int64_t)j * 2 * C + src0, row < cnt);
  }
}

// Basis rows of a chunk, 16 x K floats contiguous in memory: each lane loads
// K/8 float4 (zeros beyond the chunk) ...
template <int K>
__device__ __forceinline__ void load_basis(const float* __restrict__ basis, int base, int cnt,
                                           int lane, float4* v) {
  const float4* src = reinterpret_cast<const float4*>(basis + (int64_t)base * K);
#pragma unroll
  for (int t = 0; t < Cfg<K>::kBasisVecs; ++t) {
    const int i = lane + 32 * t;
    v[t] = (i / (K / 4) < cnt) ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Writes four consecutive k (4*a4 .. 4*a4+3) of one row, split into hi and mid,
// at their permuted positions.
template <int K>
__device__ __forceinline__ void store_split4(uint8_t* hi_row, uint8_t* mid_row, int a4,
                                             const float4& v) {
  uint32_t h01, m01, h23, m23;
  split2(v.x, v.y, h01, m01);
  split2(v.z, v.w, h23, m23);
  const int off = (16 * (a4 >> 2) + 2 * (a4 & 3)) * 2;  // bytes
  *reinterpret_cast<uint32_t*>(hi_row + off) = h01;
  *reinterpret_cast<uint32_t*>(hi_row + off + 16) = h23;
  *reinterpret_cast<uint32_t*>(mid_row + off) = m01;
  *reinterpret_cast<uint32_t*>(mid_row + off + 16) = m23;
}

// ... and stores them split into the chunk's basis tile (hi rows, then mid rows).
template <int K>
__device__ __forceinline__ void store_basis(uint8_t* tile, int lane, const float4* v) {
  typedef Cfg<K> cfg;
#pragma unroll
  for (int t = 0; t < cfg::kBasisVecs; ++t) {
    const int i = lane + 32 * t;
    const int row = i / (K / 4), a4 = i % (K / 4);
    store_split4<K>(tile + row * cfg::kKStride, tile + (kChunk + row) * cfg::kKStride, a4, v[t]);
  }
}

// ---- forward ---------------------------------------------------------------------------
//
// X[s] as D[c, k] += A[c, pair] * B[pair, k] per chunk: A comes transposed out of
// the gathered feature rows (ldmatrix.trans), B transposed out of the staged
// basis rows.  Features of chunk i+1 are in flight, and its basis rows and the
// indices of chunk i+2 are on their way to registers, while chunk i is multiplied.
// OUT = 0: fp32 [ns, C, K] (the op's output).  OUT = 1: the same values split
// into two bf16 arrays [ns, C*K] (left operand of the tensor-core GEMM).
template <int K, int OUT>
__global__ void __launch_bounds__(352, 1)
basis_proj_mma_kernel(int C, int64_t ns, const float* __restrict__ basis,
                      const __nv_bfloat16* __restrict__ fs, const int2* __restrict__ neigh,
                      const int32_t* __restrict__ ranges, float* __restrict__ out,
                      __nv_bfloat16* __restrict__ out_hi, __nv_bfloat16* __restrict__ out_mid) {
  typedef Cfg<K> cfg;
  extern __shared__ __align__(128) uint8_t bpm_smem[];
  const int lane = threadIdx.x & 31;
  const int warp_in_block = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  uint8_t* wsm = bpm_smem + (size_t)warp_in_block * cfg::kFwdWarpBytes;
  // two feature tiles, then two basis tiles
  auto feat_tile = [&](int b) { return wsm + b * cfg::kFeatBytes; };
  auto basis_tile = [&](int b) { return wsm + 2 * cfg::kFeatBytes + b * cfg::kBasisBytes; };
  const int64_t warp = (int64_t)blockIdx.x * warps_per_block + warp_in_block;
  const int64_t warps = (int64_t)gridDim.x * warps_per_block;
  const int g = lane >> 2, q = lane & 3;
  const int mi = lane >> 3, r = lane & 7;
  // ldmatrix row addresses (bytes inside a tile) of this lane
  const uint32_t a_off = (r + 8 * (mi >> 1)) * cfg::kFeatStride + 8 * (mi & 1) * 2;
  const uint32_t b_off = (r + 8 * (mi & 1)) * cfg::kKStride + 8 * (mi >> 1) * 2;

  for (int c0 = 0; c0 < C; c0 += cfg::kCC) {
    const int w = min(cfg::kCC, C - c0);
    const int mt_cnt = w >> 4;
    Walker walk;
    walk.init(ranges, ns, warp, warps, lane);
    Job cur = walk.next(), n1 = walk.next(), n2 = walk.next();
    int idx1 = load_idx(n1, neigh, lane);
    __syncwarp();
    if (cur.valid()) {
      const int idx0 = load_idx(cur, neigh, lane);
      issue_features<K>(smem_addr(feat_tile(0)), fs, C, c0, w, idx0, cur.cnt, lane);
      float4 bv[cfg::kBasisVecs];
      load_basis<K>(basis, cur.base, cur.cnt, lane, bv);
      store_basis<K>(basis_tile(0), lane, bv);
    }
    cp_commit();
    float acc[cfg::kMT][cfg::kNT][4];
    int buf = 0;
    while (cur.valid()) {
      const int idx2 = load_idx(n2, neigh, lane);
      float4 bv[cfg::kBasisVecs];
      if (n1.valid()) {
        issue_features<K>(smem_addr(feat_tile(buf ^ 1)), fs, C, c0, w, idx1, n1.cnt, lane);
        load_basis<K>(basis, n1.base, n1.cnt, lane, bv);
      }
      cp_commit();
      cp_wait<1>();   // the features of `cur` have landed
      __syncwarp();
      if (cur.first) {
#pragma unroll
        for (int mt = 0; mt < cfg::kMT; ++mt)
#pragma unroll
          for (int nt = 0; nt < cfg::kNT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.0f;
      }
      if (cur.cnt > 0) {
        const uint32_t ft = smem_addr(feat_tile(buf)) + a_off;
        const uint32_t bt = smem_addr(basis_tile(buf)) + b_off;
        uint32_t bh[cfg::kNTP][4], bm[cfg::kNTP][4];
#pragma unroll
        for (int j = 0; j < cfg::kNTP; ++j) {
          ldsm_x4_t(bt + j * 32, bh[j]);
          ldsm_x4_t(bt + kChunk * cfg::kKStride + j * 32, bm[j]);
        }
        // Two 16-channel tiles at a time, and pass by pass over all their
        // accumulator tiles: consecutive MMAs never touch the same accumulator,
        // so none of them waits for the one before it.
#pragma unroll
        for (int mt = 0; mt < cfg::kMT; mt += 2) {
          if (mt < mt_cnt) {
            const bool two = mt + 1 < mt_cnt;
            uint32_t ah[2][4], am[2][4];
            ldsm_x4_t(ft + mt * 32, ah[0]);
            ldsm_x4_t(ft + cfg::kCC * 2 + mt * 32, am[0]);
            if (two) {
              ldsm_x4_t(ft + (mt + 1) * 32, ah[1]);
              ldsm_x4_t(ft + cfg::kCC * 2 + (mt + 1) * 32, am[1]);
            }
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                if (u == 0 || two) {
                  const uint32_t* a = pass == 1 ? am[u] : ah[u];
#pragma unroll
                  for (int j = 0; j < cfg::kNTP; ++j) {
                    const uint32_t* b = pass == 0 ? bm[j] : bh[j];
                    mma16816(acc[mt + u][2 * j], a, b[0], b[1]);
                    mma16816(acc[mt + u][2 * j + 1], a, b[2], b[3]);
                  }
                }
              }
            }
          }
        }
      }
      if (cur.last) {
        // lane (g, q): channels c0 + 16*mt + g (+8), basis functions 16*j + 4*q .. +3
        const int64_t obase = (cur.s * C + c0 + g) * K + 4 * q;
#pragma unroll
        for (int mt = 0; mt < cfg::kMT; ++mt) {
          if (mt < mt_cnt) {
#pragma unroll
            for (int j = 0; j < cfg::kNTP; ++j) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {   // rows g and g + 8
                const int64_t o = obase + (int64_t)(16 * mt + 8 * h) * K + 16 * j;
                if (OUT == 0) {
                  *reinterpret_cast<float4*>(out + o) =
                      make_float4(acc[mt][2 * j][2 * h], acc[mt][2 * j][2 * h + 1],
                                  acc[mt][2 * j + 1][2 * h], acc[mt][2 * j + 1][2 * h + 1]);
                } else {
                  uint2 hv, mv;
                  split2(acc[mt][2 * j][2 * h], acc[mt][2 * j][2 * h + 1], hv.x, mv.x);
                  split2(acc[mt][2 * j + 1][2 * h], acc[mt][2 * j + 1][2 * h + 1], hv.y, mv.y);
                  *reinterpret_cast<uint2*>(out_hi + o) = hv;
                  *reinterpret_cast<uint2*>(out_mid + o) = mv;
                }
              }
            }
          }
        }
      }
      if (n1.valid()) store_basis<K>(basis_tile(buf ^ 1), lane, bv);
      __syncwarp();
      cur = n1; n1 = n2; n2 = walk.next();
      idx1 = idx2;
      buf ^= 1;
    }
    cp_wait<0>();
    __syncwarp();
  }
}

// ---- gradients ---------------------------------------------------------------------------
//
// Per sample the incoming gradient dX[s] (C x K floats) is copied raw into
// shared memory while the previous sample is still being processed, then split
// once into bf16 hi/mid rows [c][k].  Per chunk of 16 pairs:
//   (1) dbasis[pair, k] = A[pair, c] * B[c, k]: A straight out of the gathered
//       feature rows, B transposed out of the dX rows; 128-bit stores;
//   (2) dfeat[pair, c]  = A[pair, k] * B[k, c]: A out of the staged basis rows,
//       B out of the dX rows (whose order inside a tile is chosen so that a lane
//       ends up with four consecutive channels); one 128-bit reduction per lane
//       and 4 channels into dfeat[nbr(pair)].
// The feature rows are dead after (1), so the gather of the next chunk is
// started there and runs under (2).  dbasis is written, not accumulated (every
// pair belongs to exactly one sample); dfeat must be zero on entry.
template <int K>
__global__ void __launch_bounds__(224, 1)
basis_proj_grads_mma_kernel(int C, int64_t ns, int64_t M, const float* __restrict__ basis,
                            const __nv_bfloat16* __restrict__ fs, const int2* __restrict__ neigh,
                            const int32_t* __restrict__ ranges,
                            const float* __restrict__ in_grads, float* __restrict__ dbasis,
                            float* __restrict__ dfeat) {
  typedef Cfg<K> cfg;
  extern __shared__ __align__(128) uint8_t bpm_smem[];
  const int lane = threadIdx.x & 31;
  const int warp_in_block = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  uint8_t* wsm = bpm_smem + (size_t)warp_in_block * cfg::kGradWarpBytes;
  uint8_t* feat_tile = wsm;
  uint8_t* basis_tile = feat_tile + cfg::kFeatBytes;
  uint8_t* dx_raw = basis_tile + cfg::kBasisBytes;
  uint8_t* dx_tile = dx_raw + cfg::kDxRawBytes;   // hi rows [c], then mid rows [c]
  const int64_t warp = (int64_t)blockIdx.x * warps_per_block + warp_in_block;
  const int64_t warps = (int64_t)gridDim.x * warps_per_block;
  const int g = lane >> 2, q = lane & 3;
  const int mi = lane >> 3, r = lane & 7;
  // (1) A: matrices (pairs 0-7 | 8-15) x (c 0-7 | 8-15) of a 16-channel step
  const uint32_t a1_off = (r + 8 * (mi & 1)) * cfg::kFeatStride + 8 * (mi >> 1) * 2;
  // (1) B, transposed: matrices (c 0-7 | 8-15) x (positions 0-7 | 8-15)
  const uint32_t b1_off = (r + 8 * (mi & 1)) * cfg::kKStride + 8 * (mi >> 1) * 2;
  // (2) A: matrices (pairs 0-7 | 8-15) x (positions 0-7 | 8-15) of a 16-k step
  const uint32_t a2_off = (r + 8 * (mi & 1)) * cfg::kKStride + 8 * (mi >> 1) * 2;
  // (2) B: matrices (tile 2j | 2j+1) x (positions 0-7 | 8-15); row n of tile 2j+t
  // is channel 4*(n/2) + 2*t + (n%2) of the 16-channel group
  const uint32_t b2_off = (4 * (r >> 1) + 2 * (mi >> 1) + (r & 1)) * cfg::kKStride + 8 * (mi & 1) * 2;
  constexpr int kDxMid = cfg::kCC * cfg::kKStride;
  constexpr int kBasisMid = kChunk * cfg::kKStride;

  // pairs beyond the last range belong to no sample: their gradient is zero
  if (blockIdx.x == 0 && warp_in_block == 0) {
    const int64_t covered = ns > 0 ? __ldg(ranges + ns - 1) : 0;
    for (int64_t i = covered * K + lane; i < M * K; i += 32) dbasis[i] = 0.0f;
  }

  auto issue_dx = [&](int64_t s, int c0, int w) {
    // w*K floats, contiguous
    const float* src = in_grads + (s * C + c0) * K;
    const uint32_t dst = smem_addr(dx_raw);
    for (int i = lane; i < w * (K / 4); i += 32) cp_async16_zfill(dst + i * 16, src + i * 4, true);
  };

  for (int c0 = 0; c0 < C; c0 += cfg::kCC) {
    const int w = min(cfg::kCC, C - c0);
    const int ks_cnt = w >> 4;     // 16-channel steps of (1) = tile pairs of (2)
    Walker walk;
    walk.init(ranges, ns, warp, warps, lane);
    Job cur = walk.next(), n1 = walk.next(), n2 = walk.next();
    int idx0 = load_idx(cur, neigh, lane);
    int idx1 = load_idx(n1, neigh, lane);
    float4 bv[cfg::kBasisVecs];
    __syncwarp();
    if (cur.valid()) {
      issue_dx(cur.s, c0, w);
      issue_features<K>(smem_addr(feat_tile), fs, C, c0, w, idx0, cur.cnt, lane);
      load_basis<K>(basis, cur.base, cur.cnt, lane, bv);
    }
    cp_commit();
    while (cur.valid()) {
      cp_wait<0>();   // features of `cur`, and dX of its sample if this is its first chunk
      __syncwarp();
      if (cur.first) {
        const float4* raw = reinterpret_cast<const float4*>(dx_raw);
        for (int i = lane; i < w * (K / 4); i += 32) {
          const int row = i / (K / 4), a4 = i % (K / 4);
          store_split4<K>(dx_tile + row * cfg::kKStride, dx_tile + kDxMid + row * cfg::kKStride, a4,
                          raw[i]);
        }
        __syncwarp();
        const int64_t sn = next_sample(cur.s, ns, warps);
        if (sn < ns) issue_dx(sn, c0, w);
        cp_commit();
      }
      store_basis<K>(basis_tile, lane, bv);
      __syncwarp();
      const uint32_t ft = smem_addr(feat_tile), bt = smem_addr(basis_tile), dt = smem_addr(dx_tile);
      // ---- (1) dbasis
      if (cur.cnt > 0) {
        // one accumulator set per pass and per parity of the channel step: the
        // MMAs of a step are independent of each other and of the previous step
        constexpr int kPar = K == 64 ? 1 : 2;   // register budget
        float dbp[kPar][3][cfg::kNT][4];
#pragma unroll
        for (int e = 0; e < kPar; ++e)
#pragma unroll
          for (int p = 0; p < 3; ++p)
#pragma unroll
            for (int nt = 0; nt < cfg::kNT; ++nt)
#pragma unroll
              for (int i = 0; i < 4; ++i) dbp[e][p][nt][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < cfg::kMT; ++ks) {
          if (ks < ks_cnt) {
            uint32_t ah[4], am[4];
            ldsm_x4(ft + a1_off + ks * 32, ah);
            ldsm_x4(ft + a1_off + cfg::kCC * 2 + ks * 32, am);
#pragma unroll
            for (int j = 0; j < cfg::kNTP; ++j) {
              uint32_t bh[4], bm[4];
              ldsm_x4_t(dt + b1_off + ks * 16 * cfg::kKStride + j * 32, bh);
              ldsm_x4_t(dt + kDxMid + b1_off + ks * 16 * cfg::kKStride + j * 32, bm);
              mma16816(dbp[ks & (kPar - 1)][0][2 * j], ah, bm[0], bm[1]);
              mma16816(dbp[ks & (kPar - 1)][0][2 * j + 1], ah, bm[2], bm[3]);
              mma16816(dbp[ks & (kPar - 1)][1][2 * j], am, bh[0], bh[1]);
              mma16816(dbp[ks & (kPar - 1)][1][2 * j + 1], am, bh[2], bh[3]);
              mma16816(dbp[ks & (kPar - 1)][2][2 * j], ah, bh[0], bh[1]);
              mma16816(dbp[ks & (kPar - 1)][2][2 * j + 1], ah, bh[2], bh[3]);
            }
          }
        }
        float db[cfg::kNT][4];
#pragma unroll
        for (int nt = 0; nt < cfg::kNT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            db[nt][i] = ((dbp[0][0][nt][i] + dbp[kPar - 1][0][nt][i] * (kPar - 1)) +
                         (dbp[0][1][nt][i] + dbp[kPar - 1][1][nt][i] * (kPar - 1))) +
                        (dbp[0][2][nt][i] + dbp[kPar - 1][2][nt][i] * (kPar - 1));
        // lane (g, q): pairs g and g + 8, basis functions 16*j + 4*q .. +3
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int row = g + 8 * h;
          if (row < cur.cnt) {
            float4* dst = reinterpret_cast<float4*>(dbasis + (int64_t)(cur.base + row) * K + 4 * q);
#pragma unroll
            for (int j = 0; j < cfg::kNTP; ++j) {
              float4 v = make_float4(db[2 * j][2 * h], db[2 * j][2 * h + 1], db[2 * j + 1][2 * h],
                                     db[2 * j + 1][2 * h + 1]);
              if (c0 > 0) {
                const float4 o = dst[4 * j];
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              dst[4 * j] = v;
            }
          }
        }
      }
      __syncwarp();   // every lane is done with the feature tile
      // ---- prefetch for the next chunks
      const int idx2 = load_idx(n2, neigh, lane);
      if (n1.valid()) {
        issue_features<K>(smem_addr(feat_tile), fs, C, c0, w, idx1, n1.cnt, lane);
        load_basis<K>(basis, n1.base, n1.cnt, lane, bv);
      }
      cp_commit();
      // ---- (2) dfeat
      if (cur.cnt > 0) {
        float df[cfg::kMT * 2][4];
#pragma unroll
        for (int nt = 0; nt < cfg::kMT * 2; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) df[nt][i] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < cfg::kNTP; ++kk) {
          uint32_t ah[4], am[4];
          ldsm_x4(bt + a2_off + kk * 32, ah);
          ldsm_x4(bt + kBasisMid + a2_off + kk * 32, am);
#pragma unroll
          for (int j = 0; j < cfg::kMT; j += 2) {
            if (j < ks_cnt) {
              const bool two = j + 1 < ks_cnt;
              uint32_t bh[2][4], bm[2][4];
              ldsm_x4(dt + b2_off + j * 16 * cfg::kKStride + kk * 32, bh[0]);
              ldsm_x4(dt + kDxMid + b2_off + j * 16 * cfg::kKStride + kk * 32, bm[0]);
              if (two) {
                ldsm_x4(dt + b2_off + (j + 1) * 16 * cfg::kKStride + kk * 32, bh[1]);
                ldsm_x4(dt + kDxMid + b2_off + (j + 1) * 16 * cfg::kKStride + kk * 32, bm[1]);
              }
#pragma unroll
              for (int pass = 0; pass < 3; ++pass) {
                const uint32_t* a = pass == 1 ? am : ah;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  if (u == 0 || two) {
                    const uint32_t* b = pass == 0 ? bm[u] : bh[u];
                    mma16816(df[2 * (j + u)], a, b[0], b[1]);
                    mma16816(df[2 * (j + u) + 1], a, b[2], b[3]);
                  }
                }
              }
            }
          }
        }
        // lane (g, q): pairs g and g + 8, channels c0 + 16*j + 4*q .. +3
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int row = g + 8 * h;
          const int pt = __shfl_sync(0xffffffffu, idx0, row);
          if (row < cur.cnt) {
            float* dst = dfeat + (int64_t)pt * C + c0 + 4 * q;
#pragma unroll
            for (int j = 0; j < cfg::kMT; ++j) {
              if (j < ks_cnt)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 16 * j),
                             "f"(df[2 * j][2 * h]), "f"(df[2 * j][2 * h + 1]),
                             "f"(df[2 * j + 1][2 * h]), "f"(df[2 * j + 1][2 * h + 1])
                             : "memory");
            }
          }
        }
      }
      cur = n1; n1 = n2; n2 = walk.next();
      idx0 = idx1; idx1 = idx2;
    }
    cp_wait<0>();
    __syncwarp();
  }
}

}  // namespace bpm
}  // namespace tfgpc
