// Gradients of the basis projection on tcgen05 tensor cores (C = 128, K = 16).
//
// For a pair m of sample s with neighbor j:
//   dbasis[m, k]  = sum_c feat[j, c] * dX[s, c, k]
//   dfeat[j, c]  += sum_k basis[m, k] * dX[s, c, k]
// Per sample these products have only ~32 rows, too few for a 128-row tensor
// core tile.  The kernel therefore works on groups of G consecutive samples (G =
// 4, or 3 where four samples would mostly overflow one block) whose pairs
// (contiguous in the neighbor list) are cut into blocks of 128 rows, and writes
// both gradients as block-sparse products against the group's concatenated
// gradient dXcat[c, (s_local, k)] (128 x 16 G):
//   (1) D1[128 pairs, 16 G] = F[128 pairs, 128 c] * dXcat         -> a pair's own
//       sample block of 16 columns is its dbasis row, the rest is discarded;
//   (2) D2[128 c, 128 pairs] = dXcat * Bx^T, where Bx[128 pairs, 16 G] holds the
//       pair's basis row in the 16 columns of its own sample and zeros elsewhere
//       (channels on the accumulator rows, so that a warp of the epilogue adds 32
//       consecutive channels of one neighbor's gradient row per instruction).
// Most of the MMA work multiplies zeros or is thrown away, which is cheap next to
// what it saves: no per-sample staging, no warp-level bookkeeping per 16 pairs.
// fp32 accuracy comes from the 3-pass bf16 split of both operands (hi*mid +
// mid*hi + hi*hi into fp32 tensor memory), as in gemm_sm100.cu.
//
// Operands in shared memory, all as 128-byte rows with the 16-byte chunks of a
// row XOR-ed with (row % 8), i.e. the 128-byte swizzle of the MMA descriptors:
//   F      gathered from the pre-split features ([n, 2, C] bf16) by 16-byte
//          cp.async, one 64-channel block (hi 16 KB + mid 16 KB) per ring slot;
//   Bx     built by the producer warps from the fp32 basis rows;
//   dXcat  produced in exactly this image by the dX GEMM (gemm_bf16x3_grad_image)
//          and fetched with one 32 KB bulk copy per group.  The same bytes serve
//          as the MN-major B operand of (1) and the K-major A operand of (2).
// Roles: warps 0-7 gather and build; warps 8 and 9 issue the MMAs of (1) and (2)
// (the MMAs are small, and two issuing threads keep the tensor pipe fed where
// one cannot); warp 10 fetches dXcat; warps 11-18 drain the two accumulators
// (double buffered in tensor memory): dbasis rows with plain stores, dfeat with
// coalesced reductions.
// Every mbarrier wait is bounded; a wait that runs out sets the error flag and
// the kernel drains and frees its tensor memory.
#include "basis_proj_tc.cuh"

namespace tfgpc {

using namespace tc;
using namespace bptc;

namespace {

#ifdef TFGPC_TC_TIMING
__device__ long long tt_array[160 * 5 * 8];
#endif

constexpr int kProdWarps = 8;
constexpr int kMmaWarp = 8;            // issues product (1); warp 9 issues product (2)
constexpr int kDxWarp = 10;
constexpr int kEpiWarp0 = 11;          // first of the 8 epilogue warps
constexpr int kThreads = 19 * 32;
constexpr int kSlots = 3;              // ring of 64-channel feature blocks
constexpr uint32_t kPart = 16384;      // one 128 x 128-byte operand tile (hi or mid)
constexpr uint32_t kSlotBytes = 2 * kPart;
constexpr uint32_t kBxBytes = 2 * kPart;
constexpr uint32_t kDxBytes = 2 * kPart;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCols = 192;     // D1 (64 columns) + D2 (128 columns)
constexpr size_t kSmemBytes = (size_t)kSlots * kSlotBytes + 2 * kBxBytes + 2 * kDxBytes + 1024 + 256;

struct Barriers {
  uint64_t f_full[kSlots], f_empty[kSlots];
  uint64_t bx_full[2], bx_empty[2];
  uint64_t dx_full[2], dx_empty[2];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
basis_proj_grads_tc_kernel(int64_t ns, int64_t M, const float* __restrict__ basis,
                           const __nv_bfloat16* __restrict__ fs, const int2* __restrict__ neigh,
                           const int32_t* __restrict__ ranges, const uint8_t* __restrict__ image,
                           float* __restrict__ dbasis, float* __restrict__ dfeat, uint32_t idesc1,
                           uint32_t idesc2, int* err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* f_ring = smem;
  uint8_t* bx = f_ring + (size_t)kSlots * kSlotBytes;
  uint8_t* dx = bx + 2 * kBxBytes;
  Barriers* bars = (Barriers*)(dx + 2 * kDxBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t groups = (ns + G - 1) / G;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(smem_u32(&bars->f_full[i]), kProdWarps * 32);
      mbar_init(smem_u32(&bars->f_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->bx_full[i]), kProdWarps);
      mbar_init(smem_u32(&bars->bx_empty[i]), 1);
      mbar_init(smem_u32(&bars->dx_full[i]), 1);
      mbar_init(smem_u32(&bars->dx_empty[i]), 2);
      mbar_init(smem_u32(&bars->acc_full[i]), 2);
      mbar_init(smem_u32(&bars->acc_empty[i]), 8);
    }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;

  // pairs beyond the last range belong to no sample: their gradient is zero
  if (blockIdx.x == 0 && warp == kDxWarp) {
    const int64_t covered = ns > 0 ? __ldg(ranges + ns - 1) : 0;
    for (int64_t i = covered * kK + lane; i < M * kK; i += 32) dbasis[i] = 0.0f;
  }

  if (warp < kProdWarps) {
    // ------------------------------------------------------------- producers
    // warp w owns rows 16 w .. 16 w + 15 of every block.  Nothing here waits for
    // data: the neighbor ids and basis rows of block i+1 are fetched into
    // registers while block i is issued, and the gathers of a feature block
    // signal their own completion (cp.async.mbarrier.arrive), so that a warp
    // blocks only when the ring has no free slot.
    const int row_base = warp * 16;
    const int brow = lane >> 1, bh = lane & 1;     // basis: two lanes per row
    // gather: lanes 0-15 take row `it`, lanes 16-31 row `it + 8` of the warp's 16;
    // within a row, lane -> (hi | mid part, 16-byte chunk j of the 64-channel block)
    const int l4 = lane >> 4, part = (lane >> 3) & 1, j = lane & 7;
    const int idx_row = (lane & 7) + 8 * l4;
    const __nv_bfloat16* const fs_lane = fs + part * kC + j * 8;
    const uint32_t dst_lane = part * kPart + (row_base + 8 * l4) * 128;
    uint32_t unit = 0, item = 0;
    ItemWalk<G> walk;
    walk.init(ranges, ns, groups);
    // registers of the block being prefetched
    Tile t_n = walk.t;
    int m0_n = 0, idx_n = 0;
    float4 b0_n = make_float4(0.f, 0.f, 0.f, 0.f), b1_n = b0_n;
    auto prefetch = [&]() {
      t_n = walk.t;
      m0_n = walk.t.pa + walk.b * kRows + row_base;
      // ids of rows 0-7 in lanes 0-7, of rows 8-15 in lanes 16-23: a shuffle within
      // half warps then hands row it + 8 * (lane / 16) to every lane
      idx_n = ((lane & 8) == 0 && m0_n + idx_row < t_n.pe) ? __ldg(&neigh[m0_n + idx_row].x) : 0;
      b0_n = b1_n = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m0_n + brow < t_n.pe) {
        const float4* src =
            reinterpret_cast<const float4*>(basis + (int64_t)(m0_n + brow) * kK + 8 * bh);
        b0_n = __ldg(src);
        b1_n = __ldg(src + 1);
      }
    };
    if (walk.valid) prefetch();
    TT_DECL
    while (walk.valid) {
      TT_MARK(tp0)
      const Tile t = t_n;
      const int m0 = m0_n, my_idx = idx_n;
      const float4 b0 = b0_n, b1 = b1_n;
      walk.advance();
      if (walk.valid) prefetch();
      TT_MARK(tp1)
      TT_ADD(2, tp1 - tp0);
      // ---- F: two 64-channel blocks
#ifdef TFGPC_TC_PROD_HOIST
      // source rows of this lane's eight copies, the same for both channel blocks
      const __nv_bfloat16* src_row[8];
#pragma unroll
      for (int it = 0; it < 8; ++it)
        src_row[it] = fs_lane + (int64_t)__shfl_sync(0xffffffffu, my_idx, it, 16) * 2 * kC;
#endif
#pragma unroll
      for (int kb = 0; kb < 2; ++kb, ++unit) {
        const uint32_t slot = unit % kSlots;
        TT_WAIT(0, smem_u32(&bars->f_empty[slot]), ((unit / kSlots) & 1) ^ 1);
        const uint32_t base = smem_u32(f_ring + (size_t)slot * kSlotBytes) + dst_lane;
        const int nv = t.pe - m0 - 8 * l4;   // this lane's rows `it` with it < nv exist
#pragma unroll
        for (int it = 0; it < 8; ++it) {
#ifdef TFGPC_TC_PROD_HOIST
          if (it < nv) cp_async16(base + it * 128 + ((j ^ it) << 4), src_row[it] + kb * 64);
#else
          const int idx = __shfl_sync(0xffffffffu, my_idx, it, 16);
          // row row_base + 8 * l4 + it: (row % 8) == it, the swizzle is a constant
          if (it < nv)
            cp_async16(base + it * 128 + ((j ^ it) << 4), fs_lane + (int64_t)idx * 2 * kC + kb * 64);
#endif
        }
        // arrives on the slot's barrier once this thread's copies have landed
        asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];"
                     ::"r"(smem_u32(&bars->f_full[slot])) : "memory");
      }
      TT_MARK(tp2)
      TT_ADD(3, tp2 - tp1);
      // ---- Bx: this lane's half row in the columns of its sample, zeros elsewhere
      {
        const uint32_t stage = item & 1;
        TT_WAIT(1, smem_u32(&bars->bx_empty[stage]), ((item >> 1) & 1) ^ 1);
        const int bm = m0 + brow;
        uint4 hv, mv;
        split2_bf16(b0.x, b0.y, hv.x, mv.x);
        split2_bf16(b0.z, b0.w, hv.y, mv.y);
        split2_bf16(b1.x, b1.y, hv.z, mv.z);
        split2_bf16(b1.z, b1.w, hv.w, mv.w);
        const int sl = bm < t.pe ? t.local_sample(bm) : -1;
        const int r = row_base + brow;
        uint8_t* rowp = bx + (size_t)stage * kBxBytes + r * 128;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int q = 0; q < G; ++q) {
          const int pos = ((2 * q + bh) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(rowp + pos) = (q == sl) ? hv : zero;
          *reinterpret_cast<uint4*>(rowp + kPart + pos) = (q == sl) ? mv : zero;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->bx_full[stage]));
      }
      ++item;
      TT_ADD(6, 1);
      TT_MARK(tp3)
      TT_ADD(4, tp3 - tp2);
    }
#ifdef TFGPC_TC_TIMING
    if (warp == 0 && lane == 0) TT_STORE(0);
#endif
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ----------------------------------------------------------- MMA issuers
    // Both walk the same blocks; each commits to the accumulator's and the dXcat
    // buffer's barriers, which therefore expect two arrivals.
    const bool first = warp == kMmaWarp;
    if (lane == 0) {
      uint32_t unit = 0, item = 0, tile_i = 0;
      Tile next = load_tile<G>(ranges, ns, blockIdx.x);
      TT_DECL
      for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
        const Tile t = next;
        next = load_tile<G>(ranges, ns, g + gridDim.x);
        const int nb = t.blocks();
        if (nb == 0) continue;
        const uint32_t dbuf = tile_i & 1;
        TT_WAIT(0, smem_u32(&bars->dx_full[dbuf]), (tile_i >> 1) & 1);
        const uint32_t dx_hi = smem_u32(dx + (size_t)dbuf * kDxBytes), dx_mid = dx_hi + kPart;
        for (int b = 0; b < nb; ++b, ++item) {
          const uint32_t abuf = item & 1;
          TT_WAIT(1, smem_u32(&bars->acc_empty[abuf]), ((item >> 1) & 1) ^ 1);
          tc_fence_after();
          const uint32_t d1 = tmem_base + abuf * kAccCols, d2 = d1 + 64;   // D1 uses 16 G columns
          if (first) {
            // (1) D1 = F * dXcat: reduction over the 128 channels, two ring slots
            uint32_t accumulate = 0;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb, ++unit) {
              const uint32_t slot = unit % kSlots;
              TT_WAIT(2, smem_u32(&bars->f_full[slot]), (unit / kSlots) & 1);
              fence_proxy_async();   // the gathered rows were written through the generic proxy
              tc_fence_after();
              const uint32_t f_hi = smem_u32(f_ring + (size_t)slot * kSlotBytes), f_mid = f_hi + kPart;
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                // A: K-major rows of 128 bytes, 32 bytes per step.  B: MN-major, the
                // 16 channel rows of a step are 2048 bytes further on.
                const uint32_t boff = (uint32_t)(kb * 64 + kk * 16) * 128;
                const uint64_t da_hi = make_desc(f_hi + kk * 32, 16, 1024);
                const uint64_t da_mid = make_desc(f_mid + kk * 32, 16, 1024);
                const uint64_t db_hi = make_desc(dx_hi + boff, 8192, 1024);
                const uint64_t db_mid = make_desc(dx_mid + boff, 8192, 1024);
                umma_bf16(d1, da_hi, db_mid, idesc1, accumulate);
                umma_bf16(d1, da_mid, db_hi, idesc1, 1u);
                umma_bf16(d1, da_hi, db_hi, idesc1, 1u);
                accumulate = 1u;
              }
              umma_commit(smem_u32(&bars->f_empty[slot]));
            }
          } else {
            // (2) D2 = dXcat * Bx^T: reduction over the 64 (sample, k) columns
            TT_WAIT(2, smem_u32(&bars->bx_full[abuf]), (item >> 1) & 1);
            tc_fence_after();
            const uint32_t bx_hi = smem_u32(bx + (size_t)abuf * kBxBytes), bx_mid = bx_hi + kPart;
            uint32_t accumulate = 0;
#pragma unroll
            for (int kk = 0; kk < G; ++kk) {   // one step of 16 columns per sample of the group
              const uint64_t da_hi = make_desc(dx_hi + kk * 32, 16, 1024);
              const uint64_t da_mid = make_desc(dx_mid + kk * 32, 16, 1024);
              const uint64_t db_hi = make_desc(bx_hi + kk * 32, 16, 1024);
              const uint64_t db_mid = make_desc(bx_mid + kk * 32, 16, 1024);
              umma_bf16(d2, da_hi, db_mid, idesc2, accumulate);
              umma_bf16(d2, da_mid, db_hi, idesc2, 1u);
              umma_bf16(d2, da_hi, db_hi, idesc2, 1u);
              accumulate = 1u;
            }
            umma_commit(smem_u32(&bars->bx_empty[abuf]));
          }
          umma_commit(smem_u32(&bars->acc_full[abuf]));
        }
        umma_commit(smem_u32(&bars->dx_empty[dbuf]));
        ++tile_i;
      }
      TT_ADD(6, item);
      TT_STORE(first ? 1 : 2);
    }
  } else if (warp == kDxWarp) {
    // ------------------------------------------------------- dXcat loader
    if (lane == 0) {
      uint32_t tile_i = 0;
      Tile next = load_tile<G>(ranges, ns, blockIdx.x);
      TT_DECL
      for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
        const Tile t = next;
        next = load_tile<G>(ranges, ns, g + gridDim.x);
        if (t.blocks() == 0) continue;
        const uint32_t dbuf = tile_i & 1;
        TT_WAIT(0, smem_u32(&bars->dx_empty[dbuf]), ((tile_i >> 1) & 1) ^ 1);
        const uint32_t full = smem_u32(&bars->dx_full[dbuf]);
        mbar_expect_tx(full, kDxBytes);
        bulk_g2s(smem_u32(dx + (size_t)dbuf * kDxBytes), image + g * (int64_t)kDxBytes, kDxBytes, full);
        ++tile_i;
      }
      TT_ADD(6, tile_i);
      TT_STORE(3);
    }
  } else {
    // -------------------------------------------------------------- epilogue
    // Two warps per quarter of the tensor-memory lanes.  D1 (lanes = pairs):
    // warp half 0 stores the 16 columns of each row's own sample as its dbasis
    // row.  D2 (lanes = channels, columns = pairs): half h takes the 32-pair
    // column blocks h and h + 2; for every pair the warp adds its 32 channels to
    // the neighbor's gradient row, 128 contiguous bytes per instruction.
    const int quarter = warp & 3;             // tensor-memory lanes 32 * quarter ...
    const int half = (warp - kEpiWarp0) >> 2;
    const int r = quarter * 32 + lane;        // this thread's accumulator row
    float* const dcol = dfeat + r;            // channel r of every gradient row
    ItemWalk<G> walk;
    walk.init(ranges, ns, groups);
    uint32_t item = 0;
    TT_DECL
    for (; walk.valid; walk.advance(), ++item) {
      TT_MARK(te0)
      const Tile t = walk.t;
      const int m_first = t.pa + walk.b * kRows;
      const int rows = min(kRows, t.pe - m_first);   // pairs in this block
      // neighbor ids of this warp's two column blocks (lane = pair)
      int pts[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int mp = m_first + 32 * (half + 2 * u) + lane;
        pts[u] = mp < t.pe ? __ldg(&neigh[mp].x) : 0;
      }
      const uint32_t abuf = item & 1;
      TT_WAIT(0, smem_u32(&bars->acc_full[abuf]), (item >> 1) & 1);
      tc_fence_after();
      const bool ok = !*abort_flag;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + abuf * kAccCols;
      TT_MARK(te1)
      if (half == 0) {
        const int m = m_first + r;
        const bool live = ok && m < t.pe;
        const int sl = live ? t.local_sample(m) : -1;
#pragma unroll
        for (int q = 0; q < G; ++q) {
          if (__any_sync(0xffffffffu, sl == q)) {
            uint32_t v[16];
            tmem_ld_x16(taddr + 16 * q, v);
            if (sl == q) {
              // the row's 64 bytes as two whole 32-byte sectors
              float* dst = dbasis + (int64_t)m * kK;
#pragma unroll
              for (int i = 0; i < 2; ++i)
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                             ::"l"(dst + 8 * i), "r"(v[8 * i]), "r"(v[8 * i + 1]), "r"(v[8 * i + 2]),
                               "r"(v[8 * i + 3]), "r"(v[8 * i + 4]), "r"(v[8 * i + 5]),
                               "r"(v[8 * i + 6]), "r"(v[8 * i + 7]) : "memory");
            }
          }
        }
      }
      TT_MARK(te2)
      TT_ADD(1, te1 - te0);
      TT_ADD(2, te2 - te1);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int col0 = 32 * (half + 2 * u);
        if (col0 < rows && ok) {
          uint32_t v[32];
          TT_MARK(te3)
          tmem_ld_32x32(taddr + 64 + col0, v);
          TT_MARK(te4)
          TT_ADD(3, te4 - te3);
          if (col0 + 32 <= rows) {
#ifdef TFGPC_TC_EPI_LDG
            // the 32 neighbor ids by uniform loads (one sector each, served by L1),
            // all independent of one another and of the reductions
            const int2* idp = neigh + m_first + col0;
            int p[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) p[i] = __ldg(&idp[i].x);
#pragma unroll
            for (int i = 0; i < 32; ++i)
              atomicAdd(dcol + (int64_t)p[i] * kC, __uint_as_float(v[i]));
#else
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int p = __shfl_sync(0xffffffffu, pts[u], i);
#ifndef TFGPC_WHATIF_NO_RED
              atomicAdd(dcol + (int64_t)p * kC, __uint_as_float(v[i]));
#else
              if (p == -12345) dcol[i] = __uint_as_float(v[i]);
#endif
            }
#endif
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int p = __shfl_sync(0xffffffffu, pts[u], i);
              if (col0 + i < rows) atomicAdd(dcol + (int64_t)p * kC, __uint_as_float(v[i]));
            }
          }
        }
      }
      TT_MARK(te5)
      TT_ADD(4, te5 - te2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[abuf]));
    }
#ifdef TFGPC_TC_TIMING
    if (warp == kEpiWarp0 && lane == 0) { TT_ADD(6, item); TT_STORE(4); }
#endif
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

bool basis_proj_grads_tc_supported(int K, int C) { return K == kK && C == kC; }

// Samples per group for a neighbor list of M pairs over ns samples: four while a
// group's pairs mostly fit one block of 128 rows, else three (whose second block,
// when there is one, is no emptier than any other remainder).
int basis_proj_grads_tc_group(int64_t ns, int64_t M) {
  return (ns > 0 && M * 4 <= ns * 112) ? 4 : 3;
}

template <int G>
static int launch_grads_tc(cudaStream_t st, int64_t ns, int64_t M, const float* basis,
                           const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                           const void* image, float* dbasis, float* dfeat, int* err_flag) {
  auto kern = basis_proj_grads_tc_kernel<G>;
  TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kSmemBytes));
  const int64_t groups = (ns + G - 1) / G;
  const int grid = (int)(groups < sm_count() ? groups : sm_count());
  ProfScope prof(st, "basis_proj_grads_tc");
  kern<<<grid, kThreads, kSmemBytes, st>>>(ns, M, basis, fs, (const int2*)neigh, ranges,
                                           (const uint8_t*)image, dbasis, dfeat,
                                           make_idesc(kRows, 16 * G, false, true),
                                           make_idesc(kRows, kC, false, false), err_flag);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

// `image`: the dX operand image written by gemm_bf16x3_grad_image for these ns
// samples in groups of `group` (ceil(ns / group) groups of 32 KB; the columns of
// the samples beyond ns in the last group must be finite).  dfeat must be zero
// on entry; dbasis is overwritten.
int basis_proj_grads_tc(cudaStream_t st, int group, int64_t ns, int64_t M, const float* basis,
                        const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                        const void* image, float* dbasis, float* dfeat, int* err_flag) {
  TFGPC_REQUIRE((uintptr_t)image % 16 == 0 && (uintptr_t)fs % 16 == 0 && (uintptr_t)basis % 16 == 0 &&
                (uintptr_t)dbasis % 32 == 0 && (uintptr_t)dfeat % 16 == 0,
                "tensor-core projection gradients expect 16-byte aligned buffers (dbasis: 32)");
  if (group == 4)
    return launch_grads_tc<4>(st, ns, M, basis, fs, neigh, ranges, image, dbasis, dfeat, err_flag);
  TFGPC_REQUIRE(group == 3, "tensor-core projection gradients work on groups of 3 or 4 samples");
  return launch_grads_tc<3>(st, ns, M, basis, fs, neigh, ranges, image, dbasis, dfeat, err_flag);
}

#ifdef TFGPC_TC_TIMING
// Debug builds only: copies the timing words of the last launch to the host.
extern "C" int tfgpc_debug_tc_timing(long long* out, int count) {
  return (int)cudaMemcpyFromSymbol(out, tt_array, sizeof(long long) * (size_t)count);
}
#endif

}  // namespace tfgpc
