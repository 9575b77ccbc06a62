// Gradients of the basis projection on tcgen05 tensor cores, on the rows of a
// group plan (group_plan.cu): C = 128 channels, K = 16 basis functions, groups of
// four samples taken in the visiting order.
//
// For a pair m of sample s with neighbor j:
//   dbasis[m, k]  = sum_c feat[j, c] * dX[s, c, k]
//   dfeat[j, c]  += sum_k basis[m, k] * dX[s, c, k]
// The kernel in basis_proj_grads_tc.cu spends one tensor-core row, one gathered
// feature row and one 512-byte reduction per PAIR.  Here a row is a distinct
// neighbor of the group: the four samples of a group share about half of their
// neighbors, so the gathers, the reductions (which the L2's floating-point
// atomic units bound at about 4 TB/s) and the MMA rows all drop by that factor.
// With dXcat[c, (q, k)] the concatenated gradients of the group's samples q:
//   (1) D1[128 rows, 64] = F[rows, 128 c] * dXcat: the 16 columns of slot q are
//       the dbasis row of the pair through which sample q sees this neighbor;
//   (2) D2[128 c, rows] = dXcat * Bx^T, Bx[row, (q, k)] = basis row of that
//       pair (zero where sample q does not see the neighbor): column `row` is the
//       whole group's contribution to dfeat[j], added with ONE reduction.
// fp32 accuracy comes from the 3-pass bf16 split of both operands.
//
// Operands in shared memory (128-byte rows, 16-byte chunks XOR-ed with row % 8):
//   F      gathered from the pre-split features ([n, 2, C] bf16) by 16-byte
//          cp.async, one 64-channel block (hi 16 KB + mid 16 KB) per ring slot;
//   Bx     copied by 16-byte cp.async from the pre-split basis ([M, 2, K] bf16),
//          zero-filled where the plan holds no pair;
//   dXcat  the operand image the dX GEMM wrote for this group (one 32 KB bulk copy).
// Roles: warps 0-7 issue the copies (they compute nothing: every copy signals the
// consumer's barrier when it lands); warps 8 and 9 issue the MMAs of (1) and (2);
// warp 10 fetches dXcat; warps 11-18 drain the accumulators (three buffers in
// tensor memory).  Every mbarrier wait is bounded.
#include "basis_proj_tc.cuh"
#include "group_plan.cuh"

namespace tfgpc {

using namespace tc;
using namespace bptc;

namespace {

constexpr int kG = gp::kG;
constexpr int kProdWarps = 8;
constexpr int kMmaWarp = 8;
constexpr int kDxWarp = 10;
constexpr int kEpiWarp0 = 11;
constexpr int kThreads = 19 * 32;
// A block is at most kBlk = 96 rows of a group (groups of four samples have ~67
// rows at 32 neighbors per point; larger ones take a second block): D2 then needs
// 96 accumulator columns, and THREE accumulator buffers fit tensor memory, so the
// MMAs run two blocks ahead of the epilogue's reductions instead of one.  The
// MMAs of D1 still span 128 rows; the 32 beyond a block read whatever follows it
// in shared memory and their accumulator rows are never read.
constexpr int kBlk = 96;
constexpr int kSteps = kBlk / 16;
constexpr int kAccBufs = 3;
constexpr int kSlots = 4;
constexpr uint32_t kPart = kBlk * 128;     // one operand tile of a block (hi or mid)
constexpr uint32_t kSlotBytes = 2 * kPart;
constexpr uint32_t kBxBytes = 2 * kPart;
constexpr uint32_t kDxPart = 16384;        // hi (or mid) half of a group's dX image
constexpr uint32_t kDxBytes = 2 * kDxPart;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCols = 64 + kBlk;   // D1 (64 columns) + D2 (one column per row)
constexpr size_t kSmemBytes = (size_t)kSlots * kSlotBytes + 2 * kBxBytes + 2 * kDxBytes + 1024 + 256;

struct Barriers {
  uint64_t f_full[kSlots], f_empty[kSlots];
  uint64_t bx_full[2], bx_empty[2];
  uint64_t dx_full[2], dx_empty[2];
  uint64_t acc_full[kAccBufs], acc_empty[kAccBufs];
  uint32_t tmem_base;
  int abort_flag;
};

// Rows of one group: [ra, ra + rows).
struct UTile {
  int ra, rows;
  __device__ __forceinline__ int blocks() const { return (rows + kBlk - 1) / kBlk; }
};

__device__ __forceinline__ UTile load_utile(const int32_t* __restrict__ group_begin,
                                            const int32_t* __restrict__ group_rows, int64_t groups,
                                            int64_t g) {
  UTile t;
  if (g >= groups) { t.ra = 0; t.rows = 0; return t; }
  t.ra = __ldg(group_begin + g);
  t.rows = __ldg(group_rows + g);
  return t;
}

// Walk over the (group, block of kBlk rows) items of this CTA with the next group's
// descriptor already on its way.
struct UWalk {
  const int32_t *gb, *gr;
  int64_t groups, g;
  UTile t, tn;
  int b;
  bool valid;
  __device__ __forceinline__ void settle() {
    while (g < groups && b >= t.blocks()) {
      g += gridDim.x;
      t = tn;
      tn = load_utile(gb, gr, groups, g + gridDim.x);
      b = 0;
    }
    valid = g < groups;
  }
  __device__ __forceinline__ void init(const int32_t* begin, const int32_t* rows, int64_t n) {
    gb = begin; gr = rows; groups = n; g = blockIdx.x; b = 0;
    t = load_utile(gb, gr, groups, g);
    tn = load_utile(gb, gr, groups, g + gridDim.x);
    settle();
  }
  __device__ __forceinline__ void advance() { ++b; settle(); }
};

// 16-byte copy that writes zeros instead when `valid` is false.
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
               ::"r"(dst), "l"(src), "r"(valid ? 16u : 0u) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
basis_proj_grads_tcu_kernel(int64_t ns, int64_t M, int64_t groups,
                            const int32_t* __restrict__ group_begin,
                            const int32_t* __restrict__ group_rows,
                            const int32_t* __restrict__ rows_id, const int4* __restrict__ rows_pair,
                            const __nv_bfloat16* __restrict__ basis_pair,
                            const __nv_bfloat16* __restrict__ fs, const int32_t* __restrict__ ranges,
                            const uint8_t* __restrict__ image, float* __restrict__ dbasis,
                            float* __restrict__ dfeat, uint32_t idesc1, uint32_t idesc2,
                            int* err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* f_ring = smem;
  uint8_t* bx = f_ring + (size_t)kSlots * kSlotBytes;
  uint8_t* dx = bx + 2 * kBxBytes;
  Barriers* bars = (Barriers*)(dx + 2 * kDxBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(smem_u32(&bars->f_full[i]), kProdWarps * 32);
      mbar_init(smem_u32(&bars->f_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->bx_full[i]), kProdWarps * 32);
      mbar_init(smem_u32(&bars->bx_empty[i]), 1);
      mbar_init(smem_u32(&bars->dx_full[i]), 1);
      mbar_init(smem_u32(&bars->dx_empty[i]), 2);
    }
    for (int i = 0; i < kAccBufs; ++i) {
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
    // warp w owns the rows r with r % 8 == w of every block: a group's rows fill
    // the first rows of a block, so all eight warps get the same share of them,
    // however few the group has.  The plan entries of block i+1 are fetched into
    // registers while the copies of block i are issued.
    // F: in iteration `it` lanes 0-15 copy row 16 it + w, lanes 16-31 row
    // 16 it + 8 + w; lane -> (hi | mid part, 16-byte chunk j of the 64-channel block)
    const int l4 = lane >> 4, part = (lane >> 3) & 1, j = lane & 7;
    const int frow = 8 * l4 + warp;                 // this lane's row in iteration 0
    const __nv_bfloat16* const fs_lane = fs + part * kC + j * 8;
    // (row % 8 == warp: the swizzle term is a constant)
    const uint32_t f_dst_lane = part * kPart + frow * 128 + ((j ^ warp) << 4);
    // Bx: the same rows; lane -> (slot q, chunk c4 = part * 2 + half of the 16 functions)
    const int bq = (lane >> 2) & 3, c4 = lane & 3;
    const __nv_bfloat16* const bp_lane = basis_pair + (c4 >> 1) * kK + (c4 & 1) * 8;
    const uint32_t bx_dst_lane = (c4 >> 1) * kPart + frow * 128 + (((2 * bq + (c4 & 1)) ^ warp) << 4);
    uint32_t unit = 0, item = 0;
    UWalk walk;
    walk.init(group_begin, group_rows, groups);
    int rows_n = 0;
    int ids_n[kSteps], pr_n[kSteps];
    auto prefetch = [&]() {
      const int r0 = walk.t.ra + walk.b * kBlk;                    // first row of the block
      rows_n = min(kBlk, walk.t.rows - walk.b * kBlk);           // rows of the block that exist
#pragma unroll
      for (int it = 0; it < kSteps; ++it) {
        const bool have = 16 * it + frow < rows_n;
        ids_n[it] = have ? __ldg(rows_id + r0 + 16 * it + frow) : 0;
        pr_n[it] = have ? __ldg(reinterpret_cast<const int32_t*>(rows_pair + r0 + 16 * it + frow) + bq)
                        : -1;
      }
    };
    if (walk.valid) prefetch();
    while (walk.valid) {
      const int rows = rows_n;
      const int rows16 = (rows + 15) & ~15;   // rows the MMAs of the dfeat product read
      int ids[kSteps], pr[kSteps];
#pragma unroll
      for (int it = 0; it < kSteps; ++it) { ids[it] = ids_n[it]; pr[it] = pr_n[it]; }
      walk.advance();
      if (walk.valid) prefetch();
      // ---- F: two 64-channel blocks (rows beyond the group's are not read back)
#pragma unroll
      for (int kb = 0; kb < 2; ++kb, ++unit) {
        const uint32_t slot = unit % kSlots;
        mbar_wait(smem_u32(&bars->f_empty[slot]), ((unit / kSlots) & 1) ^ 1, abort_flag, err_flag);
        const uint32_t base = smem_u32(f_ring + (size_t)slot * kSlotBytes) + f_dst_lane;
#pragma unroll
        for (int it = 0; it < kSteps; ++it) {
          if (16 * it + frow < rows)
            cp_async16(base + it * (16 * 128), fs_lane + (int64_t)ids[it] * 2 * kC + kb * 64);
        }
        // arrives on the slot's barrier once this thread's copies have landed
        asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];"
                     ::"r"(smem_u32(&bars->f_full[slot])) : "memory");
      }
      // ---- Bx: the basis rows of the plan's pairs, zeros where there is none
      {
        const uint32_t stage = item & 1;
        mbar_wait(smem_u32(&bars->bx_empty[stage]), ((item >> 1) & 1) ^ 1, abort_flag, err_flag);
        const uint32_t base = smem_u32(bx + (size_t)stage * kBxBytes) + bx_dst_lane;
#pragma unroll
        for (int it = 0; it < kSteps; ++it) {
          const int m = pr[it];
          if (16 * it < rows16)
            cp_async16_zfill(base + it * (16 * 128),
                             bp_lane + (int64_t)(m < 0 ? 0 : m) * (2 * kK), m >= 0);
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];"
                     ::"r"(smem_u32(&bars->bx_full[stage])) : "memory");
      }
      ++item;
    }
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ----------------------------------------------------------- MMA issuers
    const bool first = warp == kMmaWarp;
    if (lane == 0) {
      uint32_t unit = 0, item = 0, tile_i = 0;
      UTile next = load_utile(group_begin, group_rows, groups, blockIdx.x);
      for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
        const UTile t = next;
        next = load_utile(group_begin, group_rows, groups, g + gridDim.x);
        const int nb = t.blocks();
        if (nb == 0) continue;
        const uint32_t dbuf = tile_i & 1;
        mbar_wait(smem_u32(&bars->dx_full[dbuf]), (tile_i >> 1) & 1, abort_flag, err_flag);
        const uint32_t dx_hi = smem_u32(dx + (size_t)dbuf * kDxBytes), dx_mid = dx_hi + kDxPart;
        for (int b = 0; b < nb; ++b, ++item) {
          const uint32_t abuf = item % kAccBufs;
          mbar_wait(smem_u32(&bars->acc_empty[abuf]), ((item / kAccBufs) & 1) ^ 1, abort_flag, err_flag);
          tc_fence_after();
          const uint32_t d1 = tmem_base + abuf * kAccCols, d2 = d1 + 64;
          if (first) {
            // (1) D1 = F * dXcat: reduction over the 128 channels, two ring slots
            uint32_t accumulate = 0;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb, ++unit) {
              const uint32_t slot = unit % kSlots;
              mbar_wait(smem_u32(&bars->f_full[slot]), (unit / kSlots) & 1, abort_flag, err_flag);
              fence_proxy_async();   // the copied rows were written through the generic proxy
              tc_fence_after();
              const uint32_t f_hi = smem_u32(f_ring + (size_t)slot * kSlotBytes), f_mid = f_hi + kPart;
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
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
            // (2) D2 = dXcat * Bx^T: reduction over the 64 (slot, k) columns.  Only
            // the columns of rows that exist are computed (N in steps of 16): the
            // tensor core reads that much less of Bx from shared memory.
            const int rows_b = min(kBlk, t.rows - b * kBlk);
            const uint32_t n16 = (uint32_t)((rows_b + 15) & ~15);
            const uint32_t idesc2n = (idesc2 & ~(0x3Fu << 17)) | ((n16 >> 3) << 17);
            const uint32_t stage = item & 1;
            mbar_wait(smem_u32(&bars->bx_full[stage]), (item >> 1) & 1, abort_flag, err_flag);
            fence_proxy_async();
            tc_fence_after();
            const uint32_t bx_hi = smem_u32(bx + (size_t)stage * kBxBytes), bx_mid = bx_hi + kPart;
            uint32_t accumulate = 0;
#pragma unroll
            for (int kk = 0; kk < kG; ++kk) {
              const uint64_t da_hi = make_desc(dx_hi + kk * 32, 16, 1024);
              const uint64_t da_mid = make_desc(dx_mid + kk * 32, 16, 1024);
              const uint64_t db_hi = make_desc(bx_hi + kk * 32, 16, 1024);
              const uint64_t db_mid = make_desc(bx_mid + kk * 32, 16, 1024);
              umma_bf16(d2, da_hi, db_mid, idesc2n, accumulate);
              umma_bf16(d2, da_mid, db_hi, idesc2n, 1u);
              umma_bf16(d2, da_hi, db_hi, idesc2n, 1u);
              accumulate = 1u;
            }
            umma_commit(smem_u32(&bars->bx_empty[stage]));
          }
          umma_commit(smem_u32(&bars->acc_full[abuf]));
        }
        umma_commit(smem_u32(&bars->dx_empty[dbuf]));
        ++tile_i;
      }
    }
  } else if (warp == kDxWarp) {
    // ------------------------------------------------------- dXcat loader
    if (lane == 0) {
      uint32_t tile_i = 0;
      UTile next = load_utile(group_begin, group_rows, groups, blockIdx.x);
      for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
        const UTile t = next;
        next = load_utile(group_begin, group_rows, groups, g + gridDim.x);
        if (t.blocks() == 0) continue;
        const uint32_t dbuf = tile_i & 1;
        mbar_wait(smem_u32(&bars->dx_empty[dbuf]), ((tile_i >> 1) & 1) ^ 1, abort_flag, err_flag);
        const uint32_t full = smem_u32(&bars->dx_full[dbuf]);
        mbar_expect_tx(full, kDxBytes);
        bulk_g2s(smem_u32(dx + (size_t)dbuf * kDxBytes), image + g * (int64_t)kDxBytes, kDxBytes, full);
        ++tile_i;
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue
    // Two warps per quarter of the tensor-memory lanes.  D1 (lanes = rows): warp
    // half 1 stores, for every slot q in which the row has a pair, the 16 columns
    // of q as that pair's dbasis row.  D2 (lanes = channels, columns = rows): half
    // h takes the 32-row column blocks h and h + 2; for every row the warp adds
    // its 32 channels to the neighbor's gradient row, 128 contiguous bytes per
    // instruction.  (D1 goes to half 1 because a group of ~67 rows gives half 0
    // the rows 0-31 and 64-66 and half 1 only the rows 32-63: the reductions, which
    // share the LSU with the copy warps, are what the accumulators wait for.)
    const int quarter = warp & 3;
    const int half = (warp - kEpiWarp0) >> 2;
    const int r = quarter * 32 + lane;        // this thread's accumulator row
    float* const dcol = dfeat + r;            // channel r of every gradient row
    UWalk walk;
    walk.init(group_begin, group_rows, groups);
    uint32_t item = 0;
    for (; walk.valid; walk.advance(), ++item) {
      const int r_first = walk.t.ra + walk.b * kBlk;
      const int rows = min(kBlk, walk.t.rows - walk.b * kBlk);   // rows in this block
      int pts[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = 32 * (half + 2 * u) + lane;
        pts[u] = c < rows ? __ldg(rows_id + r_first + c) : 0;
      }
      int4 pr = make_int4(-1, -1, -1, -1);
      if (half == 1 && r < rows) pr = __ldg(rows_pair + r_first + r);
      const uint32_t abuf = item % kAccBufs;
      mbar_wait(smem_u32(&bars->acc_full[abuf]), (item / kAccBufs) & 1, abort_flag, err_flag);
      tc_fence_after();
      const bool ok = !*abort_flag;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + abuf * kAccCols;
      if (half == 1) {
        const int prq[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
        for (int q = 0; q < kG; ++q) {
          const bool mine = ok && prq[q] >= 0;
          if (__any_sync(0xffffffffu, mine)) {
            uint32_t v[16];
            tmem_ld_x16(taddr + 16 * q, v);
            if (mine) {
              float* dst = dbasis + (int64_t)prq[q] * kK;
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
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int col0 = 32 * (half + 2 * u);
        if (col0 < rows && ok) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + 64 + col0, v);
          if (col0 + 32 <= rows) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int p = __shfl_sync(0xffffffffu, pts[u], i);
              atomicAdd(dcol + (int64_t)p * kC, __uint_as_float(v[i]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int p = __shfl_sync(0xffffffffu, pts[u], i);
              if (col0 + i < rows) atomicAdd(dcol + (int64_t)p * kC, __uint_as_float(v[i]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[abuf]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// `plan`: built by tfgpc_mcconv_group_plan for these ns samples and M pairs.
// `image`: the dX operand image written by the dX GEMM in groups of four
// samples taken in the plan's visiting order (ceil(ns / 4) groups of 32 KB; the
// columns of samples beyond ns in the last group must be finite).  basis_pair:
// [M, 2, 16] bf16 (hi row, mid row).  dfeat must be zero on entry; dbasis is
// overwritten.
int basis_proj_grads_tcu(cudaStream_t st, int64_t ns, int64_t M, const void* plan,
                         const __nv_bfloat16* basis_pair, const __nv_bfloat16* fs,
                         const int32_t* ranges, const void* image, float* dbasis, float* dfeat,
                         int* err_flag) {
  TFGPC_REQUIRE((uintptr_t)image % 16 == 0 && (uintptr_t)fs % 16 == 0 &&
                (uintptr_t)basis_pair % 16 == 0 && (uintptr_t)dbasis % 32 == 0 &&
                (uintptr_t)dfeat % 16 == 0 && (uintptr_t)plan % 256 == 0,
                "grouped projection gradients expect 16-byte aligned buffers (dbasis: 32)");
  gp::PlanView v = gp::plan_view(const_cast<void*>(plan), ns, M);
  auto kern = basis_proj_grads_tcu_kernel;
  TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kSmemBytes));
  const int grid = (int)(v.groups < sm_count() ? v.groups : sm_count());
  if (grid == 0) return TFGPC_OK;
  ProfScope prof(st, "basis_proj_grads_tcu");
  kern<<<grid, kThreads, kSmemBytes, st>>>(ns, M, v.groups, v.group_begin, v.group_rows, v.rows_id,
                                           v.rows_pair, basis_pair, fs, ranges,
                                           (const uint8_t*)image, dbasis, dfeat,
                                           make_idesc(128, 16 * kG, false, true),
                                           make_idesc(kC, 128, false, false), err_flag);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

}  // namespace tfgpc
