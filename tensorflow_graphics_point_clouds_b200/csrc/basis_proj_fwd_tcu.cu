// The basis projection on tcgen05 tensor cores, on the rows of a group plan
// (group_plan.cu): C = 128 channels, K = 16 basis functions, groups of four
// samples taken in the visiting order.
//
//   X[s, c, k] = sum over the pairs m of s:  feat[nbr(m), c] * basis[m, k]
// (BasisProj, basis_proj_kernels.cu.cc:30-127).  A row of the plan is a distinct
// neighbor j of the group; Bx[row, (q, k)] holds the basis row of the pair through
// which sample q of the group sees j (zero if it does not).  Then
//   Xcat[c, (q, k)] = sum over rows  F[row, c] * Bx[row, (q, k)]
// is one accumulator of 128 channels x 64 columns per group, with the rows as the
// reduction index: every feature row is gathered once per group (about half as
// often as once per pair) and no per-sample bookkeeping is left.
// Both operands are MN-major for the tensor core: F as [row][channel] and Bx as
// [row][(q, k)], 128-byte rows with the 16-byte chunks XOR-ed with row % 8, i.e.
// exactly what the copies of the gradient kernel (basis_proj_grads_tcu.cu) write.
// fp32 accuracy comes from the 3-pass bf16 split of both operands.
//
// The result is written as the bf16 (hi, mid) pair the weight GEMM consumes,
// row v = 4 g + q of X in the VISITING order (the GEMM scatters its output rows
// back to the sample order).
// Roles: warps 0-7 issue the copies, warp 8 issues the MMAs, warps 9-16 drain the
// accumulator (double buffered in tensor memory).  Every mbarrier wait is bounded.
#include "basis_proj_tc.cuh"
#include "group_plan.cuh"

namespace tfgpc {

using namespace tc;
using namespace bptc;

namespace {

#ifdef TFGPC_TC_TIMING
__device__ long long tt_array[160 * 5 * 8];
#endif

constexpr int kG = gp::kG;
constexpr int kProdWarps = 8;
constexpr int kMmaWarp = 8;
constexpr int kEpiWarp0 = 9;
constexpr int kThreads = 17 * 32;
#ifndef TFGPC_FWD_SLOTS
#define TFGPC_FWD_SLOTS 3
#endif
// Shared memory holds kSlots block-sized slots (two 64-channel feature units and
// one Bx stage each).  A block is at most kBlk rows: 96 instead of 128 leaves room
// for a third slot, i.e. lets the copy warps run two blocks ahead of the MMAs;
// groups of four samples have ~67 rows at 32 neighbors per point, larger ones take
// a second block.
constexpr int kSlots = TFGPC_FWD_SLOTS;
constexpr int kBlk = kSlots == 3 ? 96 : 128;   // rows per block (a multiple of 16)
constexpr int kSteps = kBlk / 16;
constexpr int kUnits = 2 * kSlots;     // 64-channel feature blocks; a block of rows takes two
constexpr uint32_t kPart = kBlk * 128; // one kBlk x 128-byte operand tile (hi or mid)
constexpr uint32_t kUnitBytes = 2 * kPart;
constexpr uint32_t kBxBytes = 2 * kPart;
constexpr uint32_t kTmemCols = 128;    // two accumulators of 64 columns
constexpr size_t kSmemBytes = (size_t)kUnits * kUnitBytes + kSlots * kBxBytes + 1024 + 256;

// One pair of barriers per block-sized slot (two ring units of features and one
// Bx stage): the MMA-issuing thread, which is what bounds this kernel, then waits
// once and commits once per block.
struct Barriers {
  uint64_t slot_full[kSlots], slot_empty[kSlots];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

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

__device__ __forceinline__ void st_global_256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]),
                 "r"(v[6]), "r"(v[7]) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
basis_proj_fwd_tcu_kernel(int64_t ns, int64_t groups, const int32_t* __restrict__ group_begin,
                          const int32_t* __restrict__ group_rows,
                          const int32_t* __restrict__ rows_id, const int4* __restrict__ rows_pair,
                          const __nv_bfloat16* __restrict__ basis_pair,
                          const __nv_bfloat16* __restrict__ fs, __nv_bfloat16* __restrict__ x_hi,
                          __nv_bfloat16* __restrict__ x_mid, uint32_t idesc, int* err_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* f_ring = smem;
  uint8_t* bx = f_ring + (size_t)kUnits * kUnitBytes;
  Barriers* bars = (Barriers*)(bx + kSlots * kBxBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(smem_u32(&bars->slot_full[i]), kProdWarps * 32);
      mbar_init(smem_u32(&bars->slot_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->acc_full[i]), 1);
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

  if (warp < kProdWarps) {
    // ------------------------------------------------------------- producers
    // warp w owns the rows r with r % 8 == w of every block (a group's rows fill
    // the first ceil(rows / 16) steps of 16 rows, so all eight warps get the same
    // share of them, however few rows the group has).  The plan entries of block
    // i+1 are fetched into registers while the copies of block i are issued;
    // every copy signals the consumer's barrier when it lands.
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
    uint32_t item = 0;
    UWalk walk;
    walk.init(group_begin, group_rows, groups);
    // plan entries of the next block: the ids of this lane's (up to) eight rows and
    // the pair indices of its two slots
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
    TT_DECL
    while (walk.valid) {
      TT_MARK(tp0)
      const int rows = rows_n;
      const int rows16 = (rows + 15) & ~15;     // the MMAs read whole steps of 16 rows
      int ids[kSteps], pr[kSteps];
#pragma unroll
      for (int it = 0; it < kSteps; ++it) { ids[it] = ids_n[it]; pr[it] = pr_n[it]; }
      walk.advance();
      if (walk.valid) prefetch();
      TT_MARK(tp1)
      TT_ADD(2, tp1 - tp0);
      // ---- F: two 64-channel blocks (units 2 item and 2 item + 1).  Rows between
      // the group's last row and the end of its last step are zero-filled (their
      // id was replaced by 0: it is only the address of a copy of zero bytes).
      const uint32_t stage = item % kSlots;
      TT_WAIT(0, smem_u32(&bars->slot_empty[stage]), ((item / kSlots) & 1) ^ 1);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        const uint32_t unit = 2 * stage + kb;
        const uint32_t base = smem_u32(f_ring + (size_t)unit * kUnitBytes) + f_dst_lane;
#pragma unroll
        for (int it = 0; it < kSteps; ++it) {
          if (16 * it < rows16)
            cp_async16_zfill(base + it * (16 * 128),
                             fs_lane + (int64_t)ids[it] * 2 * kC + kb * 64, 16 * it + frow < rows);
        }
      }
      TT_MARK(tp2)
      TT_ADD(3, tp2 - tp1);
      // ---- Bx: the basis rows of the plan's pairs, zeros where there is none
      {
        const uint32_t base = smem_u32(bx + (size_t)stage * kBxBytes) + bx_dst_lane;
#pragma unroll
        for (int it = 0; it < kSteps; ++it) {
          const int m = pr[it];
          if (16 * it < rows16)
            cp_async16_zfill(base + it * (16 * 128),
                             bp_lane + (int64_t)(m < 0 ? 0 : m) * (2 * kK), m >= 0);
        }
        // arrives on the slot's barrier once all of this thread's copies have landed
        asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];"
                     ::"r"(smem_u32(&bars->slot_full[stage])) : "memory");
      }
      ++item;
      TT_MARK(tp3)
      TT_ADD(4, tp3 - tp2);
      TT_ADD(6, 1);
    }
#ifdef TFGPC_TC_TIMING
    if (warp == 0 && lane == 0) TT_STORE(0);
#endif
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t item = 0, tile_i = 0;
      UTile next = load_utile(group_begin, group_rows, groups, blockIdx.x);
      TT_DECL
      for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
        const UTile t = next;
        next = load_utile(group_begin, group_rows, groups, g + gridDim.x);
        const int nb = t.blocks();
        if (nb == 0) continue;
        const uint32_t abuf = tile_i & 1;
        TT_WAIT(0, smem_u32(&bars->acc_empty[abuf]), ((tile_i >> 1) & 1) ^ 1);
        tc_fence_after();
        const uint32_t d = tmem_base + abuf * 64;
        uint32_t accumulate = 0;
        for (int b = 0; b < nb; ++b, ++item) {
          const uint32_t stage = item % kSlots;
          const uint32_t u0 = 2 * stage;                    // u0 + 1 is the next unit in memory
          TT_WAIT(1, smem_u32(&bars->slot_full[stage]), (item / kSlots) & 1);
          TT_MARK(tm0)
          fence_proxy_async();   // the copied rows were written through the generic proxy
          tc_fence_after();
          TT_MARK(tm1)
          TT_ADD(3, tm1 - tm0);
          const uint32_t f_hi = smem_u32(f_ring + (size_t)u0 * kUnitBytes), f_mid = f_hi + kPart;
          const uint32_t bx_hi = smem_u32(bx + (size_t)stage * kBxBytes), bx_mid = bx_hi + kPart;
          const int steps = (min(kBlk, t.rows - b * kBlk) + 15) >> 4;
          // both operands MN-major: 8 rows (reduction index) per 1024-byte atom, a
          // step of 16 rows is 2048 bytes (128 in the descriptor's 16-byte units);
          // the two 64-channel blocks of A lie one ring unit apart
          uint64_t da_hi = make_desc(f_hi, kUnitBytes, 1024);
          uint64_t da_mid = make_desc(f_mid, kUnitBytes, 1024);
          uint64_t db_hi = make_desc(bx_hi, 8192, 1024);
          uint64_t db_mid = make_desc(bx_mid, 8192, 1024);
          for (int kk = 0; kk < steps; ++kk) {
            umma_bf16(d, da_hi, db_mid, idesc, accumulate);
            umma_bf16(d, da_mid, db_hi, idesc, 1u);
            umma_bf16(d, da_hi, db_hi, idesc, 1u);
            accumulate = 1u;
            da_hi += 128; da_mid += 128; db_hi += 128; db_mid += 128;
          }
          TT_MARK(tm2)
          TT_ADD(4, tm2 - tm1);
          umma_commit(smem_u32(&bars->slot_empty[stage]));   // free once these MMAs have read it
          TT_MARK(tm3)
          TT_ADD(5, tm3 - tm2);
        }
        umma_commit(smem_u32(&bars->acc_full[abuf]));
        ++tile_i;
      }
      TT_ADD(6, item);
      TT_STORE(1);
    }
  } else {
    // -------------------------------------------------------------- epilogue
    // Two warps per quarter of the tensor-memory lanes (lane = channel).  Half h
    // takes samples 2 h and 2 h + 1 of the group: 16 columns each, i.e. this
    // channel's 16 basis functions, 32 contiguous bytes of the sample's row in
    // each of the hi and mid arrays; a warp writes 1 KB runs.
    const int quarter = warp & 3;
    const int half = (warp - kEpiWarp0) >> 2;
    const int c = quarter * 32 + lane;
    uint32_t tile_i = 0;
    UTile next = load_utile(group_begin, group_rows, groups, blockIdx.x);
    TT_DECL
    for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
      const UTile t = next;
      next = load_utile(group_begin, group_rows, groups, g + gridDim.x);
      if (t.blocks() == 0) {
        // no pair at all: the projection of these samples is zero
        const uint32_t zero[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int64_t v = g * kG + 2 * half + u;
          if (v < ns) {
            const int64_t off = v * (kC * kK) + c * kK;
            st_global_256(x_hi + off, zero); st_global_256(x_hi + off + 8, zero);
            st_global_256(x_mid + off, zero); st_global_256(x_mid + off + 8, zero);
          }
        }
        continue;
      }
      const uint32_t abuf = tile_i & 1;
      TT_WAIT(0, smem_u32(&bars->acc_full[abuf]), (tile_i >> 1) & 1);
      tc_fence_after();
      const bool ok = !*abort_flag;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + abuf * 64;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = 2 * half + u;
        const int64_t v = g * kG + q;
        uint32_t a[16];
        tmem_ld_x16(taddr + 16 * q, a);
        if (v < ns && ok) {
          uint32_t hv[8], mv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            split2_bf16(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1]), hv[i], mv[i]);
          const int64_t off = v * (kC * kK) + c * kK;
          st_global_256(x_hi + off, hv);
          st_global_256(x_mid + off, mv);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[abuf]));
      ++tile_i;
    }
#ifdef TFGPC_TC_TIMING
    if (warp == kEpiWarp0 && lane == 0) { TT_ADD(6, tile_i); TT_STORE(4); }
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

// X in the plan's visiting order as the bf16 (hi, mid) pair: x_hi, x_mid
// [ns, C * K], row v = the sample at position v of the order the plan was built
// with.  basis_pair [M, 2, 16] bf16, fs [n_in, 2, C] bf16.
int basis_proj_fwd_tcu(cudaStream_t st, int64_t ns, int64_t M, const void* plan,
                       const __nv_bfloat16* basis_pair, const __nv_bfloat16* fs,
                       __nv_bfloat16* x_hi, __nv_bfloat16* x_mid, int* err_flag) {
  TFGPC_REQUIRE((uintptr_t)fs % 16 == 0 && (uintptr_t)basis_pair % 16 == 0 &&
                (uintptr_t)x_hi % 32 == 0 && (uintptr_t)x_mid % 32 == 0 &&
                (uintptr_t)plan % 256 == 0,
                "grouped projection expects 16-byte aligned inputs and 32-byte aligned outputs");
  gp::PlanView v = gp::plan_view(const_cast<void*>(plan), ns, M);
  auto kern = basis_proj_fwd_tcu_kernel;
  TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kSmemBytes));
  const int grid = (int)(v.groups < sm_count() ? v.groups : sm_count());
  if (grid == 0) return TFGPC_OK;
  ProfScope prof(st, "basis_proj_fwd_tcu");
  kern<<<grid, kThreads, kSmemBytes, st>>>(ns, v.groups, v.group_begin, v.group_rows, v.rows_id,
                                           v.rows_pair, basis_pair, fs, x_hi, x_mid,
                                           make_idesc(kC, 16 * kG, true, true), err_flag);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

#ifdef TFGPC_TC_TIMING
// Debug builds only: copies the timing words of the last launch to the host.
extern "C" int tfgpc_debug_fwd_timing(long long* out, int count) {
  return (int)cudaMemcpyFromSymbol(out, tt_array, sizeof(long long) * (size_t)count);
}
#endif

}  // namespace tfgpc
