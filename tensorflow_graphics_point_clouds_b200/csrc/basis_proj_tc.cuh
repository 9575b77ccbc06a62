// Pieces shared by the tcgen05 basis-projection kernels (forward and
// gradients): both work on groups of three or four consecutive samples, whose
// pairs are contiguous in the neighbor list.
#pragma once

#include "basis_proj.cuh"
#include "tc_common.cuh"

namespace tfgpc {
namespace bptc {

using namespace tc;

constexpr int kC = 128;        // channels
constexpr int kK = 16;         // basis functions
constexpr int kRows = 128;     // pairs per 128-row block of the gradient kernel

// Pair range of a group of G consecutive samples (G = 3 or 4) and the ends of
// all but its last sample.
struct Tile {
  int pa, e0, e1, e2, pe;
  __device__ __forceinline__ int blocks() const { return (pe - pa + kRows - 1) / kRows; }
  // (e2 == pe for groups of three, so the third comparison is then always false)
  __device__ __forceinline__ int local_sample(int m) const {
    return (m >= e0) + (m >= e1) + (m >= e2);
  }
};

template <int G>
__device__ __forceinline__ Tile load_tile(const int32_t* __restrict__ ranges, int64_t ns, int64_t g) {
  Tile t;
  const int64_t s0 = g * G;
  if (s0 >= ns) { t.pa = t.e0 = t.e1 = t.e2 = t.pe = 0; return t; }
  t.pa = s0 > 0 ? __ldg(ranges + s0 - 1) : 0;
  t.e0 = __ldg(ranges + s0);
  t.e1 = __ldg(ranges + min(s0 + 1, ns - 1));
  t.e2 = __ldg(ranges + min(s0 + 2, ns - 1));
  t.pe = G == 4 ? __ldg(ranges + min(s0 + 3, ns - 1)) : t.e2;
  return t;
}

// Walk over the blocks (tile, 128-row block) of this CTA, with the next tile's
// ranges already on their way.
template <int G>
struct ItemWalk {
  const int32_t* ranges;
  int64_t ns, groups, g;
  Tile t, tn;
  int b;
  bool valid;
  __device__ __forceinline__ void settle() {
    while (g < groups && b >= t.blocks()) {
      g += gridDim.x;
      t = tn;
      tn = load_tile<G>(ranges, ns, g + gridDim.x);
      b = 0;
    }
    valid = g < groups;
  }
  __device__ __forceinline__ void init(const int32_t* r, int64_t n, int64_t gr) {
    ranges = r; ns = n; groups = gr; g = blockIdx.x; b = 0;
    t = load_tile<G>(ranges, ns, g);
    tn = load_tile<G>(ranges, ns, g + gridDim.x);
    settle();
  }
  __device__ __forceinline__ void advance() { ++b; settle(); }
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


// Debug builds (-DTFGPC_TC_TIMING) record, per CTA and role, the clock cycles
// spent inside each barrier wait and in the role's whole loop, in a file-scope
// array `tt_array` [160 * 5 * 8] that the including file defines.
#ifdef TFGPC_TC_TIMING
#define TT_DECL long long tt_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long tt_start = clock64();
#define TT_WAIT(site, bar, parity)                                        \
  do {                                                                    \
    const long long tt0 = clock64();                                      \
    mbar_wait(bar, parity, abort_flag, err_flag);                         \
    tt_acc[site] += clock64() - tt0;                                      \
  } while (0)
#define TT_ADD(site, v) tt_acc[site] += (v)
#define TT_MARK(name) const long long name = clock64();
#define TT_STORE(role)                                                    \
  do {                                                                    \
    tt_acc[7] = clock64() - tt_start;                                     \
    for (int i = 0; i < 8; ++i) tt_array[(blockIdx.x * 5 + (role)) * 8 + i] = tt_acc[i]; \
  } while (0)
#else
#define TT_DECL
#define TT_WAIT(site, bar, parity) mbar_wait(bar, parity, abort_flag, err_flag)
#define TT_ADD(site, v)
#define TT_MARK(name)
#define TT_STORE(role)
#endif

// Instruction descriptor of tcgen05.mma kind::f16: D fp32, A and B bf16.
inline uint32_t make_idesc(int m, int n, bool a_mn, bool b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                       // D: f32
  d |= 1u << 7;                       // A: bf16
  d |= 1u << 10;                      // B: bf16
  d |= (a_mn ? 1u : 0u) << 15;        // A major: 0 = K, 1 = MN
  d |= (b_mn ? 1u : 0u) << 16;        // B major
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(m >> 4) << 24;
  return d;
}

}  // namespace bptc
}  // namespace tfgpc
