// tcgen05 / TMEM / TMA GEMM with 3-pass bf16 operand splitting (see
// gemm_sm100.cuh).  Persistent kernel, one CTA per SM, warp-specialised:
//   warp 0     TMA producer: streams 128 x 64 tiles of A (hi, mid) and
//              BN x 64 tiles of B (hi, mid) into a shared-memory ring;
//   warp 1     allocates tensor memory and issues the tcgen05.mma instructions
//              (one elected lane); completion is tracked with tcgen05.commit
//              on mbarriers, which also hands ring slots back to the producer;
//   warps 2-5  epilogue: tcgen05.ld the 128 x BN fp32 accumulator out of
//              tensor memory, stage it in swizzled 32 x 32 boxes and hand those
//              to TMA stores, while the MMA warp already works on the next tile
//              in the second accumulator buffer.
// Every wait is bounded: after about a second without progress the kernel sets
// the caller's error flag, stops waiting and drains, so it always terminates
// and frees its tensor memory.
#include <cuda.h>

#include "gemm_sm100.cuh"
#include "basis_proj.cuh"
#include "tc_common.cuh"

namespace tfgpc {

namespace {

constexpr int kBM = 128;           // rows of C per tile (TMEM lanes)
constexpr int kBNMax = 256;        // columns of C per tile (TMEM columns per buffer)
constexpr int kBK = 64;            // reduction elements per ring slot: 128 bytes of bf16
constexpr int kStages = 2;
constexpr int kUmmaK = 16;         // reduction elements per tcgen05.mma (kind::f16)
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;     // two accumulator buffers of 256 columns
constexpr uint32_t kABytes = kBM * kBK * 2;        // one A tile (hi or mid)
constexpr uint32_t kBBytes = kBNMax * kBK * 2;     // one B tile (hi or mid)
constexpr uint32_t kStageBytes = 2 * kABytes + 2 * kBBytes;
constexpr uint32_t kOutBoxBytes = 32 * 32 * 4;     // one 32 x 32 fp32 box of the epilogue
constexpr uint32_t kOutStageBytes = 4 * 2 * kOutBoxBytes;  // 4 epilogue warps, double buffered
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + kOutStageBytes +
                              1024 /*alignment*/ + 256 /*barriers*/;

using namespace tc;

// One 32-byte store (sm_100: 256-bit vector access to global memory).
__device__ __forceinline__ void st_global_256(void* p, const uint4& lo, const uint4& hi) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y),
                 "r"(hi.z), "r"(hi.w) : "memory");
}

// Writes 2 channels x 16 basis functions (v[0..31]) of sample `row` into the
// operand image of the tensor-core gradient kernel (basis_proj_grads_tc.cu).
// The row's two chunks (k 0-7, k 8-15) of a channel share one 32-byte sector,
// in swapped order when the channel is odd: one 256-bit store per part, and the
// lanes of neighboring samples fill whole 128-byte lines.
__device__ __forceinline__ void store_image_row(uint8_t* image, int channels, int group_size,
                                                int64_t row, int ch0, const uint32_t* v) {
  const int64_t part = (int64_t)channels * 128;   // bytes of the hi (or mid) rows of a group
  const int64_t gi = row / group_size;
  uint8_t* group = image + gi * (2 * part);
  const int sl = (int)(row - gi * group_size);
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int ch = ch0 + u;
    uint4 hv[2], mv[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int b = 16 * u + 8 * h;
      split2_bf16(__uint_as_float(v[b]), __uint_as_float(v[b + 1]), hv[h].x, mv[h].x);
      split2_bf16(__uint_as_float(v[b + 2]), __uint_as_float(v[b + 3]), hv[h].y, mv[h].y);
      split2_bf16(__uint_as_float(v[b + 4]), __uint_as_float(v[b + 5]), hv[h].z, mv[h].z);
      split2_bf16(__uint_as_float(v[b + 6]), __uint_as_float(v[b + 7]), hv[h].w, mv[h].w);
    }
    const bool swap = (ch & 1) != 0;
    const uint4 h_lo = swap ? hv[1] : hv[0], h_hi = swap ? hv[0] : hv[1];
    const uint4 m_lo = swap ? mv[1] : mv[0], m_hi = swap ? mv[0] : mv[1];
    uint8_t* dst = group + (int64_t)ch * 128 + (((2 * sl) ^ (ch & 6)) << 4);
    st_global_256(dst, h_lo, h_hi);
    st_global_256(dst + part, m_lo, m_hi);
  }
}

struct TileSchedule {
  int m_tiles, n_tiles, k_splits;
  int k_blocks;         // ring slots over the whole reduction
  int k_blocks_per_split;
  int add_slices;       // 1: every slice of the reduction is added into the one output
};

struct Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// OUT = 0: C as fp32 through TMA stores.  OUT = 1: C is the gradient of a
// [rows, channels, 16] projection and is written as the bf16 hi/mid operand
// image the tensor-core gradient kernel loads with one bulk copy per group of
// four rows (basis_proj_grads_tc.cu describes the layout).  OUT = 2: the map of C
// describes C^T ([N, M] row-major): boxes are transposed on their way through
// shared memory, for products whose natural left operand is the small matrix.
// OUT = 4: like 2, but row j of C^T goes to row row_order[j] of the output
// (`image` is then the fp32 output, image_channels its row length): the rows of a
// product computed in another sequence than the caller's are put back in place.
template <bool A_MN, bool B_MN, int OUT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16x3_kernel(const __grid_constant__ CUtensorMap tm_a_hi,
                   const __grid_constant__ CUtensorMap tm_a_mid,
                   const __grid_constant__ CUtensorMap tm_b_hi,
                   const __grid_constant__ CUtensorMap tm_b_mid,
                   const __grid_constant__ CUtensorMap tm_c, int64_t m_total, int64_t n_total,
                   int bn, uint32_t idesc, TileSchedule sch, int* err_flag, uint8_t* image,
                   int image_channels, int image_group, const int32_t* __restrict__ row_order) {
  extern __shared__ uint8_t smem_raw[];
  // the swizzled tiles need 1024-byte alignment
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* out_stage = smem + (size_t)kStages * kStageBytes;  // 1024-byte aligned
  Barriers* bars = (Barriers*)(out_stage + kOutStageBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = sch.m_tiles * sch.n_tiles * sch.k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars->acc_full[b]), 1);
      mbar_init(smem_u32(&bars->acc_empty[b]), 4);
    }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;

  // tile -> (m, n, split); m fastest so that CTAs running together share B/k-slices
  auto decode = [&](int t, int& m, int& n, int& sp) {
    m = t % sch.m_tiles;
    int r = t / sch.m_tiles;
    n = r % sch.n_tiles;
    sp = r / sch.n_tiles;
  };
  const uint32_t b_tile_bytes = (uint32_t)bn * kBK * 2;

  if (warp == 0) {
    // ---------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        int m, n, sp;
        decode(t, m, n, sp);
        const int kb0 = sp * sch.k_blocks_per_split;
        const int kb1 = min(kb0 + sch.k_blocks_per_split, sch.k_blocks);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1, abort_flag, err_flag);
          const uint32_t full = smem_u32(&bars->full[s]);
          mbar_expect_tx(full, 2 * kABytes + 2 * b_tile_bytes);
          uint8_t* st = smem + (size_t)s * kStageBytes;
          const uint32_t a_hi = smem_u32(st), a_mid = a_hi + kABytes;
          const uint32_t b_hi = a_mid + kABytes, b_mid = b_hi + kBBytes;
          if (!A_MN) {
            tma_load_2d(a_hi, &tm_a_hi, kb * kBK, m * kBM, full);
            tma_load_2d(a_mid, &tm_a_mid, kb * kBK, m * kBM, full);
          } else {
            // two boxes of 64 (M) x 64 (K rows): 8 KB each
            for (int j = 0; j < kBM / 64; ++j) {
              tma_load_2d(a_hi + j * 8192, &tm_a_hi, m * kBM + j * 64, kb * kBK, full);
              tma_load_2d(a_mid + j * 8192, &tm_a_mid, m * kBM + j * 64, kb * kBK, full);
            }
          }
          if (!B_MN) {
            tma_load_2d(b_hi, &tm_b_hi, kb * kBK, n * bn, full);
            tma_load_2d(b_mid, &tm_b_mid, kb * kBK, n * bn, full);
          } else {
            for (int j = 0; j < bn / 64; ++j) {
              tma_load_2d(b_hi + j * 8192, &tm_b_hi, n * bn + j * 64, kb * kBK, full);
              tma_load_2d(b_mid + j * 8192, &tm_b_mid, n * bn + j * 64, kb * kBK, full);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0;
      int tile_iter = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_iter) {
        int m, n, sp;
        decode(t, m, n, sp);
        const int kb0 = sp * sch.k_blocks_per_split;
        const int kb1 = min(kb0 + sch.k_blocks_per_split, sch.k_blocks);
        const int buf = tile_iter & 1;
        mbar_wait(smem_u32(&bars->acc_empty[buf]), ((tile_iter >> 1) & 1) ^ 1, abort_flag, err_flag);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * kBNMax;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag, err_flag);
          tc_fence_after();
          uint8_t* st = smem + (size_t)s * kStageBytes;
          const uint32_t a_hi = smem_u32(st), a_mid = a_hi + kABytes;
          const uint32_t b_hi = a_mid + kABytes, b_mid = b_hi + kBBytes;
          // K-major: rows of 128 bytes, 8-row swizzle atoms 1024 bytes apart;
          // one UMMA_K step is 32 bytes inside the row.
          // MN-major: 64 (MN) x 8 (K) atoms of 1024 bytes; atoms along K are
          // 1024 bytes apart (stride offset), blocks of 64 along MN are 8192
          // bytes apart (leading offset); one UMMA_K step is 16 K rows.
          const uint32_t a_step = A_MN ? 16 * 128 : 32;
          const uint32_t b_step = B_MN ? 16 * 128 : 32;
          const uint32_t a_lbo = A_MN ? 8192 : 16, b_lbo = B_MN ? 8192 : 16;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t da_hi = make_desc(a_hi + kk * a_step, a_lbo, 1024);
            const uint64_t da_mid = make_desc(a_mid + kk * a_step, a_lbo, 1024);
            const uint64_t db_hi = make_desc(b_hi + kk * b_step, b_lbo, 1024);
            const uint64_t db_mid = make_desc(b_mid + kk * b_step, b_lbo, 1024);
            umma_bf16(d_tmem, da_hi, db_mid, idesc, accumulate);
            umma_bf16(d_tmem, da_mid, db_hi, idesc, 1u);
            umma_bf16(d_tmem, da_hi, db_hi, idesc, 1u);
            accumulate = 1u;
          }
          umma_commit(smem_u32(&bars->empty[s]));  // slot free once these MMAs have read it
        }
        umma_commit(smem_u32(&bars->acc_full[buf]));
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue
    // Each warp drains its 32 accumulator rows 32 columns at a time: tcgen05.ld
    // to registers, a 128-byte-swizzled 32 x 32 box in shared memory (lane =
    // row, so the swizzle makes the 16-byte writes of a quarter warp hit
    // distinct banks), then one TMA store per box, double buffered.  TMA clips
    // the rows and columns beyond the edge of C.
    const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter ...
    uint8_t* my_stage = out_stage + (size_t)quarter * 2 * kOutBoxBytes;
    uint32_t box_iter = 0;
    int tile_iter = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_iter) {
      int m, n, sp;
      decode(t, m, n, sp);
      const int buf = tile_iter & 1;
      mbar_wait(smem_u32(&bars->acc_full[buf]), (tile_iter >> 1) & 1, abort_flag, err_flag);
      tc_fence_after();
      const int row0 = m * kBM + quarter * 32;
      for (int c0 = 0; c0 < bn; c0 += 32, ++box_iter) {
        // Boxes beyond the last column or row hold nothing to store.  They must
        // not touch the staging buffers either: the wait below only covers the
        // buffer's previous store if every box written here also issues one.
        if ((int64_t)n * bn + c0 >= n_total || row0 >= m_total) break;
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                               (uint32_t)(buf * kBNMax + c0);
        tmem_ld_32x32(taddr, r);
        if (OUT == 1) {
          // this thread holds 2 channels x 16 basis functions of row `row`
          const int64_t row = (int64_t)row0 + lane;
          if (row < m_total && !*abort_flag)
            store_image_row(image, image_channels, image_group, row, (n * bn + c0) / 16, r);
          continue;
        }
        if (OUT == 4) {
          // as OUT == 3 below: after the transposition this thread holds columns
          // row0 .. row0 + 31 of C^T's row n * bn + c0 + lane, 128 contiguous bytes
          uint8_t* box = my_stage;
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            *reinterpret_cast<uint32_t*>(box + i * 128 + (((lane >> 2) ^ (i & 7)) << 4) +
                                         (lane & 3) * 4) = r[i];
          __syncwarp();
          const int64_t j = (int64_t)n * bn + c0 + lane;
          if (j < n_total && !*abort_flag) {
            float* dst = reinterpret_cast<float*>(image) +
                         (int64_t)__ldg(row_order + j) * image_channels + row0;
            if (row0 + 32 <= m_total) {
#pragma unroll
              for (int q = 0; q < 8; q += 2)   // whole 32-byte sectors per store
                st_global_256(dst + 4 * q,
                              *reinterpret_cast<const uint4*>(box + lane * 128 + ((q ^ (lane & 7)) << 4)),
                              *reinterpret_cast<const uint4*>(box + lane * 128 + (((q + 1) ^ (lane & 7)) << 4)));
            } else {
              for (int e = 0; row0 + e < m_total; ++e)
                dst[e] = *reinterpret_cast<const float*>(box + lane * 128 +
                                                         (((e >> 2) ^ (lane & 7)) << 4) + (e & 3) * 4);
            }
          }
          continue;
        }
        if (OUT == 3) {
          // C^T tile: this thread holds 32 rows (samples c0 .. c0+31 of the tile)
          // of column row0 + lane.  Transposed through the warp's staging box, it
          // holds 32 consecutive columns (2 channels x 16) of sample c0 + lane.
          uint8_t* box = my_stage;
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            *reinterpret_cast<uint32_t*>(box + i * 128 + (((lane >> 2) ^ (i & 7)) << 4) +
                                         (lane & 3) * 4) = r[i];
          __syncwarp();
          uint32_t v[32];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint4 t4 = *reinterpret_cast<const uint4*>(box + lane * 128 + ((q ^ (lane & 7)) << 4));
            v[4 * q] = t4.x; v[4 * q + 1] = t4.y; v[4 * q + 2] = t4.z; v[4 * q + 3] = t4.w;
          }
          const int64_t sample = (int64_t)n * bn + c0 + lane;
          if (sample < n_total && !*abort_flag)
            store_image_row(image, image_channels, image_group, sample, row0 / 16, v);
          continue;
        }
        uint8_t* box = my_stage + (size_t)(box_iter & 1) * kOutBoxBytes;
        if (lane == 0) tma_store_wait_read<1>();  // the store that last used this box has read it
        __syncwarp();
        if (OUT == 2) {
          // box row i = column c0 + i of the tile, box column = this lane's row:
          // a warp store fills one (swizzled) 128-byte row, no bank conflicts
#pragma unroll
          for (int i = 0; i < 32; ++i)
            *reinterpret_cast<uint32_t*>(box + i * 128 + ((((lane >> 2) ^ (i & 7))) << 4) +
                                         (lane & 3) * 4) = r[i];
        } else {
          float4* rowp = reinterpret_cast<float4*>(box + lane * 128);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            rowp[q ^ (lane & 7)] =
                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                            __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        }
        fence_proxy_async();
        __syncwarp();
        const int col0 = n * bn + c0;
        if (lane == 0 && row0 < m_total && col0 < n_total && !*abort_flag) {
          if (OUT == 2)
            tma_store_3d(&tm_c, smem_u32(box), row0, col0, sp);
          else if (sch.add_slices)
            tma_reduce_add_3d(&tm_c, smem_u32(box), col0, row0, 0);
          else
            tma_store_3d(&tm_c, smem_u32(box), col0, row0, sp);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[buf]));
    }
    if (lane == 0) tma_store_wait_read<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ---------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D bf16 tensor map: dim0 (contiguous) x dim1 rows, 128-byte swizzle, zero fill.
int make_map(CUtensorMap* map, const __nv_bfloat16* base, int64_t dim0, int64_t dim1, int64_t ld,
             int box0, int box1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TFGPC_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((uintptr_t)base % 16 != 0 || (ld * 2) % 16 != 0)
    return fail(TFGPC_EINVAL, "tensor-core GEMM operands need 16-byte aligned rows (ld %lld)",
                (long long)ld);
  cuuint64_t dims[2] = {(cuuint64_t)dim0, (cuuint64_t)dim1};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box0, (cuuint32_t)box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TFGPC_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return TFGPC_OK;
}

// 3-D fp32 tensor map of C: (columns, rows, k slices), boxes of 32 x 32 x 1 with
// the 128-byte swizzle the epilogue writes its staging boxes in.
int make_map_c(CUtensorMap* map, float* base, int64_t n, int64_t m, int64_t slices, int64_t ldc,
               int64_t split_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TFGPC_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((uintptr_t)base % 16 != 0 || ldc % 4 != 0 || split_stride % 4 != 0)
    return fail(TFGPC_EINVAL, "tensor-core GEMM output needs 16-byte aligned rows (ld %lld)",
                (long long)ldc);
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)slices};
  cuuint64_t strides[2] = {(cuuint64_t)ldc * 4,
                           (cuuint64_t)(slices > 1 ? split_stride : m * ldc) * 4};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TFGPC_ECUDA, "cuTensorMapEncodeTiled (C) failed with %d", (int)r);
  return TFGPC_OK;
}

// Instruction descriptor of tcgen05.mma kind::f16: D fp32, A and B bf16.
uint32_t make_idesc(int m, int n, bool a_mn, bool b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                       // D format: f32
  d |= 1u << 7;                       // A format: bf16
  d |= 1u << 10;                      // B format: bf16
  d |= (a_mn ? 1u : 0u) << 15;        // A major: 0 = K, 1 = MN
  d |= (b_mn ? 1u : 0u) << 16;        // B major
  d |= (uint32_t)(n >> 3) << 17;      // N / 8
  d |= (uint32_t)(m >> 4) << 24;      // M / 16
  return d;
}

template <bool A_MN, bool B_MN, int OUT = 0>
int launch(cudaStream_t st, const CUtensorMap* maps, int64_t M, int64_t N, int bn,
           TileSchedule sch, int* err_flag, uint8_t* image = nullptr, int image_channels = 0,
           int image_group = 4, const int32_t* row_order = nullptr) {
  auto kern = gemm_bf16x3_kernel<A_MN, B_MN, OUT>;
  TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kSmemBytes));
  const int tiles = sch.m_tiles * sch.n_tiles * sch.k_splits;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  ProfScope prof(st, OUT == 4 ? "gemm_bf16x3_mn_k_scatter" : OUT == 3 ? "gemm_bf16x3_mn_k_image"
                     : OUT == 2 ? "gemm_bf16x3_mn_k_t"
                     : OUT == 1 ? (B_MN ? "gemm_bf16x3_k_mn_image" : "gemm_bf16x3_k_k_image")
                              : A_MN ? (B_MN ? "gemm_bf16x3_mn_mn" : "gemm_bf16x3_mn_k")
                                     : (B_MN ? "gemm_bf16x3_k_mn" : "gemm_bf16x3_k_k"));
  kern<<<grid, kThreads, kSmemBytes, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], M, N, bn,
                                           make_idesc(kBM, bn, A_MN, B_MN), sch, err_flag, image,
                                           image_channels, image_group, row_order);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

// One warp that waits, through the same bounded wait as every role of the
// GEMM, for a barrier phase that nothing ever completes: the wait gives up after
// `limit_ns`, records that in the status word and the kernel returns.
__global__ void wait_probe_kernel(int* err_flag, unsigned long long limit_ns, int* returned) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, err_flag, limit_ns);
    *returned = 1;
  }
}

__global__ void split_kernel(const float* __restrict__ x, int64_t n, __nv_bfloat16* __restrict__ hi,
                             __nv_bfloat16* __restrict__ mid) {
  int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n && ((uintptr_t)x % 16 == 0) && ((uintptr_t)hi % 8 == 0) && ((uintptr_t)mid % 8 == 0)) {
    float4 v = __ldg(reinterpret_cast<const float4*>(x + i));
    __nv_bfloat16 h[4], l[4];
    split_bf16(v.x, h[0], l[0]); split_bf16(v.y, h[1], l[1]);
    split_bf16(v.z, h[2], l[2]); split_bf16(v.w, h[3], l[3]);
    *reinterpret_cast<uint2*>(hi + i) = *reinterpret_cast<uint2*>(h);
    *reinterpret_cast<uint2*>(mid + i) = *reinterpret_cast<uint2*>(l);
  } else {
    for (int64_t j = i; j < n && j < i + 4; ++j) split_bf16(__ldg(x + j), hi[j], mid[j]);
  }
}

// Row v of the output is the split of row order[v] of x (cols a multiple of 4,
// 16-byte aligned rows).
__global__ void split_rows_gather_kernel(const float* __restrict__ x,
                                         const int32_t* __restrict__ order, int64_t rows,
                                         int cols4, __nv_bfloat16* __restrict__ hi,
                                         __nv_bfloat16* __restrict__ mid) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols4) return;
  const int64_t v = i / cols4;
  const int c = (int)(i - v * cols4);
  const float4 val = __ldg(reinterpret_cast<const float4*>(x + (int64_t)__ldg(order + v) * cols4 * 4) + c);
  uint2 h, m;
  split2_bf16(val.x, val.y, h.x, m.x);
  split2_bf16(val.z, val.w, h.y, m.y);
  *reinterpret_cast<uint2*>(hi + i * 4) = h;
  *reinterpret_cast<uint2*>(mid + i * 4) = m;
}

__global__ void split_transpose_kernel(const float* __restrict__ x, int64_t rows, int64_t cols,
                                       __nv_bfloat16* __restrict__ hi_t,
                                       __nv_bfloat16* __restrict__ mid_t) {
  __shared__ float tile[32][33];
  const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int64_t r = r0 + j, cc = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && cc < cols) ? __ldg(x + r * cols + cc) : 0.0f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int64_t cc = c0 + j, r = r0 + threadIdx.x;
    if (cc < cols && r < rows) {
      __nv_bfloat16 h, l;
      split_bf16(tile[threadIdx.x][j], h, l);
      hi_t[cc * rows + r] = h;
      mid_t[cc * rows + r] = l;
    }
  }
}

__global__ void reduce_splits_kernel(const float* __restrict__ partial, int splits, int64_t stride,
                                     int64_t n, float* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.0f;
  for (int s = 0; s < splits; ++s) acc += __ldg(partial + (int64_t)s * stride + i);
  out[i] = acc;
}

}  // namespace

// The tensor cores add into their fp32 accumulator by truncation, so the error of
// a sum grows with the number of terms one accumulator takes: measured on the
// weight-gradient product of the layer (K = 524 288 samples in 9 slices) it was
// 7e-4 of the result's rms, against 9e-5 for K = 65 536 and 2e-5 for an fp32
// FMA loop; with slices of 8192 / 4096 / 2048 terms 9.6e-5 / 5.9e-5 / 3.4e-5.
// K is therefore cut into slices of at most kMaxChain terms, whose results are
// summed in round-to-nearest fp32.
constexpr int64_t kMaxChain = 2048;

int gemm_pick_k_splits(int64_t M, int64_t N, int64_t K) {
  const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + kBNMax - 1) / kBNMax);
  const int64_t k_blocks = (K + kBK - 1) / kBK;
  int64_t splits = sm_count() / (tiles > 0 ? tiles : 1);
  if (splits < 1) splits = 1;
  const int64_t for_chain = (K + kMaxChain - 1) / kMaxChain;
  if (splits < for_chain) splits = for_chain;
  if (splits > k_blocks) splits = k_blocks > 0 ? k_blocks : 1;
  return (int)splits;
}

int gemm_bf16x3_grad_image(cudaStream_t stream, int64_t M, int channels, int64_t K,
                           const GemmOperand& a, const GemmOperand& b, void* image, int group,
                           int* err_flag) {
  const int64_t N = (int64_t)channels * 16;
  TFGPC_REQUIRE(M > 0 && channels > 0 && K > 0 && M < (int64_t)INT32_MAX && K < (int64_t)INT32_MAX,
                "GEMM expects positive sizes below 2^31");
  TFGPC_REQUIRE(a.major == Major::K && channels % 2 == 0 && (uintptr_t)image % 32 == 0 &&
                group >= 1 && group <= 4,
                "gradient-image GEMM expects a K-major left operand and groups of 1 to 4 rows");
  const bool b_mn = b.major == Major::MN;
  int bn = (int)(N < kBNMax ? N : kBNMax);
  const int gran = b_mn ? 64 : 32;
  bn = (bn + gran - 1) / gran * gran;
  CUtensorMap maps[5] = {};
  int rc;
  if ((rc = make_map(&maps[0], a.hi, K, M, a.ld, kBK, kBM))) return rc;
  if ((rc = make_map(&maps[1], a.mid, K, M, a.ld, kBK, kBM))) return rc;
  const __nv_bfloat16* bp[2] = {b.hi, b.mid};
  for (int i = 0; i < 2; ++i) {
    rc = b_mn ? make_map(&maps[2 + i], bp[i], N, K, b.ld, 64, kBK)
              : make_map(&maps[2 + i], bp[i], K, N, b.ld, kBK, bn);
    if (rc) return rc;
  }
  TileSchedule sch;
  sch.m_tiles = (int)((M + kBM - 1) / kBM);
  sch.n_tiles = (int)((N + bn - 1) / bn);
  sch.k_blocks = (int)((K + kBK - 1) / kBK);
  sch.k_splits = 1;
  sch.add_slices = 0;
  sch.k_blocks_per_split = sch.k_blocks;
  if (b_mn)
    return launch<false, true, 1>(stream, maps, M, N, bn, sch, err_flag, (uint8_t*)image, channels,
                                  group);
  return launch<false, false, 1>(stream, maps, M, N, bn, sch, err_flag, (uint8_t*)image, channels,
                                 group);
}

int gemm_bf16x3_grad_image_tn(cudaStream_t stream, int channels, int64_t N, int64_t K,
                              const GemmOperand& a, const GemmOperand& b, void* image, int group,
                              int* err_flag) {
  const int64_t M = (int64_t)channels * 16;
  TFGPC_REQUIRE(channels > 0 && N > 0 && K > 0 && N < (int64_t)INT32_MAX && K < (int64_t)INT32_MAX,
                "GEMM expects positive sizes below 2^31");
  TFGPC_REQUIRE(a.major == Major::MN && b.major == Major::K && channels % 2 == 0 &&
                (uintptr_t)image % 32 == 0 && group >= 1 && group <= 4,
                "gradient-image GEMM (transposed form) expects an MN-major left and a K-major "
                "right operand and groups of 1 to 4 rows");
  int bn = (int)(N < kBNMax ? N : kBNMax);
  bn = (bn + 31) / 32 * 32;
  CUtensorMap maps[5] = {};
  int rc;
  if ((rc = make_map(&maps[0], a.hi, M, K, a.ld, 64, kBK))) return rc;
  if ((rc = make_map(&maps[1], a.mid, M, K, a.ld, 64, kBK))) return rc;
  if ((rc = make_map(&maps[2], b.hi, K, N, b.ld, kBK, bn))) return rc;
  if ((rc = make_map(&maps[3], b.mid, K, N, b.ld, kBK, bn))) return rc;
  TileSchedule sch;
  sch.m_tiles = (int)((M + kBM - 1) / kBM);
  sch.n_tiles = (int)((N + bn - 1) / bn);
  sch.k_blocks = (int)((K + kBK - 1) / kBK);
  sch.k_splits = 1;
  sch.add_slices = 0;
  sch.k_blocks_per_split = sch.k_blocks;
  return launch<true, false, 3>(stream, maps, M, N, bn, sch, err_flag, (uint8_t*)image, channels,
                                group);
}

int gemm_bf16x3_tn_scatter(cudaStream_t stream, int64_t M, int64_t N, int64_t K,
                           const GemmOperand& a, const GemmOperand& b, float* out, int64_t ld_out,
                           const int32_t* row_order, int* err_flag) {
  TFGPC_REQUIRE(M > 0 && N > 0 && K > 0 && M < (int64_t)INT32_MAX && N < (int64_t)INT32_MAX &&
                K < (int64_t)INT32_MAX && ld_out < (int64_t)INT32_MAX,
                "GEMM expects positive sizes below 2^31");
  TFGPC_REQUIRE(a.major == Major::MN && b.major == Major::K && row_order && out &&
                (uintptr_t)out % 32 == 0 && ld_out % 8 == 0,
                "row-scattering GEMM expects an MN-major left and a K-major right operand and "
                "32-byte aligned output rows");
  int bn = (int)(N < kBNMax ? N : kBNMax);
  bn = (bn + 31) / 32 * 32;
  CUtensorMap maps[5] = {};
  int rc;
  if ((rc = make_map(&maps[0], a.hi, M, K, a.ld, 64, kBK))) return rc;
  if ((rc = make_map(&maps[1], a.mid, M, K, a.ld, 64, kBK))) return rc;
  if ((rc = make_map(&maps[2], b.hi, K, N, b.ld, kBK, bn))) return rc;
  if ((rc = make_map(&maps[3], b.mid, K, N, b.ld, kBK, bn))) return rc;
  TileSchedule sch;
  sch.m_tiles = (int)((M + kBM - 1) / kBM);
  sch.n_tiles = (int)((N + bn - 1) / bn);
  sch.k_blocks = (int)((K + kBK - 1) / kBK);
  sch.k_splits = 1;
  sch.add_slices = 0;
  sch.k_blocks_per_split = sch.k_blocks;
  return launch<true, false, 4>(stream, maps, M, N, bn, sch, err_flag, (uint8_t*)out, (int)ld_out, 4,
                                row_order);
}

int gemm_bf16x3_tn(cudaStream_t stream, int64_t M, int64_t N, int64_t K, const GemmOperand& a,
                   const GemmOperand& b, float* ct, int64_t ldct, int* err_flag) {
  TFGPC_REQUIRE(M > 0 && N > 0 && K > 0 && M < (int64_t)INT32_MAX && N < (int64_t)INT32_MAX &&
                K < (int64_t)INT32_MAX, "GEMM expects positive sizes below 2^31");
  TFGPC_REQUIRE(a.major == Major::MN && b.major == Major::K,
                "transposed-output GEMM expects an MN-major left and a K-major right operand");
  int bn = (int)(N < kBNMax ? N : kBNMax);
  bn = (bn + 31) / 32 * 32;
  CUtensorMap maps[5];
  int rc;
  if ((rc = make_map(&maps[0], a.hi, M, K, a.ld, 64, kBK))) return rc;
  if ((rc = make_map(&maps[1], a.mid, M, K, a.ld, 64, kBK))) return rc;
  if ((rc = make_map(&maps[2], b.hi, K, N, b.ld, kBK, bn))) return rc;
  if ((rc = make_map(&maps[3], b.mid, K, N, b.ld, kBK, bn))) return rc;
  // C^T: N rows of M columns
  if ((rc = make_map_c(&maps[4], ct, M, N, 1, ldct, 0))) return rc;
  TileSchedule sch;
  sch.m_tiles = (int)((M + kBM - 1) / kBM);
  sch.n_tiles = (int)((N + bn - 1) / bn);
  sch.k_blocks = (int)((K + kBK - 1) / kBK);
  sch.k_splits = 1;
  sch.add_slices = 0;
  sch.k_blocks_per_split = sch.k_blocks;
  return launch<true, false, 2>(stream, maps, M, N, bn, sch, err_flag);
}

int gemm_bf16x3(cudaStream_t stream, int64_t M, int64_t N, int64_t K, const GemmOperand& a,
                const GemmOperand& b, float* c, int64_t ldc, int k_splits, int64_t split_stride,
                int* err_flag) {
  TFGPC_REQUIRE(M > 0 && N > 0 && K > 0, "GEMM expects positive sizes");
  TFGPC_REQUIRE(M < (int64_t)INT32_MAX && N < (int64_t)INT32_MAX && K < (int64_t)INT32_MAX,
                "GEMM sizes must stay below 2^31");
  TFGPC_REQUIRE(k_splits >= 1, "GEMM expects k_splits >= 1");
  const bool a_mn = a.major == Major::MN, b_mn = b.major == Major::MN;
  // columns of C per tile: a multiple of 32 (epilogue chunk), of 64 for MN-major B boxes
  int bn = (int)(N < kBNMax ? N : kBNMax);
  const int gran = b_mn ? 64 : 32;
  bn = (bn + gran - 1) / gran * gran;
  CUtensorMap maps[5];
  int rc;
  const __nv_bfloat16* ap[2] = {a.hi, a.mid};
  const __nv_bfloat16* bp[2] = {b.hi, b.mid};
  for (int i = 0; i < 2; ++i) {
    rc = a_mn ? make_map(&maps[i], ap[i], M, K, a.ld, 64, kBK)
              : make_map(&maps[i], ap[i], K, M, a.ld, kBK, kBM);
    if (rc) return rc;
    rc = b_mn ? make_map(&maps[2 + i], bp[i], N, K, b.ld, 64, kBK)
              : make_map(&maps[2 + i], bp[i], K, N, b.ld, kBK, bn);
    if (rc) return rc;
  }
  TileSchedule sch;
  sch.m_tiles = (int)((M + kBM - 1) / kBM);
  sch.n_tiles = (int)((N + bn - 1) / bn);
  sch.k_blocks = (int)((K + kBK - 1) / kBK);
  sch.k_splits = k_splits < sch.k_blocks ? k_splits : sch.k_blocks;
  sch.k_blocks_per_split = (sch.k_blocks + sch.k_splits - 1) / sch.k_splits;
  // drop empty trailing slices
  sch.k_splits = (sch.k_blocks + sch.k_blocks_per_split - 1) / sch.k_blocks_per_split;
  // split_stride 0 with several slices: all of them are added into c, which
  // starts from zero, by the store unit (the order of the additions, and with it
  // the last bits of the sums, varies from run to run)
  sch.add_slices = (sch.k_splits > 1 && split_stride == 0) ? 1 : 0;
  if (sch.add_slices) {
    TFGPC_CUDA(cudaMemset2DAsync(c, sizeof(float) * (size_t)ldc, 0, sizeof(float) * (size_t)N,
                                 (size_t)M, stream));
  } else if (sch.k_splits < k_splits && split_stride != 0) {
    // the caller sums k_splits slices: the unused ones must read as zero
    TFGPC_CUDA(cudaMemsetAsync(c + (int64_t)sch.k_splits * split_stride, 0,
                               sizeof(float) * (size_t)(k_splits - sch.k_splits) * split_stride,
                               stream));
  }
  rc = make_map_c(&maps[4], c, N, M, sch.add_slices ? 1 : sch.k_splits, ldc, split_stride);
  if (rc) return rc;
  if (a_mn && b_mn) return launch<true, true>(stream, maps, M, N, bn, sch, err_flag);
  if (a_mn) return launch<true, false>(stream, maps, M, N, bn, sch, err_flag);
  if (b_mn) return launch<false, true>(stream, maps, M, N, bn, sch, err_flag);
  return launch<false, false>(stream, maps, M, N, bn, sch, err_flag);
}

int split_to_bf16(cudaStream_t stream, const float* x, int64_t n, __nv_bfloat16* hi,
                  __nv_bfloat16* mid) {
  if (n <= 0) return TFGPC_OK;
  ProfScope prof(stream, "split_bf16");
  split_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, stream>>>(x, n, hi, mid);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

int split_rows_gather_to_bf16(cudaStream_t stream, const float* x, const int32_t* order,
                              int64_t rows, int64_t cols, __nv_bfloat16* hi, __nv_bfloat16* mid) {
  if (rows <= 0 || cols <= 0) return TFGPC_OK;
  TFGPC_REQUIRE(cols % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)hi % 8 == 0 &&
                (uintptr_t)mid % 8 == 0, "split_rows_gather expects 16-byte aligned rows");
  ProfScope prof(stream, "split_bf16");
  split_rows_gather_kernel<<<blocks_for(rows * (cols / 4), 256), 256, 0, stream>>>(
      x, order, rows, (int)(cols / 4), hi, mid);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

int split_transpose_to_bf16(cudaStream_t stream, const float* x, int64_t rows, int64_t cols,
                            __nv_bfloat16* hi_t, __nv_bfloat16* mid_t) {
  if (rows <= 0 || cols <= 0) return TFGPC_OK;
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  split_transpose_kernel<<<grid, dim3(32, 8), 0, stream>>>(x, rows, cols, hi_t, mid_t);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

int reduce_splits(cudaStream_t stream, const float* partial, int splits, int64_t stride, int64_t n,
                  float* out) {
  if (n <= 0) return TFGPC_OK;
  ProfScope prof(stream, "reduce_splits");
  reduce_splits_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(partial, splits, stride, n, out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

}  // namespace tfgpc

// Exercises the bounded wait of the tensor-core kernels (see include/tfgpc.h).
extern "C" int tfgpc_debug_bounded_wait(void* stream, void* ws, size_t ws_bytes,
                                        unsigned limit_us, int* returned_out) {
  using namespace tfgpc;
  TFGPC_REQUIRE(ws && returned_out && ws_bytes >= 1024 && (uintptr_t)ws % 256 == 0,
                "debug_bounded_wait expects a 256-byte aligned workspace of at least 1024 bytes");
  TFGPC_REQUIRE(limit_us >= 1 && limit_us <= 100000,
                "debug_bounded_wait expects a limit between 1 us and 100 ms");
  cudaStream_t st = (cudaStream_t)stream;
  // word 0 is the status word tfgpc_mcconv_status reads, word 1 the kernel's
  // "I returned" mark
  int* words = (int*)ws;
  TFGPC_CUDA(cudaMemsetAsync(words, 0, 2 * sizeof(int), st));
  wait_probe_kernel<<<1, 32, 0, st>>>(words, (unsigned long long)limit_us * 1000ull, words + 1);
  TFGPC_LAUNCH_CHECK();
  int back[2] = {0, 0};
  int rc = read_small(st, words, sizeof(back), back);
  if (rc) return rc;
  *returned_out = back[1];
  return TFGPC_OK;
}

