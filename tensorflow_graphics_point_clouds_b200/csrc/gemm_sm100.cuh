// fp32-accurate GEMM on the sm_100a tensor cores (tcgen05 + TMEM + TMA).
//
// C[M,N] (fp32) = A[M,K] * B[N,K]^T where both operands are given as two bf16
// arrays each, x ~= hi + mid (see split_bf16): three tensor-core passes
// (hi*hi + hi*mid + mid*hi) accumulate in fp32 in tensor memory and reproduce
// the fp32 product to about 2^-17 relative, well inside the 1e-4 parity bound,
// where a single bf16 or tf32 pass is not.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace tfgpc {

// How an operand lies in global memory.
enum class Major : int {
  K = 0,   // [rows, K] row-major: the reduction index is contiguous
  MN = 1,  // [K, rows] row-major: the M (or N) index is contiguous
};

struct GemmOperand {
  const __nv_bfloat16* hi;
  const __nv_bfloat16* mid;
  int64_t ld;  // elements between consecutive rows of the global array
  Major major;
};

// C = A * B^T over k in [0, K).  With k_splits > 1 the reduction range is cut
// into k_splits slices and slice s writes its partial result to
// C + s * split_stride (the caller sums the slices); with split_stride 0 the
// slices are added into the one C instead (zeroed first; the order of the
// additions is not fixed).  M, N, K are the logical
// sizes; edges are handled by TMA zero fill and masked stores.
// err_flag (device int, zero-initialised by the caller) is set to 1 if a
// bounded wait inside the kernel ran out.
int gemm_bf16x3(cudaStream_t stream, int64_t M, int64_t N, int64_t K, const GemmOperand& a,
                const GemmOperand& b, float* c, int64_t ldc, int k_splits, int64_t split_stride,
                int* err_flag);

// The same product for C = [M, channels * 16] (K-major left operand), written not as
// fp32 but as the bf16 hi/mid operand image of the tensor-core projection
// gradients: per group of `group` rows (1 to 4), [hi | mid][channel][128 bytes],
// where the 16-byte chunk 2 * (row % group) + (k / 8) of a channel's line sits at
// position chunk ^ (channel % 8).  `image` holds ceil(M / group) groups.
int gemm_bf16x3_grad_image(cudaStream_t stream, int64_t M, int channels, int64_t K,
                           const GemmOperand& a, const GemmOperand& b, void* image, int group,
                           int* err_flag);

// The gradient image of C^T = (A * B^T)^T, A MN-major with M = channels * 16 rows,
// B K-major with one row per sample: the same image as gemm_bf16x3_grad_image
// for the product written with the roles swapped (see gemm_bf16x3_tn).
int gemm_bf16x3_grad_image_tn(cudaStream_t stream, int channels, int64_t N, int64_t K,
                              const GemmOperand& a, const GemmOperand& b, void* image, int group,
                              int* err_flag);

// C^T[N, M] (row-major, ldct elements per row) = (A * B^T)^T for an MN-major A
// ([K, M] row-major) and a K-major B ([N, K] row-major): the form to use when the
// small matrix is the natural left operand -- the tensor pipe reads an MN-major
// left operand faster than a K-major one (0.63 ms against 0.72 ms for
// 256 x 262144 x 2048) -- and the result is wanted with the large index first.
int gemm_bf16x3_tn(cudaStream_t stream, int64_t M, int64_t N, int64_t K, const GemmOperand& a,
                   const GemmOperand& b, float* ct, int64_t ldct, int* err_flag);

// The same product with row j of C^T written to row row_order[j] of `out`
// ([*, ld_out] fp32, 32-byte aligned rows): for right operands whose rows come in
// another sequence than the caller's.
int gemm_bf16x3_tn_scatter(cudaStream_t stream, int64_t M, int64_t N, int64_t K,
                           const GemmOperand& a, const GemmOperand& b, float* out, int64_t ld_out,
                           const int32_t* row_order, int* err_flag);

// Number of k slices that fills the GPU for an [M,N] output with reduction K.
int gemm_pick_k_splits(int64_t M, int64_t N, int64_t K);

// x -> (hi, mid) over n elements.
int split_to_bf16(cudaStream_t stream, const float* x, int64_t n, __nv_bfloat16* hi,
                  __nv_bfloat16* mid);
// [rows, cols] fp32 -> transposed [cols, rows] bf16 pair.
// hi/mid row v = split of row order[v] of x [rows, cols] (cols a multiple of 4).
int split_rows_gather_to_bf16(cudaStream_t stream, const float* x, const int32_t* order,
                              int64_t rows, int64_t cols, __nv_bfloat16* hi, __nv_bfloat16* mid);
int split_transpose_to_bf16(cudaStream_t stream, const float* x, int64_t rows, int64_t cols,
                            __nv_bfloat16* hi_t, __nv_bfloat16* mid_t);
// out[i] = sum_s partial[s * stride + i], i < n.
int reduce_splits(cudaStream_t stream, const float* partial, int splits, int64_t stride,
                  int64_t n, float* out);

}  // namespace tfgpc
