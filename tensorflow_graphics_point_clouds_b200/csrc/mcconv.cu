// Monte-Carlo convolution forward and backward: the basis projection followed
// by (forward) or preceded by (backward) the weight GEMMs on the tensor cores.
//
// Forward:  X[s, c*K+k] = sum_m basis[m,k] * feat[nbr(m), c]   (basis_proj.cu,
//           written directly as the bf16 hi/mid pair the GEMM consumes)
//           out = X * W                                        (gemm_sm100.cu)
// Backward: dX = dOut * W^T, (dbasis, dfeat) = BasisProjGrads(dX),
//           dW = X^T * dOut  (split over the sample range, slices summed).
// This is the pair BasisProj -> tf.matmul of pylib/pc/layers/MCConv.py:174-191
// and its autodiff, without the fp32 [Ns, C, K] tensor between the two.
#include "basis_proj.cuh"
#include "gemm_sm100.cuh"

namespace tfgpc {

int basis_proj_split(cudaStream_t st, int K, int C, int64_t ns, const float* basis,
                     const float* feat, const int32_t* neigh, const int32_t* ranges,
                     __nv_bfloat16* hi, __nv_bfloat16* mid);
// basis_proj_mma.cu: the projection on warp-level tensor-core MMAs
bool basis_proj_mma_supported(int K, int C);
int split_features(cudaStream_t st, const float* feat, int64_t n, int C, __nv_bfloat16* fs);
int basis_proj_mma_split(cudaStream_t st, int K, int C, int64_t ns, const float* basis,
                         const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                         __nv_bfloat16* hi, __nv_bfloat16* mid);
int basis_proj_grads_mma(cudaStream_t st, int K, int C, int64_t ns, int64_t M, const float* basis,
                         const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                         const float* in_grads, float* dbasis, float* dfeat);

// basis_proj_grads_tc.cu: the gradients on tcgen05 tensor cores
bool basis_proj_grads_tc_supported(int K, int C);
int basis_proj_grads_tc_group(int64_t ns, int64_t M);
int basis_proj_grads_tc(cudaStream_t st, int group, int64_t ns, int64_t M, const float* basis,
                        const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                        const void* image, float* dbasis, float* dfeat, int* err_flag);

// basis_proj_grads_tcu.cu: the gradients on the rows of a group plan
int basis_proj_grads_tcu(cudaStream_t st, int64_t ns, int64_t M, const void* plan,
                         const __nv_bfloat16* basis_pair, const __nv_bfloat16* fs,
                         const int32_t* ranges, const void* image, float* dbasis, float* dfeat,
                         int* err_flag);

// basis_proj_fwd_tcu.cu: the projection on the rows of a group plan
int basis_proj_fwd_tcu(cudaStream_t st, int64_t ns, int64_t M, const void* plan,
                       const __nv_bfloat16* basis_pair, const __nv_bfloat16* fs,
                       __nv_bfloat16* x_hi, __nv_bfloat16* x_mid, int* err_flag);

namespace {

struct McWs {
  int* err;                  // [0] set by a GEMM whose bounded wait ran out
  __nv_bfloat16 *x_hi, *x_mid;      // [ns, C*K]
  __nv_bfloat16 *w_hi, *w_mid;      // [C*K, Cout]
  __nv_bfloat16 *g_hi, *g_mid;      // [ns, Cout]   (backward)
  float* dx;                        // [ns, C*K]    (backward)
  __nv_bfloat16* fs;                // [n_in, 2, C] split features (tensor-core projection)
  __nv_bfloat16 *wt_hi, *wt_mid;    // [Cout, C*K]: W transposed (backward)
  int dw_splits;
  size_t bytes;
};

McWs carve(void* ws, int K, int C, int Cout, int64_t ns, int64_t n_in, bool backward) {
  McWs w;
  char* p = (char*)ws;
  auto take = [&](size_t b) { char* r = p; p += align_up(b, 1024); return r; };
  const size_t ck = (size_t)C * K;
  w.err = (int*)take(256);
  w.x_hi = (__nv_bfloat16*)take((size_t)ns * ck * 2);
  w.x_mid = (__nv_bfloat16*)take((size_t)ns * ck * 2);
  w.w_hi = (__nv_bfloat16*)take(ck * Cout * 2);
  w.w_mid = (__nv_bfloat16*)take(ck * Cout * 2);
  // ahead of the backward-only buffers, so that a forward and a backward carve
  // of the same workspace agree on where it lies
  w.fs = nullptr;
  if (basis_proj_mma_supported(K, C)) w.fs = (__nv_bfloat16*)take((size_t)n_in * C * 4);
  w.dw_splits = 1;
  w.g_hi = w.g_mid = nullptr; w.dx = nullptr; w.wt_hi = w.wt_mid = nullptr;
  if (backward) {
    w.g_hi = (__nv_bfloat16*)take((size_t)ns * Cout * 2);
    w.g_mid = (__nv_bfloat16*)take((size_t)ns * Cout * 2);
    // as operand image of the tensor-core gradient kernel: one slot of 4*ck floats
    // per group of three (or four) samples
    w.dx = (float*)take((size_t)((ns + 2) / 3) * 4 * ck * 4);
    w.wt_hi = (__nv_bfloat16*)take(ck * Cout * 2);
    w.wt_mid = (__nv_bfloat16*)take(ck * Cout * 2);
    w.dw_splits = gemm_pick_k_splits((int64_t)ck, Cout, ns);
  }
  w.bytes = (size_t)(p - (char*)ws);
  return w;
}

int check_mc_args(const char* op, int K, int C, int Cout, int64_t ns, int64_t n_in, int64_t M) {
  TFGPC_REQUIRE(valid_basis(K), "%s expects a valid number of basis functions.", op);
  TFGPC_REQUIRE(valid_features(C), "%s expects a valid number of input features, between 1 and 8 "
                "or multiple of 8", op);
  TFGPC_REQUIRE(Cout > 0 && Cout % 8 == 0, "%s expects a number of output features that is a "
                "multiple of 8", op);
  TFGPC_REQUIRE(ns >= 0 && ns < (int64_t)INT32_MAX && n_in >= 0 && n_in < (int64_t)INT32_MAX &&
                M >= 0 && M <= (int64_t)INT32_MAX, "%s expects 0 <= ns, n_in, M < 2^31", op);
  return TFGPC_OK;
}

}  // namespace
}  // namespace tfgpc

using namespace tfgpc;

extern "C" size_t tfgpc_mcconv_workspace_bytes(int K, int C, int Cout, int64_t ns, int64_t n_in,
                                               int backward) {
  if (K <= 0 || C <= 0 || Cout <= 0 || ns < 0 || n_in < 0) return 0;
  return carve(nullptr, K, C, Cout, ns, n_in, backward != 0).bytes + 1024;
}

// The projection, written as the GEMM's bf16 operand pair: on tensor-core MMAs
// where the shape allows it, else on the SIMT kernels.
static int project(cudaStream_t st, int K, int C, int64_t ns, int64_t n_in, const float* basis,
                   const float* features, const int32_t* neighbors, const int32_t* ranges,
                   const McWs& w) {
  if (w.fs && (uintptr_t)features % 16 == 0) {
    int rc = split_features(st, features, n_in, C, w.fs);
    if (rc) return rc;
    return basis_proj_mma_split(st, K, C, ns, basis, w.fs, neighbors, ranges, w.x_hi, w.x_mid);
  }
  return basis_proj_split(st, K, C, ns, basis, features, neighbors, ranges, w.x_hi, w.x_mid);
}

extern "C" int tfgpc_mcconv_forward(void* stream, int K, int C, int Cout, int64_t ns, int64_t n_in,
                                    int64_t M, const float* basis, const float* features,
                                    const int32_t* neighbors, const int32_t* ranges,
                                    const float* weights, float* out, void* ws, size_t ws_bytes) {
  int rc = check_mc_args("MCConvForward", K, C, Cout, ns, n_in, M);
  if (rc) return rc;
  if (ns == 0) return TFGPC_OK;
  TFGPC_REQUIRE(ranges && weights && out && ws && (M == 0 || (basis && features && neighbors)),
                "MCConvForward got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)ws % 256 == 0,
                "MCConvForward expects 16-byte aligned buffers and a 256-byte aligned workspace");
  if (ws_bytes < tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 0))
    return fail(TFGPC_ENOMEM, "MCConvForward workspace too small: %zu < %zu", ws_bytes,
                tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 0));
  cudaStream_t st = (cudaStream_t)stream;
  McWs w = carve(ws, K, C, Cout, ns, n_in, false);
  const int64_t ck = (int64_t)C * K;
  TFGPC_CUDA(cudaMemsetAsync(w.err, 0, sizeof(int), st));
  rc = project(st, K, C, ns, n_in, basis, features, neighbors, ranges, w);
  if (rc) return rc;
  rc = split_to_bf16(st, weights, ck * Cout, w.w_hi, w.w_mid);
  if (rc) return rc;
  GemmOperand a{w.x_hi, w.x_mid, ck, Major::K};
  GemmOperand b{w.w_hi, w.w_mid, (int64_t)Cout, Major::MN};  // W is [C*K, Cout]: N contiguous
  // With at least one full tile of output features the roles are swapped,
  // out^T = W^T * X^T with W as the (MN-major) left operand, and the tiles are
  // transposed on their way out.
  if (Cout >= 128) return gemm_bf16x3_tn(st, Cout, ns, ck, b, a, out, Cout, w.err);
  return gemm_bf16x3(st, ns, Cout, ck, a, b, out, Cout, 1, 0, w.err);
}

extern "C" int tfgpc_mcconv_backward(void* stream, int K, int C, int Cout, int64_t ns,
                                     int64_t n_in, int64_t M, const float* basis,
                                     const float* features, const int32_t* neighbors,
                                     const int32_t* ranges, const float* weights,
                                     const float* out_grads, int x_in_workspace, float* dbasis_out,
                                     float* dfeat_out, float* dweights_out, void* ws,
                                     size_t ws_bytes) {
  int rc = check_mc_args("MCConvBackward", K, C, Cout, ns, n_in, M);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t ck = (int64_t)C * K;
  TFGPC_REQUIRE(dweights_out && weights, "MCConvBackward got a null pointer");
  if (ns == 0 || M == 0) {
    TFGPC_CUDA(cudaMemsetAsync(dweights_out, 0, sizeof(float) * (size_t)ck * Cout, st));
    if (M > 0 && dbasis_out) TFGPC_CUDA(cudaMemsetAsync(dbasis_out, 0, sizeof(float) * (size_t)M * K, st));
    if (n_in > 0 && dfeat_out) TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
    return TFGPC_OK;
  }
  TFGPC_REQUIRE(basis && features && neighbors && ranges && out_grads && dbasis_out && dfeat_out && ws,
                "MCConvBackward got a null pointer");
  TFGPC_REQUIRE((uintptr_t)basis % 16 == 0 && (uintptr_t)out_grads % 16 == 0 &&
                (uintptr_t)ws % 256 == 0,
                "MCConvBackward expects 16-byte aligned buffers and a 256-byte aligned workspace");
  if (ws_bytes < tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 1))
    return fail(TFGPC_ENOMEM, "MCConvBackward workspace too small: %zu < %zu", ws_bytes,
                tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 1));
  McWs w = carve(ws, K, C, Cout, ns, n_in, true);
  if (!x_in_workspace) {
    // (with x_in_workspace the word keeps what the forward call left: a timeout
    // there means that the projection this call is about to read is incomplete)
    TFGPC_CUDA(cudaMemsetAsync(w.err, 0, sizeof(int), st));
    rc = project(st, K, C, ns, n_in, basis, features, neighbors, ranges, w);
    if (rc) return rc;
  }
  // The weights are split again on every call (2 MB): every branch below then
  // works on the values of this call's `weights`, whatever the forward call saw.
  rc = split_to_bf16(st, weights, ck * Cout, w.w_hi, w.w_mid);
  if (rc) return rc;
  rc = split_to_bf16(st, out_grads, ns * Cout, w.g_hi, w.g_mid);
  if (rc) return rc;
  // dX[ns, C*K] = dOut[ns, Cout] * W^T: B rows are W's rows, reduction over Cout
  GemmOperand g_k{w.g_hi, w.g_mid, (int64_t)Cout, Major::K};
  GemmOperand w_k{w.w_hi, w.w_mid, (int64_t)Cout, Major::K};
  const bool fs_ok = w.fs && (uintptr_t)features % 16 == 0 && (uintptr_t)dbasis_out % 32 == 0 &&
                     (uintptr_t)dfeat_out % 16 == 0;
  if (fs_ok && basis_proj_grads_tc_supported(K, C)) {
    // dX goes straight into the operand image of the tcgen05 gradient kernel
    const int group = basis_proj_grads_tc_group(ns, M);
    if (ns % group != 0) {
      // columns of the samples that do not exist must read as finite values
      char* last = (char*)w.dx + (size_t)(ns / group) * 4 * ck * 4;
      TFGPC_CUDA(cudaMemsetAsync(last, 0, (size_t)4 * ck * 4, st));
    }
    // dX^T = W * dOut^T with W^T [Cout, C*K] as the MN-major left operand (the
    // tensor pipe reads it faster than a K-major one; transposing 2 MB is free),
    // tiles transposed back on their way into the image
    rc = split_transpose_to_bf16(st, weights, ck, Cout, w.wt_hi, w.wt_mid);
    if (rc) return rc;
    GemmOperand wt_mn{w.wt_hi, w.wt_mid, ck, Major::MN};
    rc = gemm_bf16x3_grad_image_tn(st, C, ns, Cout, wt_mn, g_k, w.dx, group, w.err);
    if (rc) return rc;
    TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
    rc = basis_proj_grads_tc(st, group, ns, M, basis, w.fs, neighbors, ranges, w.dx, dbasis_out,
                             dfeat_out, w.err);
  } else {
    rc = gemm_bf16x3(st, ns, ck, Cout, g_k, w_k, w.dx, ck, 1, 0, w.err);
    if (rc) return rc;
    if (fs_ok) {
      TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
      rc = basis_proj_grads_mma(st, K, C, ns, M, basis, w.fs, neighbors, ranges, w.dx, dbasis_out,
                                dfeat_out);
    } else {
      rc = tfgpc_basis_proj_grads(stream, K, C, ns, n_in, M, basis, features, neighbors, ranges,
                                  w.dx, dbasis_out, dfeat_out);
    }
  }
  if (rc) return rc;
  // dW[C*K, Cout] = X^T * dOut: both operands have the reduction (sample) index
  // as their row index, i.e. they are MN-major
  GemmOperand x_mn{w.x_hi, w.x_mid, ck, Major::MN};
  GemmOperand g_mn{w.g_hi, w.g_mid, (int64_t)Cout, Major::MN};
  // the reduction over the samples is cut into slices (see gemm_pick_k_splits)
  // that the GEMM adds into dweights_out
  return gemm_bf16x3(st, ck, Cout, ns, x_mn, g_mn, dweights_out, Cout, w.dw_splits, 0, w.err);
}

extern "C" int tfgpc_mcconv_grouped_supported(int K, int C) {
  return basis_proj_grads_tc_supported(K, C) ? 1 : 0;
}

namespace {

int check_grouped_args(const char* op, int K, int C, int Cout, const void* features,
                       const void* basis_pair, const void* ws, const void* plan) {
  TFGPC_REQUIRE(basis_proj_grads_tc_supported(K, C),
                "%s on a group plan expects K = 16 basis functions and C = 128 features", op);
  TFGPC_REQUIRE(Cout >= 128, "%s on a group plan expects at least 128 output features", op);
  TFGPC_REQUIRE((uintptr_t)features % 16 == 0 && (uintptr_t)basis_pair % 32 == 0 &&
                (uintptr_t)ws % 256 == 0 && (uintptr_t)plan % 256 == 0,
                "%s on a group plan expects 16-byte aligned features, a 32-byte aligned basis pair "
                "and 256-byte aligned workspace and plan", op);
  return TFGPC_OK;
}

// The projection in the plan's visiting order, into the workspace.
int project_grouped(cudaStream_t st, int C, int64_t ns, int64_t n_in, int64_t M,
                    const void* basis_pair, const float* features, const void* plan,
                    const McWs& w) {
  int rc = split_features(st, features, n_in, C, w.fs);
  if (rc) return rc;
  return basis_proj_fwd_tcu(st, ns, M, plan, (const __nv_bfloat16*)basis_pair, w.fs, w.x_hi,
                            w.x_mid, w.err);
}

}  // namespace

// Forward pass on the rows of a group plan: the projection is computed once per
// distinct neighbor of a group and written in the plan's visiting order; the
// weight GEMM puts its output rows back into the sample order.
extern "C" int tfgpc_mcconv_forward_grouped(
    void* stream, int K, int C, int Cout, int64_t ns, int64_t n_in, int64_t M,
    const void* basis_pair, const float* features, const float* weights, const int32_t* order,
    const void* plan, float* out, void* ws, size_t ws_bytes) {
  int rc = check_mc_args("MCConvForward", K, C, Cout, ns, n_in, M);
  if (rc) return rc;
  if (ns == 0) return TFGPC_OK;
  TFGPC_REQUIRE(weights && out && ws && order && plan && (M == 0 || (basis_pair && features)),
                "MCConvForward got a null pointer");
  rc = check_grouped_args("MCConvForward", K, C, Cout, features, basis_pair, ws, plan);
  if (rc) return rc;
  TFGPC_REQUIRE((uintptr_t)out % 32 == 0, "MCConvForward on a group plan expects a 32-byte aligned output");
  if (ws_bytes < tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 0))
    return fail(TFGPC_ENOMEM, "MCConvForward workspace too small: %zu < %zu", ws_bytes,
                tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 0));
  cudaStream_t st = (cudaStream_t)stream;
  McWs w = carve(ws, K, C, Cout, ns, n_in, false);
  const int64_t ck = (int64_t)C * K;
  TFGPC_CUDA(cudaMemsetAsync(w.err, 0, sizeof(int), st));
  rc = project_grouped(st, C, ns, n_in, M, basis_pair, features, plan, w);
  if (rc) return rc;
  rc = split_to_bf16(st, weights, ck * Cout, w.w_hi, w.w_mid);
  if (rc) return rc;
  GemmOperand a{w.x_hi, w.x_mid, ck, Major::K};
  GemmOperand b{w.w_hi, w.w_mid, (int64_t)Cout, Major::MN};
  // out^T = W^T * X^T; column v of out^T is the sample order[v]
  return gemm_bf16x3_tn_scatter(st, Cout, ns, ck, b, a, out, Cout, order, w.err);
}

// The backward pass on the rows of a group plan: dX is produced in the plan's
// visiting order (the rows of out_grads are gathered while they are split), the
// projection gradients run per distinct neighbor of a group instead of per
// pair, dW is unchanged.
extern "C" int tfgpc_mcconv_backward_grouped(
    void* stream, int K, int C, int Cout, int64_t ns, int64_t n_in, int64_t M,
    const void* basis_pair, const float* features, const int32_t* ranges, const float* weights,
    const float* out_grads, int x_in_workspace, const int32_t* order, const void* plan,
    float* dbasis_out, float* dfeat_out, float* dweights_out, void* ws, size_t ws_bytes) {
  int rc = check_mc_args("MCConvBackward", K, C, Cout, ns, n_in, M);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t ck = (int64_t)C * K;
  TFGPC_REQUIRE(dweights_out && weights, "MCConvBackward got a null pointer");
  if (ns == 0 || M == 0) {
    TFGPC_CUDA(cudaMemsetAsync(dweights_out, 0, sizeof(float) * (size_t)ck * Cout, st));
    if (M > 0 && dbasis_out) TFGPC_CUDA(cudaMemsetAsync(dbasis_out, 0, sizeof(float) * (size_t)M * K, st));
    if (n_in > 0 && dfeat_out) TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
    return TFGPC_OK;
  }
  TFGPC_REQUIRE(basis_pair && features && ranges && out_grads && order && plan && dbasis_out &&
                dfeat_out && ws, "MCConvBackward got a null pointer");
  rc = check_grouped_args("MCConvBackward", K, C, Cout, features, basis_pair, ws, plan);
  if (rc) return rc;
  TFGPC_REQUIRE((uintptr_t)out_grads % 16 == 0 && (uintptr_t)dbasis_out % 32 == 0 &&
                (uintptr_t)dfeat_out % 16 == 0,
                "MCConvBackward on a group plan expects 16-byte aligned gradients (dbasis 32)");
  if (ws_bytes < tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 1))
    return fail(TFGPC_ENOMEM, "MCConvBackward workspace too small: %zu < %zu", ws_bytes,
                tfgpc_mcconv_workspace_bytes(K, C, Cout, ns, n_in, 1));
  McWs w = carve(ws, K, C, Cout, ns, n_in, true);
  if (!x_in_workspace) {
    TFGPC_CUDA(cudaMemsetAsync(w.err, 0, sizeof(int), st));
    rc = project_grouped(st, C, ns, n_in, M, basis_pair, features, plan, w);
    if (rc) return rc;
  }
  // X lies in the visiting order (tfgpc_mcconv_forward_grouped wrote it so): the
  // rows of out_grads are brought into the same order while they are split, for
  // both products
  rc = split_rows_gather_to_bf16(st, out_grads, order, ns, Cout, w.g_hi, w.g_mid);
  if (rc) return rc;
  constexpr int group = 4;
  if (ns % group != 0) {
    char* last = (char*)w.dx + (size_t)(ns / group) * 4 * ck * 4;
    TFGPC_CUDA(cudaMemsetAsync(last, 0, (size_t)4 * ck * 4, st));
  }
  rc = split_transpose_to_bf16(st, weights, ck, Cout, w.wt_hi, w.wt_mid);
  if (rc) return rc;
  GemmOperand wt_mn{w.wt_hi, w.wt_mid, ck, Major::MN};
  GemmOperand gv_k{w.g_hi, w.g_mid, (int64_t)Cout, Major::K};
  rc = gemm_bf16x3_grad_image_tn(st, C, ns, Cout, wt_mn, gv_k, w.dx, group, w.err);
  if (rc) return rc;
  TFGPC_CUDA(cudaMemsetAsync(dfeat_out, 0, sizeof(float) * (size_t)n_in * C, st));
  rc = basis_proj_grads_tcu(st, ns, M, plan, (const __nv_bfloat16*)basis_pair, w.fs, ranges, w.dx,
                            dbasis_out, dfeat_out, w.err);
  if (rc) return rc;
  GemmOperand x_mn{w.x_hi, w.x_mid, ck, Major::MN};
  GemmOperand g_mn{w.g_hi, w.g_mid, (int64_t)Cout, Major::MN};
  return gemm_bf16x3(st, ck, Cout, ns, x_mn, g_mn, dweights_out, Cout, w.dw_splits, 0, w.err);
}

extern "C" int tfgpc_mcconv_status(void* stream, const void* ws, int* status_out) {
  TFGPC_REQUIRE(ws && status_out, "mcconv_status got a null pointer");
  int flag = 0;
  int rc = read_small((cudaStream_t)stream, ws, sizeof(int), &flag);
  if (rc) return rc;
  *status_out = flag ? TFGPC_ETIMEOUT : TFGPC_OK;
  if (flag) return fail(TFGPC_ETIMEOUT, "a bounded wait inside the tensor-core GEMM ran out");
  return TFGPC_OK;
}

// ---- plain fp32 matrix product on the same GEMM -------------------------------

extern "C" size_t tfgpc_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 1024;
  return 1024 + 2 * align_up((size_t)M * K * 2, 1024) + 2 * align_up((size_t)N * K * 2, 1024) +
         1024;
}

extern "C" int tfgpc_matmul_f32(void* stream, int64_t M, int64_t N, int64_t K, const float* a,
                                int a_transposed, const float* b, int b_transposed, float* c,
                                void* ws, size_t ws_bytes) {
  TFGPC_REQUIRE(M > 0 && N > 0 && K > 0, "matmul expects positive sizes");
  TFGPC_REQUIRE(a && b && c && ws, "matmul got a null pointer");
  TFGPC_REQUIRE((uintptr_t)ws % 256 == 0, "matmul expects a 256-byte aligned workspace");
  TFGPC_REQUIRE((a_transposed ? M : K) % 8 == 0 && (b_transposed ? K : N) % 8 == 0,
                "matmul expects row lengths that are multiples of 8");
  if (ws_bytes < tfgpc_matmul_workspace_bytes(M, N, K))
    return fail(TFGPC_ENOMEM, "matmul workspace too small: %zu < %zu", ws_bytes,
                tfgpc_matmul_workspace_bytes(M, N, K));
  cudaStream_t st = (cudaStream_t)stream;
  char* p = (char*)ws;
  int* err = (int*)p; p += 1024;
  __nv_bfloat16* a_hi = (__nv_bfloat16*)p; p += align_up((size_t)M * K * 2, 1024);
  __nv_bfloat16* a_mid = (__nv_bfloat16*)p; p += align_up((size_t)M * K * 2, 1024);
  __nv_bfloat16* b_hi = (__nv_bfloat16*)p; p += align_up((size_t)N * K * 2, 1024);
  __nv_bfloat16* b_mid = (__nv_bfloat16*)p; p += align_up((size_t)N * K * 2, 1024);
  TFGPC_CUDA(cudaMemsetAsync(err, 0, sizeof(int), st));
  int rc = split_to_bf16(st, a, M * K, a_hi, a_mid);
  if (rc) return rc;
  rc = split_to_bf16(st, b, N * K, b_hi, b_mid);
  if (rc) return rc;
  // a is [M,K] (K-major) or, transposed, [K,M] (MN-major); b is [K,N] (MN-major)
  // or, transposed, [N,K] (K-major)
  GemmOperand ao{a_hi, a_mid, a_transposed ? M : K, a_transposed ? Major::MN : Major::K};
  GemmOperand bo{b_hi, b_mid, b_transposed ? K : N, b_transposed ? Major::K : Major::MN};
  // several slices of the reduction are added into c by the GEMM itself
  return gemm_bf16x3(st, M, N, K, ao, bo, c, N, gemm_pick_k_splits(M, N, K), 0, err);
}
