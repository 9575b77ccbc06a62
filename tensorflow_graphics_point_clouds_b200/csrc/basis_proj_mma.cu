// Host side of the tensor-core basis projection (basis_proj_mma.cuh): the
// one-off split of the feature matrix and the two launchers.
#include "basis_proj_mma.cuh"

namespace tfgpc {

namespace {

// feat [n, C] fp32 -> fs [n, 2, C] bf16: row 0 the hi terms, row 1 the mid terms.
__global__ void split_features_kernel(const float* __restrict__ feat, int64_t n, int C,
                                      __nv_bfloat16* __restrict__ fs) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n * C) return;
  const int64_t row = i / C;
  const int c = (int)(i - row * C);
  const float4 v = __ldg(reinterpret_cast<const float4*>(feat + i));
  uint2 h, m;
  bpm::split2(v.x, v.y, h.x, m.x);
  bpm::split2(v.z, v.w, h.y, m.y);
  *reinterpret_cast<uint2*>(fs + row * 2 * C + c) = h;
  *reinterpret_cast<uint2*>(fs + row * 2 * C + C + c) = m;
}

constexpr size_t kMaxBlockSmem = 227 * 1024;

template <typename Kern>
int launch_persistent(Kern kern, int warp_bytes, int max_warps, int64_t ns, int* grid_out,
                      int* threads_out, size_t* smem_out) {
  int warps = (int)(kMaxBlockSmem / (size_t)warp_bytes);
  if (warps > max_warps) warps = max_warps;
  const size_t smem = (size_t)warps * warp_bytes;
  TFGPC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int64_t sample_blocks = (ns + 31) / 32;
  int64_t grid = (sample_blocks + warps - 1) / warps;
  if (grid > sm_count()) grid = sm_count();
  if (grid < 1) grid = 1;
  *grid_out = (int)grid; *threads_out = warps * 32; *smem_out = smem;
  return TFGPC_OK;
}

template <int K, int OUT>
int launch_fwd(cudaStream_t st, int C, int64_t ns, const float* basis, const __nv_bfloat16* fs,
               const int2* neigh, const int32_t* ranges, float* out, __nv_bfloat16* hi,
               __nv_bfloat16* mid) {
  auto kern = bpm::basis_proj_mma_kernel<K, OUT>;
  int grid, threads; size_t smem;
  int rc = launch_persistent(kern, bpm::Cfg<K>::kFwdWarpBytes, 11, ns, &grid, &threads, &smem);
  if (rc) return rc;
  ProfScope prof(st, OUT == 0 ? "basis_proj_mma" : "basis_proj_split_mma");
  kern<<<grid, threads, smem, st>>>(C, ns, basis, fs, neigh, ranges, out, hi, mid);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

template <int K>
int launch_grads(cudaStream_t st, int C, int64_t ns, int64_t M, const float* basis,
                 const __nv_bfloat16* fs, const int2* neigh, const int32_t* ranges,
                 const float* in_grads, float* dbasis, float* dfeat) {
  auto kern = bpm::basis_proj_grads_mma_kernel<K>;
  int grid, threads; size_t smem;
  int rc = launch_persistent(kern, bpm::Cfg<K>::kGradWarpBytes, 7, ns, &grid, &threads, &smem);
  if (rc) return rc;
  ProfScope prof(st, "basis_proj_grads_mma");
  kern<<<grid, threads, smem, st>>>(C, ns, M, basis, fs, neigh, ranges, in_grads, dbasis, dfeat);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

}  // namespace

bool basis_proj_mma_supported(int K, int C) {
  return (K == 16 || K == 32 || K == 64) && C >= 16 && C % 16 == 0;
}

int split_features(cudaStream_t st, const float* feat, int64_t n, int C, __nv_bfloat16* fs) {
  if (n <= 0) return TFGPC_OK;
  TFGPC_REQUIRE(C % 4 == 0 && (uintptr_t)feat % 16 == 0 && (uintptr_t)fs % 16 == 0,
                "split_features expects 16-byte aligned rows");
  ProfScope prof(st, "split_features");
  split_features_kernel<<<blocks_for(n * C / 4, 256), 256, 0, st>>>(feat, n, C, fs);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

int basis_proj_mma_split(cudaStream_t st, int K, int C, int64_t ns, const float* basis,
                         const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                         __nv_bfloat16* hi, __nv_bfloat16* mid) {
  const int2* nb = (const int2*)neigh;
  switch (K) {
    case 16: return launch_fwd<16, 1>(st, C, ns, basis, fs, nb, ranges, nullptr, hi, mid);
    case 32: return launch_fwd<32, 1>(st, C, ns, basis, fs, nb, ranges, nullptr, hi, mid);
    case 64: return launch_fwd<64, 1>(st, C, ns, basis, fs, nb, ranges, nullptr, hi, mid);
  }
  return fail(TFGPC_EINVAL, "tensor-core projection expects 16, 32 or 64 basis functions");
}

// The same projection as fp32 [ns, C, K] (the drop-in op's output).
int basis_proj_mma_f32(cudaStream_t st, int K, int C, int64_t ns, const float* basis,
                       const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                       float* out) {
  const int2* nb = (const int2*)neigh;
  switch (K) {
    case 16: return launch_fwd<16, 0>(st, C, ns, basis, fs, nb, ranges, out, nullptr, nullptr);
    case 32: return launch_fwd<32, 0>(st, C, ns, basis, fs, nb, ranges, out, nullptr, nullptr);
    case 64: return launch_fwd<64, 0>(st, C, ns, basis, fs, nb, ranges, out, nullptr, nullptr);
  }
  return fail(TFGPC_EINVAL, "tensor-core projection expects 16, 32 or 64 basis functions");
}

int basis_proj_grads_mma(cudaStream_t st, int K, int C, int64_t ns, int64_t M, const float* basis,
                         const __nv_bfloat16* fs, const int32_t* neigh, const int32_t* ranges,
                         const float* in_grads, float* dbasis, float* dfeat) {
  const int2* nb = (const int2*)neigh;
  switch (K) {
    case 16: return launch_grads<16>(st, C, ns, M, basis, fs, nb, ranges, in_grads, dbasis, dfeat);
    case 32: return launch_grads<32>(st, C, ns, M, basis, fs, nb, ranges, in_grads, dbasis, dfeat);
    case 64: return launch_grads<64>(st, C, ns, M, basis, fs, nb, ranges, in_grads, dbasis, dfeat);
  }
  return fail(TFGPC_EINVAL, "tensor-core projection expects 16, 32 or 64 basis functions");
}

}  // namespace tfgpc
