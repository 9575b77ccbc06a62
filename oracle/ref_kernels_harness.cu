// TEST INFRASTRUCTURE ONLY -- never linked into the product library.
//
// Host harness around the reference's own CUDA kernels, so that the oracle
// (and through it the product) can be pinned to what the reference computes on
// the same GPU.  The reference's *_kernels.cu.cc translation units include no
// TensorFlow header; they only need an implementation of their IGPUDevice
// interface (custom_ops/tfg_custom_ops/shared/cc/kernels/gpu_device.hpp:56-181),
// which its TensorFlow build provides in tf_gpu_device.cpp.  This file provides
// a plain-CUDA one and C entry points that drive the kernel functions in the
// order the reference's OpKernels do:
//   FindNeighbors  find_neighbors/cc/ops/find_neighbors_ops.cpp:158-249
//   Sampling       sampling/cc/ops/sampling_ops.cpp:128-194
// The reference sources are compiled where they lie (see build_ref.py); nothing
// of them is copied into this repository.  All pointers are HOST pointers: the
// harness owns its device memory.  D = 3 only.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>

#include "tfg_custom_ops/shared/cc/kernels/defines.hpp"
#include "tfg_custom_ops/shared/cc/kernels/gpu_device.hpp"
#include "tfg_custom_ops/compute_keys/cc/kernels/compute_keys.h"
#include "tfg_custom_ops/build_grid_ds/cc/kernels/build_grid_ds.h"
// find_ranges_grid_ds.h reuses build_grid_ds.h's include guard
#undef BUILD_GRID_DS_CUH_
#include "tfg_custom_ops/find_neighbors/cc/kernels/find_ranges_grid_ds.h"
#include "tfg_custom_ops/find_neighbors/cc/kernels/count_neighbors.h"
#include "tfg_custom_ops/find_neighbors/cc/kernels/scan_alg.h"
#include "tfg_custom_ops/find_neighbors/cc/kernels/store_neighbors.h"
#include "tfg_custom_ops/compute_pdf/cc/kernels/compute_pdf.h"
#include "tfg_custom_ops/basis_proj/cc/kernels/basis_proj.h"
#include "tfg_custom_ops/basis_proj/cc/kernels/basis_proj_grads.h"
#include "tfg_custom_ops/sampling/cc/kernels/count_unique_keys.h"
#include "tfg_custom_ops/sampling/cc/kernels/store_unique_keys.h"
#include "tfg_custom_ops/sampling/cc/kernels/count_sampling_pd.h"
#include "tfg_custom_ops/sampling/cc/kernels/store_sampled_pts.h"
#include "tfg_custom_ops/sampling/cc/kernels/sampling_avg.h"

namespace {

int g_error = 0;  // sticky: first CUDA error seen by check_error

// Device buffers are recycled between calls, so that a repeated call measures
// the kernels and not cudaMalloc (the reference gets its temporaries from
// TensorFlow's pooled allocator).
struct PoolEntry { void* p; size_t bytes; bool busy; };
std::vector<PoolEntry> g_pool;

void* pool_get(size_t bytes) {
  for (auto& e : g_pool)
    if (!e.busy && e.bytes >= bytes && e.bytes <= 2 * bytes + 4096) { e.busy = true; return e.p; }
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  g_pool.push_back({p, bytes, true});
  return p;
}

void pool_put(void* p) {
  for (auto& e : g_pool)
    if (e.p == p) e.busy = false;
}

class PlainCudaDevice : public mccnn::IGPUDevice {
 public:
  PlainCudaDevice() : stream_(0) {
    cudaDeviceProp p;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaGetDeviceProperties(&p, dev);
    deviceProps_.warpSize_ = p.warpSize;
    deviceProps_.numMPs_ = p.multiProcessorCount;
    deviceProps_.maxThreadsXBlock_ = p.maxThreadsPerBlock;
    deviceProps_.maxThreadsXMP_ = p.maxThreadsPerMultiProcessor;
    deviceProps_.maxRegistersXBlock_ = p.regsPerBlock;
    deviceProps_.maxRegistersXMP_ = p.regsPerMultiprocessor;
    deviceProps_.sharedMemXBlock_ = p.sharedMemPerBlock;
    deviceProps_.sharedMemXMP_ = p.sharedMemPerMultiprocessor;
    deviceProps_.majorVersion_ = p.major;
    deviceProps_.minorVersion_ = p.minor;
  }
  ~PlainCudaDevice() override {
    cudaStreamSynchronize(stream_);
    for (void* p : dev_) pool_put(p);
    for (void* p : host_) cudaFreeHost(p);
  }
  void memset(void* d, int v, size_t n) override { cudaMemsetAsync(d, v, n, stream_); }
  void memcpy_device_to_device(void* d, void* s, size_t n) override {
    cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, stream_);
  }
  void memcpy_device_to_host(void* d, void* s, size_t n) override {
    cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToHost, stream_);
  }
  void memcpy_host_to_device(void* d, void* s, size_t n) override {
    cudaMemcpyAsync(d, s, n, cudaMemcpyHostToDevice, stream_);
  }
  void memcpy_host_to_symbol(void* d, void* s, size_t n) override {
    cudaMemcpyToSymbolAsync(d, s, n, 0, cudaMemcpyHostToDevice, stream_);
  }
  int get_max_active_block_x_sm(const unsigned int block, const void* f, const size_t smem) override {
    int n = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, f, (int)block, smem);
    return n;
  }
  void check_error(const char* file, int line) override {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess && !g_error) {
      g_error = (int)e;
      fprintf(stderr, "reference harness: CUDA error %s at %s:%d\n", cudaGetErrorString(e), file, line);
    }
  }
  float* getFloatTmpGPUBuffer(const unsigned int n, bool cpu = false) override {
    return (float*)alloc(sizeof(float) * (size_t)n, cpu);
  }
  int* getIntTmpGPUBuffer(const unsigned int n, bool cpu = false) override {
    return (int*)alloc(sizeof(int) * (size_t)n, cpu);
  }
  mccnn::int64_m* getInt64TmpGPUBuffer(const unsigned int n, bool cpu = false) override {
    return (mccnn::int64_m*)alloc(sizeof(mccnn::int64_m) * (size_t)n, cpu);
  }
  const cudaStream_t& getCUDAStream() override { return stream_; }

  // device copy of a host array (freed with the device object)
  template <class T>
  T* upload(const T* host, size_t n) {
    T* d = (T*)alloc(sizeof(T) * (n ? n : 1), false);
    if (n) cudaMemcpyAsync(d, host, sizeof(T) * n, cudaMemcpyHostToDevice, stream_);
    return d;
  }
  template <class T>
  void download(T* host, const T* dev, size_t n) {
    if (n) cudaMemcpyAsync(host, dev, sizeof(T) * n, cudaMemcpyDeviceToHost, stream_);
    cudaStreamSynchronize(stream_);
  }

 private:
  void* alloc(size_t bytes, bool cpu) {
    void* p = nullptr;
    if (bytes == 0) bytes = 4;
    if (cpu) { cudaMallocHost(&p, bytes); host_.push_back(p); }
    else { p = pool_get(bytes); dev_.push_back(p); }
    return p;
  }
  cudaStream_t stream_;
  std::vector<void*> dev_, host_;
};

struct Timer {
  cudaEvent_t a, b;
  Timer() { cudaEventCreate(&a); cudaEventCreate(&b); cudaEventRecord(a, 0); }
  float stop() {
    cudaEventRecord(b, 0); cudaEventSynchronize(b);
    float ms = 0; cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a); cudaEventDestroy(b);
    return ms;
  }
};

int finish() {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess && !g_error) g_error = (int)e;
  int r = g_error;
  g_error = 0;
  return r;
}

constexpr int kOffsetsPerBlock = 9;  // NUM_OFFSETS_X_COMPUTE_BLOCK, find_neighbors_ops.cpp:37

}  // namespace

extern "C" {

int ref_compute_keys(int n, const float* pts, const int* bids, int batch, const float* smin,
                     const int* num_cells, const float* inv_cell, long long* keys_out, float* ms) {
  std::unique_ptr<mccnn::IGPUDevice> dev(new PlainCudaDevice());
  auto* d = static_cast<PlainCudaDevice*>(dev.get());
  float* dp = d->upload(pts, (size_t)n * 3);
  int* db = d->upload(bids, n);
  float* ds = d->upload(smin, (size_t)batch * 3);
  int* dc = d->upload(num_cells, 3);
  float* di = d->upload(inv_cell, 3);
  mccnn::int64_m* dk = dev->getInt64TmpGPUBuffer(n);
  Timer t;
  mccnn::compute_keys_gpu<3>(dev, n, dp, db, ds, dc, di, dk);
  if (ms) *ms = t.stop();
  d->download((mccnn::int64_m*)keys_out, dk, n);
  return finish();
}

int ref_build_grid_ds(int n, const long long* sorted_keys, const int* num_cells, int batch,
                      int* ds_out, float* ms) {
  std::unique_ptr<mccnn::IGPUDevice> dev(new PlainCudaDevice());
  auto* d = static_cast<PlainCudaDevice*>(dev.get());
  mccnn::int64_m* dk = d->upload((const mccnn::int64_m*)sorted_keys, n);
  int* dc = d->upload(num_cells, 3);
  const unsigned ds_size = (unsigned)batch * num_cells[0] * num_cells[1];
  int* dd = dev->getIntTmpGPUBuffer(ds_size * 2);
  Timer t;
  mccnn::build_grid_ds_gpu<3>(dev, ds_size, n, dk, dc, dd);   // build_grid_ds_ops.cpp:98-104
  if (ms) *ms = t.stop();
  d->download(ds_out, dd, (size_t)ds_size * 2);
  return finish();
}

// Returns the number of pairs, or -1 on error.  ranges_out [ns]; neigh_out must
// hold 2 * capacity ints; if the count exceeds capacity only ranges are written.
long long ref_find_neighbors(int ns, const float* samples, const int* sbids, int n,
                             const float* pts, const long long* keys, const int* grid_ds, int batch,
                             const int* num_cells, const float* smin, const float* inv_cell,
                             const float* inv_radii, int* ranges_out, int* neigh_out,
                             long long capacity, float* ms) {
  std::unique_ptr<mccnn::IGPUDevice> dev(new PlainCudaDevice());
  auto* d = static_cast<PlainCudaDevice*>(dev.get());
  float* dsmp = d->upload(samples, (size_t)ns * 3);
  int* dsb = d->upload(sbids, ns);
  float* dp = d->upload(pts, (size_t)n * 3);
  mccnn::int64_m* dk = d->upload((const mccnn::int64_m*)keys, n);
  const size_t ds_elems = (size_t)batch * num_cells[0] * num_cells[1] * 2;
  int* dds = d->upload(grid_ds, ds_elems);
  int* dc = d->upload(num_cells, 3);
  float* dmin = d->upload(smin, (size_t)batch * 3);
  float* dic = d->upload(inv_cell, 3);
  float* dir = d->upload(inv_radii, 3);
  Timer t;
  int* out1 = dev->getIntTmpGPUBuffer(ns);
  dev->memset(out1, 0, sizeof(int) * (size_t)ns);
  mccnn::int64_m* tmp1 = dev->getInt64TmpGPUBuffer(ns);
  int* tmp2 = dev->getIntTmpGPUBuffer((unsigned)ns * kOffsetsPerBlock * 2);
  int* tmp3 = dev->getIntTmpGPUBuffer(kOffsetsPerBlock * 3);
  mccnn::compute_keys_gpu<3>(dev, ns, dsmp, dsb, dmin, dc, dic, tmp1);
  std::vector<int> offsets;
  unsigned num_offsets = mccnn::computeTotalNumOffsets(3, 1, offsets);
  if (num_offsets != (unsigned)kOffsetsPerBlock) return -1;
  int* pinned = dev->getIntTmpGPUBuffer((unsigned)offsets.size(), true);
  memcpy(pinned, offsets.data(), sizeof(int) * offsets.size());
  dev->memcpy_host_to_device(tmp3, pinned, sizeof(int) * offsets.size());
  mccnn::find_ranges_grid_ds_gpu<3>(dev, ns, n, 1, kOffsetsPerBlock, tmp3, tmp1, dk, dds, dc, tmp2);
  mccnn::count_neighbors<3>(dev, ns, kOffsetsPerBlock, dsmp, dp, tmp2, dir, out1);
  unsigned total = mccnn::scan_alg(dev, ns, out1);
  int* out2 = nullptr;
  if ((long long)total <= capacity) {
    out2 = dev->getIntTmpGPUBuffer(total * 2);
    dev->memset(out2, 0, sizeof(int) * (size_t)total * 2);
    mccnn::store_neighbors<3>(dev, 0, ns, kOffsetsPerBlock, dsmp, dp, tmp2, dir, nullptr, out1, out2);
  }
  if (ms) *ms = t.stop();
  if (out2) {
    d->download(neigh_out, out2, (size_t)total * 2);
    d->download(ranges_out, out1, ns);   // end offsets after store_neighbors' atomicAdd
  }
  int err = finish();
  return err ? -1 : (long long)total;
}

int ref_compute_pdf(int mode, int n, const float* pts, long long m, const int* neigh,
                    const int* ranges, const float* inv_bw, const float* inv_r, float* pdf_out,
                    const float* pdf_grads, float* pt_grads_out, float* ms) {
  std::unique_ptr<mccnn::IGPUDevice> dev(new PlainCudaDevice());
  auto* d = static_cast<PlainCudaDevice*>(dev.get());
  float* dp = d->upload(pts, (size_t)n * 3);
  int* dn = d->upload(neigh, (size_t)m * 2);
  int* dr = d->upload(ranges, n);
  float* db = d->upload(inv_bw, 3);
  float* dir = d->upload(inv_r, 3);
  float* dout = dev->getFloatTmpGPUBuffer(n);
  Timer t;
  mccnn::compute_pdf_gpu<3>(dev, mode, n, (unsigned)m, dir, db, dp, dn, dr, dout);
  if (ms) *ms = t.stop();
  d->download(pdf_out, dout, n);
  if (pdf_grads && pt_grads_out) {
    float* dg = d->upload(pdf_grads, n);
    float* dgo = dev->getFloatTmpGPUBuffer((unsigned)n * 3);
    dev->memset(dgo, 0, sizeof(float) * (size_t)n * 3);       // compute_pdf_ops.cpp:226-229
    mccnn::compute_pdf_grads_gpu<3>(dev, mode, n, n, (unsigned)m, dir, db, dp, dn, dr, dg, dgo);
    d->download(pt_grads_out, dgo, (size_t)n * 3);
  }
  return finish();
}

}  // extern "C"

template <int K>
static int basis_proj_impl(int c, int ns, int n_in, long long m, const float* basis,
                           const float* feat, const int* neigh, const int* ranges, float* out,
                           const float* in_grads, float* dbasis, float* dfeat, float* ms) {
  std::unique_ptr<mccnn::IGPUDevice> dev(new PlainCudaDevice());
  auto* d = static_cast<PlainCudaDevice*>(dev.get());
  float* db = d->upload(basis, (size_t)m * K);
  float* df = d->upload(feat, (size_t)n_in * c);
  int* dn = d->upload(neigh, (size_t)m * 2);
  int* dr = d->upload(ranges, ns);
  float* dout = dev->getFloatTmpGPUBuffer((unsigned)((size_t)ns * c * K));
  dev->memset(dout, 0, sizeof(float) * (size_t)ns * c * K);      // basis_proj_ops.cpp:121-124
  Timer t;
  mccnn::basis_proj_gpu<K>(dev, ns, c, df, db, dn, dr, dout);
  if (ms) *ms = t.stop();
  d->download(out, dout, (size_t)ns * c * K);
  if (in_grads && dbasis && dfeat) {
    float* dg = d->upload(in_grads, (size_t)ns * c * K);
    float* dgb = dev->getFloatTmpGPUBuffer((unsigned)((size_t)m * K));
    float* dgf = dev->getFloatTmpGPUBuffer((unsigned)((size_t)n_in * c));
    dev->memset(dgb, 0, sizeof(float) * (size_t)m * K);          // basis_proj_ops.cpp:205-212
    dev->memset(dgf, 0, sizeof(float) * (size_t)n_in * c);
    mccnn::basis_proj_grads_gpu<K>(dev, n_in, ns, (unsigned)m, c, df, db, dn, dr, dg, dgf, dgb);
    d->download(dbasis, dgb, (size_t)m * K);
    d->download(dfeat, dgf, (size_t)n_in * c);
  }
  return finish();
}

extern "C" {

int ref_basis_proj(int k, int c, int ns, int n_in, long long m, const float* basis,
                   const float* feat, const int* neigh, const int* ranges, float* out,
                   const float* in_grads, float* dbasis, float* dfeat, float* ms) {
  switch (k) {
    case 8: return basis_proj_impl<8>(c, ns, n_in, m, basis, feat, neigh, ranges, out, in_grads, dbasis, dfeat, ms);
    case 16: return basis_proj_impl<16>(c, ns, n_in, m, basis, feat, neigh, ranges, out, in_grads, dbasis, dfeat, ms);
    case 32: return basis_proj_impl<32>(c, ns, n_in, m, basis, feat, neigh, ranges, out, in_grads, dbasis, dfeat, ms);
    case 64: return basis_proj_impl<64>(c, ns, n_in, m, basis, feat, neigh, ranges, out, in_grads, dbasis, dfeat, ms);
  }
  return -1;
}

// mode 0 Poisson disk, 1 cell average (sampling_ops.cpp:141,174).  Outputs sized
// for n samples; returns the number of samples or -1.
long long ref_sampling(int mode, int n, const float* pts, const int* bids, const long long* keys,
                       const int* num_cells, long long m, const int* neigh, const int* ranges,
                       float* pts_out, int* bids_out, int* idx_out, float* ms) {
  std::unique_ptr<mccnn::IGPUDevice> dev(new PlainCudaDevice());
  auto* d = static_cast<PlainCudaDevice*>(dev.get());
  float* dp = d->upload(pts, (size_t)n * 3);
  int* db = d->upload(bids, n);
  mccnn::int64_m* dk = d->upload((const mccnn::int64_m*)keys, n);
  int* dc = d->upload(num_cells, 3);
  int* dn = d->upload(neigh, (size_t)m * 2);
  int* dr = d->upload(ranges, n);
  Timer t;
  unsigned num_keys = mccnn::count_unique_keys_gpu(dev, n, dk);
  int* tmp1 = dev->getIntTmpGPUBuffer(num_keys);
  mccnn::store_unique_keys_gpu(dev, n, dk, tmp1);
  long long result = 0;
  float* op = dev->getFloatTmpGPUBuffer((unsigned)n * 3);
  int* ob = dev->getIntTmpGPUBuffer(n);
  int* oi = dev->getIntTmpGPUBuffer(n);
  if (mode == 0) {
    int* tmp2 = dev->getIntTmpGPUBuffer(n);
    int num_sampled = 0;
    mccnn::count_sampling_pd_gpu<3>(dev, n, num_keys, tmp1, dk, dp, dn, dr, dc, num_sampled, tmp2);
    mccnn::store_sampled_pts_gpu<3>(dev, n, num_sampled, dp, db, tmp2, op, ob, oi);
    result = num_sampled;
  } else {
    mccnn::sampling_avg_gpu<3>(dev, n, num_keys, dk, dp, dc, tmp1, op, ob);
    result = num_keys;
  }
  if (ms) *ms = t.stop();
  d->download(pts_out, op, (size_t)result * 3);
  d->download(bids_out, ob, (size_t)result);
  if (mode == 0) d->download(idx_out, oi, (size_t)result);
  int err = finish();
  return err ? -1 : result;
}

}  // extern "C"
