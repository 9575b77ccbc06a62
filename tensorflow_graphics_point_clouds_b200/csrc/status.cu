// Status reporting and small host utilities of the tfgpc library.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace tfgpc {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_err[0] = '\0'; }

struct ProfRecord { const char* name; cudaEvent_t a, b; };
static thread_local bool g_prof_on = false;
static thread_local ProfRecord* g_prof = nullptr;
static thread_local int g_prof_n = 0, g_prof_cap = 0;

ProfScope::ProfScope(cudaStream_t stream, const char* name) : slot(-1), st(stream) {
  if (!g_prof_on) return;
  if (g_prof_n == g_prof_cap) {
    int cap = g_prof_cap ? g_prof_cap * 2 : 256;
    ProfRecord* r = (ProfRecord*)realloc(g_prof, sizeof(ProfRecord) * cap);
    if (!r) return;
    for (int i = g_prof_cap; i < cap; ++i) { r[i].a = nullptr; r[i].b = nullptr; }
    g_prof = r; g_prof_cap = cap;
  }
  ProfRecord& r = g_prof[g_prof_n];
  if (!r.a && (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess)) return;
  r.name = name;
  slot = g_prof_n++;
  cudaEventRecord(r.a, st);
}

ProfScope::~ProfScope() {
  if (slot >= 0) cudaEventRecord(g_prof[slot].b, st);
}

ProfPause::ProfPause() : was_on(g_prof_on) { g_prof_on = false; }
ProfPause::~ProfPause() { g_prof_on = was_on; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- small device -> host reads ---------------------------------------------------
// The blocking entries need a count from the device (pairs found, samples kept).
// A cudaMemcpy for it would share the copy engine with whatever bulk download the
// caller has in flight on another stream and wait behind all of it (measured:
// 16 ms behind an 800 MB download).  Instead a one-warp kernel writes the values
// into a page of mapped pinned host memory and the host reads them after
// synchronising the stream.  One page per host thread and device, allocated on
// first use and kept.
namespace {

struct Mailbox { void* host; void* dev; };
thread_local Mailbox g_mail[64] = {};

__global__ void mailbox_kernel(const uint32_t* __restrict__ src, uint32_t* dst, int words) {
  for (int i = threadIdx.x; i < words; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
}

}  // namespace

int read_small(cudaStream_t st, const void* dev_src, size_t bytes, void* host_dst) {
  TFGPC_REQUIRE(bytes > 0 && bytes <= 4096 && bytes % 4 == 0 && (uintptr_t)dev_src % 4 == 0,
                "read_small expects 4 .. 4096 bytes, a multiple of 4");
  int dev = 0;
  TFGPC_CUDA(cudaGetDevice(&dev));
  TFGPC_REQUIRE(dev >= 0 && dev < 64, "read_small: device index out of range");
  Mailbox& m = g_mail[dev];
  if (!m.host) {
    TFGPC_CUDA(cudaHostAlloc(&m.host, 4096, cudaHostAllocMapped));
    TFGPC_CUDA(cudaHostGetDevicePointer(&m.dev, m.host, 0));
  }
  mailbox_kernel<<<1, 32, 0, st>>>((const uint32_t*)dev_src, (uint32_t*)m.dev, (int)(bytes / 4));
  TFGPC_LAUNCH_CHECK();
  TFGPC_CUDA(cudaStreamSynchronize(st));
  memcpy(host_dst, m.host, bytes);
  return TFGPC_OK;
}

}  // namespace tfgpc

extern "C" int tfgpc_read_device(void* stream, const void* device_src, size_t bytes,
                                 void* host_dst) {
  using namespace tfgpc;
  TFGPC_REQUIRE(device_src && host_dst, "read_device got a null pointer");
  return read_small((cudaStream_t)stream, device_src, bytes, host_dst);
}

extern "C" const char* tfgpc_last_error(void) { return tfgpc::g_err; }
extern "C" int tfgpc_version(void) { return 2; }   // 2: pdf_by_neighbor on the kernel-basis entries

extern "C" int tfgpc_profile_enable(int on) {
  tfgpc::g_prof_on = on != 0;
  if (!on) tfgpc::g_prof_n = 0;
  return TFGPC_OK;
}

extern "C" int tfgpc_profile_collect(char* names_out, size_t names_bytes, float* ms_out,
                                     int max_records, int* count_out) {
  using namespace tfgpc;
  TFGPC_REQUIRE(names_out && ms_out && count_out && names_bytes > 0, "profile_collect got a null pointer");
  size_t pos = 0;
  int n = 0;
  names_out[0] = '\0';
  for (int i = 0; i < g_prof_n && n < max_records; ++i) {
    ProfRecord& r = g_prof[i];
    TFGPC_CUDA(cudaEventSynchronize(r.b));
    float ms = 0.0f;
    TFGPC_CUDA(cudaEventElapsedTime(&ms, r.a, r.b));
    size_t len = strlen(r.name);
    if (pos + len + 2 > names_bytes) break;
    memcpy(names_out + pos, r.name, len);
    pos += len;
    names_out[pos++] = '\n';
    names_out[pos] = '\0';
    ms_out[n++] = ms;
  }
  *count_out = n;
  g_prof_n = 0;
  return TFGPC_OK;
}
