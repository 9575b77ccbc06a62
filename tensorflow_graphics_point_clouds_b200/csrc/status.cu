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

}  // namespace tfgpc

extern "C" const char* tfgpc_last_error(void) { return tfgpc::g_err; }
extern "C" int tfgpc_version(void) { return 1; }

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
