// Error reporting, device facts and fb_query for the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "fb_common.cuh"

namespace fb {

static thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int cuda_fail(cudaError_t err, const char* what) {
  return fail(FB_ECUDA, "%s: %s", what, cudaGetErrorString(err));
}

bool pdl_allowed() {
  static const bool allowed = getenv("FB_NO_PDL") == nullptr;
  return allowed;
}

const DeviceInfo* device_info() {
  static DeviceInfo table[64];
  static bool known[64] = {};
  static std::mutex lock;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) { cuda_fail(err, "cudaGetDevice"); return nullptr; }
  if (device < 0 || device >= 64) { fail(FB_ELIMIT, "device ordinal %d outside 0..63", device); return nullptr; }
  std::lock_guard<std::mutex> guard(lock);
  if (!known[device]) {
    DeviceInfo info;
    int major = 0;
    err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (err != cudaSuccess) { cuda_fail(err, "cudaDeviceGetAttribute"); return nullptr; }
    if (major != 10) { fail(FB_ECUDA, "this library is built for sm_100a only; device %d has compute capability major %d", device, major); return nullptr; }
    table[device] = info;
    known[device] = true;
  }
  return &table[device];
}

}  // namespace fb

extern "C" const char* fb_last_error(void) { return fb::g_error; }

extern "C" int64_t fb_query(const char* key) {
  if (!key) return fb::fail(FB_EINVAL, "fb_query: null key");
  if (!strcmp(key, "version")) return 1;
  if (!strcmp(key, "w3_max_m")) return 4;            // table-lookup kernel
  if (!strcmp(key, "w3_mma_max_m")) return 16;       // tensor-core kernel
  if (!strcmp(key, "w3_max_splits")) return 16;      // contributions combined per output
  if (!strcmp(key, "w3_ctas_per_sm")) return 2;
  if (!strcmp(key, "w3_smem_bytes")) return 32768 + 8 * 3 * 3072 + 8 * 3 * 8;  // M = 1: tables + per-warp rings + barriers
  if (!strcmp(key, "tp_max_world")) return 8;
  if (!strcmp(key, "sm_count") || !strcmp(key, "max_smem")) {
    const fb::DeviceInfo* info = fb::device_info();
    if (!info) return FB_ECUDA;
    return !strcmp(key, "sm_count") ? info->sm_count : info->max_smem_optin;
  }
  return fb::fail(FB_EINVAL, "fb_query: unknown key '%s'", key);
}
