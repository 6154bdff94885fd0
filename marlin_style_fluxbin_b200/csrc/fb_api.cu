// Error reporting, device facts and fb_query for the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

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

namespace {
// One cache for every descriptor this library encodes, keyed by (address, O, G, kind).
struct MapKey {
  const void* ptr;
  int O, G, kind;
  bool operator==(const MapKey& other) const { return ptr == other.ptr && O == other.O && G == other.G && kind == other.kind; }
};
struct MapHash {
  size_t operator()(const MapKey& key) const {
    return std::hash<const void*>()(key.ptr) ^ ((size_t)key.O * 1315423911u) ^ ((size_t)key.G << 40) ^ ((size_t)key.kind << 52);
  }
};
std::mutex g_map_lock;
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;
PFN_cuTensorMapEncodeTiled g_encode = nullptr;

// Caller holds g_map_lock.
bool encoder_ready() {
  if (g_encode) return true;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult status;
  cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
  if (err != cudaSuccess || status != cudaDriverEntryPointSuccess || !fn) {
    cuda_fail(err, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    return false;
  }
  g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
  return true;
}
}  // namespace

bool plane_tensor_map(const uint8_t* planes, int O, int G, int box_units, int box_runs, CUtensorMap* out) {
  std::lock_guard<std::mutex> guard(g_map_lock);
  if (!encoder_ready()) return false;
  const MapKey key{planes, O, G, box_units * 256 + box_runs};
  auto found = g_maps.find(key);
  if (found != g_maps.end()) {
    *out = found->second;
    return true;
  }
  const cuuint64_t dims[3] = {128, (cuuint64_t)(O / 32), (cuuint64_t)G * 3};
  const cuuint64_t strides[2] = {512, (cuuint64_t)O * 16};  // bytes, dims 1 and 2
  const cuuint32_t box[3] = {128, (cuuint32_t)box_units, (cuuint32_t)box_runs};
  const cuuint32_t step[3] = {1, 1, 1};
  CUtensorMap map;
  const CUresult rc = g_encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t*>(planes), dims, strides, box, step,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    fail(FB_ECUDA, "cuTensorMapEncodeTiled failed with code %d for planes [%d,3,%d,16]", (int)rc, G, O);
    return false;
  }
  if (g_maps.size() >= 16384) g_maps.clear();
  g_maps.emplace(key, map);
  *out = map;
  return true;
}

bool group_row_tensor_map(const void* base, int elem_bytes, int O, int G, CUtensorMap* out) {
  std::lock_guard<std::mutex> guard(g_map_lock);
  if (!encoder_ready()) return false;
  const MapKey key{base, O, G, 1 << 20 | elem_bytes};
  auto found = g_maps.find(key);
  if (found != g_maps.end()) {
    *out = found->second;
    return true;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)O, (cuuint64_t)G};
  const cuuint64_t strides[1] = {(cuuint64_t)O * elem_bytes};
  const cuuint32_t box[2] = {32, 2};
  const cuuint32_t step[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = g_encode(&map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                               strides, box, step, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    fail(FB_ECUDA, "cuTensorMapEncodeTiled failed with code %d for a [%d,%d] tensor of %d-byte elements", (int)rc, G, O, elem_bytes);
    return false;
  }
  if (g_maps.size() >= 16384) g_maps.clear();
  g_maps.emplace(key, map);
  *out = map;
  return true;
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
  if (!strcmp(key, "w3_smem_bytes")) return 32768 + 8 * 3 * 3328 + 8 * 3 * 8;  // M = 1: tables + per-warp rings (planes, scales, zero points) + barriers
  if (!strcmp(key, "tp_max_world")) return 8;
  if (!strcmp(key, "sm_count") || !strcmp(key, "max_smem")) {
    const fb::DeviceInfo* info = fb::device_info();
    if (!info) return FB_ECUDA;
    return !strcmp(key, "sm_count") ? info->sm_count : info->max_smem_optin;
  }
  return fb::fail(FB_EINVAL, "fb_query: unknown key '%s'", key);
}
