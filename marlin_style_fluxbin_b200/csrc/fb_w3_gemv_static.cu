// fb_w3_gemv_static: the W3 GEMV for callers that cannot hand over a scratch buffer.
//
// Some hosts of this library have no way to allocate device memory at the point where they
// call it: a serving engine that has already given every free byte to its KV-cache pool, a
// plugin that runs under a framework allocator it must not bypass, or code that is in the
// middle of capturing a CUDA graph, where allocation calls are not allowed.  For them the
// split-K scratch lives in this library's own image: a fixed array in device memory that
// every GPU which loads the library holds until the process exits.
//
// The array's name below is, in host code, only a handle for the runtime; it is not a
// device address.  The address a kernel can use is looked up once per device with
// cudaGetSymbolAddress while that device is current.
#include <mutex>

#include "fb_common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = (size_t)FB_W3_STATIC_SCRATCH_BYTES;
constexpr size_t kControlBytes = 16384;  // status word; the split-K combine words follow it (8 bytes per activation row and output row)

static __device__ __align__(256) unsigned char g_w3_static_scratch[kStaticScratchBytes];

// Device address of the array on the current device; nullptr after recording an error.
void* static_scratch_address() {
  static std::mutex lock;
  static void* address[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    fb::cuda_fail(err, "cudaGetDevice");
    return nullptr;
  }
  if (device < 0 || device >= 64) {
    fb::fail(FB_ELIMIT, "device ordinal %d outside 0..63", device);
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(lock);
  if (!address[device]) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_w3_static_scratch);
    if (err != cudaSuccess || !ptr) {
      fb::cuda_fail(err, "cudaGetSymbolAddress(static W3 scratch)");
      return nullptr;
    }
    address[device] = ptr;
  }
  return address[device];
}

}  // namespace

extern "C" int fb_w3_gemv_static(const void* x, int act_dtype, int m, const uint8_t* planes, const void* scales,
                                 int scale_dtype, const uint8_t* zeros, const int16_t* perm, void* out,
                                 int out_features, int in_features, unsigned flags, fb_stream_t stream) {
  const size_t need = fb_w3_gemv_scratch_bytes(m, out_features, in_features);
  if (need == 0) return fb::fail(FB_ELIMIT, "fb_w3_gemv_static: M=%d, O=%d, K=%d is outside the supported range", m, out_features, in_features);
  if (need > kStaticScratchBytes)
    return fb::fail(FB_ELIMIT,
                    "fb_w3_gemv_static: this problem needs %zu bytes of split-K scratch but the built-in scratch holds %zu; "
                    "use fb_w3_gemv with a caller-owned buffer",
                    need, kStaticScratchBytes);
  void* scratch = static_scratch_address();
  if (!scratch) return FB_ECUDA;
  // The array keeps whatever the previous call left (a call that failed on the device may leave
  // combine words behind); the status word and this call's combine words have to start at zero.
  cudaError_t err = cudaMemsetAsync(scratch, 0, kControlBytes + (size_t)m * out_features * 8, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fb::cuda_fail(err, "cudaMemsetAsync(static W3 scratch control block)");
  return fb_w3_gemv(x, act_dtype, m, planes, scales, scale_dtype, zeros, perm, out, out_features, in_features,
                    scratch, kStaticScratchBytes, flags, stream);
}
