// Shared helpers of the sm_100a kernels: error reporting for the C ABI, 16-bit float
// conversion, and thin wrappers over the PTX used for bulk asynchronous copies
// (cp.async.bulk + mbarrier).  Every device-side wait is bounded.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fluxbin_b200.h"

namespace fb {

// ---- host side --------------------------------------------------------------------
int fail(int code, const char* fmt, ...);  // records the message, returns `code`
int cuda_fail(cudaError_t err, const char* what);

struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
};
// Facts about the current device, cached per device ordinal.  Returns nullptr on error
// (after recording it).
const DeviceInfo* device_info();

// Programmatic dependent launch can be switched off for the whole library by setting the
// environment variable FB_NO_PDL (read once); used to tell launch-overlap effects apart.
bool pdl_allowed();

// Tiled-copy descriptor of a W3 planes tensor [G,3,O,16] seen as uint32 [G*3][O/32][128] (a
// 512-byte run per 32 rows, plane and group); one box is `box_runs` (group, plane) runs of
// `box_units` 32-row units.  Encoding is pure host work; descriptors are cached per
// (address, O, G, box).  Returns false after recording the error.
bool plane_tensor_map(const uint8_t* planes, int O, int G, int box_units, int box_runs, CUtensorMap* out);
// Descriptor of a per-(group, row) tensor [G][O] of 1- or 2-byte elements (zero points, scales),
// box = 32 rows x 2 groups; rows of the box beyond G read as zero.
bool group_row_tensor_map(const void* base, int elem_bytes, int O, int G, CUtensorMap* out);

// Launch with the programmatic-dependent-launch attribute (unless switched off): the kernel's
// prologue may overlap the tail of the previous kernel in the stream.
template <class Kernel, class... Args>
int launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const char* what, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl_allowed() ? 1 : 0;
  cudaError_t err = cudaLaunchKernelEx(&config, kernel, args...);
  if (err != cudaSuccess) return cuda_fail(err, what);
  return FB_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline bool overlaps(const void* a, size_t na, const void* b, size_t nb) {
  auto pa = reinterpret_cast<uintptr_t>(a), pb = reinterpret_cast<uintptr_t>(b);
  return pa < pb + nb && pb < pa + na;
}

// ---- device side ------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float load_act(const void* base, int dtype, int index) {
  if (dtype == FB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[index]);
  return __half2float(reinterpret_cast<const __half*>(base)[index]);
}

__device__ __forceinline__ float bits_to_float(unsigned short bits, int dtype) {
  if (dtype == FB_BF16) return __uint_as_float(static_cast<unsigned>(bits) << 16);
  return __half2float(__ushort_as_half(bits));
}

// v rounded to the 16-bit dtype and widened again
__device__ __forceinline__ float round_to(float v, int dtype) {
  if (dtype == FB_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ void store_act(void* base, int dtype, int index, float value) {
  if (dtype == FB_BF16)
    reinterpret_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(value);
  else
    reinterpret_cast<__half*>(base)[index] = __float2half_rn(value);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(20000u)  // let the hardware park the thread for up to ~20 us per try
      : "memory");
  return done != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits for the barrier phase; gives up after about two seconds and returns false.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - start > 2000000000ull) return false;
  }
}

// Untiled bulk copy global -> this CTA's shared memory, completion counted on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
#endif  // __CUDACC__

}  // namespace fb
