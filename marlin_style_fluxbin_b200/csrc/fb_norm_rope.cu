// Fused RMSNorm and fused rotary embedding for the decode step (one token): each replaces a
// chain of small elementwise / reduction kernels with one launch.
//
// RMSNorm follows the stock Qwen3 arithmetic that the reference keeps
// (fused_modules.py:30-41): variance and normalisation in fp32, the result is cast to the
// 16-bit dtype BEFORE it is multiplied by the weight, and that product is rounded again.
// RoPE follows fused_modules.py:66-85: out = dtype(dtype(v*cos) + rotate_half(v)*sin) with
// rotate_half(v) = (-v[d/2:], v[:d/2]); q and k heads share one cos/sin row.
#include "fb_common.cuh"

namespace {

using namespace fb;

// One warp per row when LANES == 32, one 256-thread CTA per row otherwise.
template <int LANES>
__global__ void rmsnorm_kernel(const unsigned short* __restrict__ x, const unsigned short* __restrict__ weight,
                               unsigned short* __restrict__ out, int rows, int dim, float eps, int dtype) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int row = LANES == 32 ? (int)(blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32) : (int)blockIdx.x;
  const int t = LANES == 32 ? (int)(threadIdx.x & 31) : (int)threadIdx.x;
  if (row >= rows) return;
  const unsigned short* xr = x + (size_t)row * dim;
  float ss = 0.f;
  for (int i = t; i < dim; i += LANES) {
    const float v = bits_to_float(xr[i], dtype);
    ss += v * v;
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if (LANES > 32) {
    __shared__ float part[LANES / 32];
    if ((t & 31) == 0) part[t >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < LANES / 32; ++w) ss += part[w];
  }
  const float inv = rsqrtf(ss / (float)dim + eps);
  for (int i = t; i < dim; i += LANES) {
    const float normed = round_to(bits_to_float(xr[i], dtype) * inv, dtype);
    const float y = bits_to_float(weight[i], dtype) * normed;
    out[(size_t)row * dim + i] = dtype == FB_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y))
                                                  : __half_as_ushort(__float2half_rn(y));
  }
}

__global__ void rope_kernel(const unsigned short* __restrict__ q, const unsigned short* __restrict__ k,
                            const unsigned short* __restrict__ cosv, const unsigned short* __restrict__ sinv,
                            unsigned short* __restrict__ q_out, unsigned short* __restrict__ k_out,
                            int q_heads, int k_heads, int dim, int dtype) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int half = dim / 2;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (q_heads + k_heads) * half) return;
  const int head = idx / half, i = idx - head * half;
  const unsigned short* src = head < q_heads ? q + (size_t)head * dim : k + (size_t)(head - q_heads) * dim;
  unsigned short* dst = head < q_heads ? q_out + (size_t)head * dim : k_out + (size_t)(head - q_heads) * dim;
  const float lo = bits_to_float(src[i], dtype), hi = bits_to_float(src[i + half], dtype);
  const float c0 = bits_to_float(cosv[i], dtype), c1 = bits_to_float(cosv[i + half], dtype);
  const float s0 = bits_to_float(sinv[i], dtype), s1 = bits_to_float(sinv[i + half], dtype);
  // products of two 16-bit floats are exact in fp32, so mul+add equals torch's addcmul
  const float y0 = round_to(lo * c0, dtype) + (-hi) * s0;
  const float y1 = round_to(hi * c1, dtype) + lo * s1;
  dst[i] = dtype == FB_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y0)) : __half_as_ushort(__float2half_rn(y0));
  dst[i + half] = dtype == FB_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y1)) : __half_as_ushort(__float2half_rn(y1));
}

}  // namespace

extern "C" int fb_rmsnorm(const void* x, const void* weight, void* out, int rows, int dim, float eps, int dtype,
                          fb_stream_t stream) {
  if (!x || !weight || !out) return fail(FB_EINVAL, "fb_rmsnorm: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_rmsnorm: dtype must be FB_F16 or FB_BF16");
  if (rows < 1 || dim < 1 || dim > 65536 || rows > (1 << 24)) return fail(FB_ELIMIT, "fb_rmsnorm: rows=%d dim=%d outside bounds", rows, dim);
  if (!(eps >= 0.f)) return fail(FB_EINVAL, "fb_rmsnorm: eps must be non-negative");
  auto xs = static_cast<const unsigned short*>(x);
  auto ws = static_cast<const unsigned short*>(weight);
  auto os = static_cast<unsigned short*>(out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dim <= 512) {
    const int rows_per_block = 4;
    return launch_pdl(rmsnorm_kernel<32>, dim3((rows + rows_per_block - 1) / rows_per_block), dim3(32 * rows_per_block), 0, s,
                      "rmsnorm_kernel launch", xs, ws, os, rows, dim, eps, dtype);
  }
  return launch_pdl(rmsnorm_kernel<256>, dim3(rows), dim3(256), 0, s, "rmsnorm_kernel launch", xs, ws, os, rows, dim, eps, dtype);
}

extern "C" int fb_rope_qk(const void* q, const void* k, const void* cosv, const void* sinv, void* q_out, void* k_out,
                          int q_heads, int k_heads, int head_dim, int dtype, fb_stream_t stream) {
  if (!q || !k || !cosv || !sinv || !q_out || !k_out) return fail(FB_EINVAL, "fb_rope_qk: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_rope_qk: dtype must be FB_F16 or FB_BF16");
  if (q_heads < 0 || k_heads < 0 || q_heads + k_heads < 1 || q_heads + k_heads > 65536 || head_dim < 2 || head_dim % 2 || head_dim > 1024)
    return fail(FB_ELIMIT, "fb_rope_qk: heads=%d+%d head_dim=%d outside bounds", q_heads, k_heads, head_dim);
  const int work = (q_heads + k_heads) * (head_dim / 2);
  return launch_pdl(rope_kernel, dim3((work + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), "rope_kernel launch",
                    static_cast<const unsigned short*>(q), static_cast<const unsigned short*>(k),
                    static_cast<const unsigned short*>(cosv), static_cast<const unsigned short*>(sinv),
                    static_cast<unsigned short*>(q_out), static_cast<unsigned short*>(k_out), q_heads, k_heads, head_dim, dtype);
}
