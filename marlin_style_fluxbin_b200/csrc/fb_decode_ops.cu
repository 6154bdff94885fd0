// Small fused kernels of one decode step (one token), the glue between the packed GEMVs:
//   fb_qknorm_rope_cache  per-head RMSNorm of q and k, rotary embedding, and the write of the new
//                         k / v into the static KV cache, in one launch
//   fb_attn_decode        single-query attention over the cached positions (grouped-query heads)
//   fb_silu_mul           SwiGLU gate: out = silu(gate) * up
// The reference leaves these steps to stock HF modules (static_decode.py:43-76); after the Linears
// shrink by 5x they dominate the step, so each becomes one launch here.  All are launched with
// programmatic dependent launch and let the next kernel start its prologue at once.
#include <mutex>

#include "fb_common.cuh"

namespace {

using namespace fb;

__device__ __forceinline__ unsigned short to_bits(float v, int dtype) {
  return dtype == FB_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// One warp per head (q heads first, then k heads, then v heads which are only copied).
// Arithmetic per head follows the stock modules: RMSNorm (fp32 statistics, cast, weight), then
// out = T(T(v*cos) + rotate_half(v)*sin).
__global__ void qknorm_rope_cache_kernel(const unsigned short* __restrict__ q, const unsigned short* __restrict__ k,
                                         const unsigned short* __restrict__ v, const unsigned short* __restrict__ q_weight,
                                         const unsigned short* __restrict__ k_weight, const unsigned short* __restrict__ cosv,
                                         const unsigned short* __restrict__ sinv, unsigned short* __restrict__ q_out,
                                         unsigned short* __restrict__ k_cache, unsigned short* __restrict__ v_cache,
                                         int q_heads, int kv_heads, int dim, int position, int max_positions, float eps,
                                         int dtype) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x & 31;
  if (head >= q_heads + 2 * kv_heads) return;
  if (head >= q_heads + kv_heads) {  // v: straight into the cache
    const int hv = head - q_heads - kv_heads;
    for (int i = lane; i < dim; i += 32) v_cache[((size_t)hv * max_positions + position) * dim + i] = v[(size_t)hv * dim + i];
    return;
  }
  const bool is_q = head < q_heads;
  const unsigned short* src = is_q ? q + (size_t)head * dim : k + (size_t)(head - q_heads) * dim;
  const unsigned short* weight = is_q ? q_weight : k_weight;
  unsigned short* dst = is_q ? q_out + (size_t)head * dim : k_cache + ((size_t)(head - q_heads) * max_positions + position) * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float x = bits_to_float(src[i], dtype);
    ss += x * x;
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  const float inv = rsqrtf(ss / (float)dim + eps);
  const int half = dim / 2;
  for (int i = lane; i < half; i += 32) {
    const float lo = bits_to_float(weight[i], dtype) * round_to(bits_to_float(src[i], dtype) * inv, dtype);
    const float hi = bits_to_float(weight[i + half], dtype) * round_to(bits_to_float(src[i + half], dtype) * inv, dtype);
    const float nlo = round_to(lo, dtype), nhi = round_to(hi, dtype);  // the normed head, as stored
    const float y0 = round_to(nlo * bits_to_float(cosv[i], dtype), dtype) + (-nhi) * bits_to_float(sinv[i], dtype);
    const float y1 = round_to(nhi * bits_to_float(cosv[i + half], dtype), dtype) + nlo * bits_to_float(sinv[i + half], dtype);
    dst[i] = to_bits(y0, dtype);
    dst[i + half] = to_bits(y1, dtype);
  }
}

// Single-query attention, split over the cached positions: grid (query heads, splits); a CTA
// of 8 warps takes one contiguous chunk of positions, each warp ten positions at a time (all
// their loads issued before any use) with an online softmax.  The CTAs of a head form a
// thread-block cluster: each stores its (max, sum, output) into the first CTA's shared memory,
// one cluster barrier later that CTA merges the splits in ascending order.  (The variant
// without clusters keeps the scratch slots and the ticket; it runs when there is one split.)
// head_dim 128: a lane holds four consecutive dims.
constexpr int kAttnWarps = 8;
constexpr int kAttnMaxSplits = 16;
constexpr int kAttnBatch = 10;  // positions per warp with all their loads in flight: 80 per CTA and round
constexpr int kAttnSlot = 132;  // 128 outputs + max + sum, padded

__device__ __forceinline__ void unpack4(uint2 raw, int dtype, float* f) {
  f[0] = bits_to_float((unsigned short)(raw.x & 0xffff), dtype);
  f[1] = bits_to_float((unsigned short)(raw.x >> 16), dtype);
  f[2] = bits_to_float((unsigned short)(raw.y & 0xffff), dtype);
  f[3] = bits_to_float((unsigned short)(raw.y >> 16), dtype);
}

// What the fused form needs besides the attention arguments: the raw q/k/v rows of the new
// token (outputs of the q/k/v GEMV), the per-head norm weights and this position's rotary row.
struct NewToken {
  const unsigned short *q, *k, *v, *q_weight, *k_weight, *cosv, *sinv;
  float eps;
};

// Per-head RMSNorm + rotary embedding of one 128-wide head by one warp, result (in the 16-bit
// dtype's bits) into shared memory; the arithmetic of qknorm_rope_cache_kernel.  A lane owns the
// dims lane, lane + 32 and their partners + 64.  The constants (norm weight, rotary row) never
// change during a decode and are loaded separately, ahead of the wait on the preceding launch.
struct HeadConstants {
  float w[4], c[4], s[4];  // dims lane, lane + 32, lane + 64, lane + 96
};

__device__ __forceinline__ HeadConstants load_head_constants(const unsigned short* weight, const unsigned short* cosv,
                                                             const unsigned short* sinv, int dtype, int lane) {
  HeadConstants k;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    k.w[j] = bits_to_float(weight[lane + 32 * j], dtype);
    k.c[j] = bits_to_float(cosv[lane + 32 * j], dtype);
    k.s[j] = bits_to_float(sinv[lane + 32 * j], dtype);
  }
  return k;
}

__device__ __forceinline__ void norm_rope_head(const unsigned short* src, const HeadConstants& k, float eps, int dtype, int lane,
                                               unsigned short* dst) {
  constexpr int dim = 128;
  float x[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) x[j] = bits_to_float(src[lane + 32 * j], dtype);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  const float inv = rsqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float lo = k.w[j] * round_to(x[j] * inv, dtype);
    const float hi = k.w[j + 2] * round_to(x[j + 2] * inv, dtype);
    const float nlo = round_to(lo, dtype), nhi = round_to(hi, dtype);
    const float y0 = round_to(nlo * k.c[j], dtype) + (-nhi) * k.s[j];
    const float y1 = round_to(nhi * k.c[j + 2], dtype) + nlo * k.s[j + 2];
    dst[lane + 32 * j] = to_bits(y0, dtype);
    dst[lane + 32 * j + 64] = to_bits(y1, dtype);
  }
}

// FUSED: q arrives raw; the kernel norms and rotates q and the new k itself (every CTA of a head
// repeats that small piece of work), takes the new token's k / v from shared memory instead of
// the cache, and one CTA per k/v head writes them into the cache for the steps to come.
// PARTIAL: every CTA leaves its (output, max, sum) in its scratch slot and the launch ends there;
// the consumer of the attention output (fb_w3_gemv_attn_merge) merges the splits while it builds
// its tables, with the arithmetic of the merge below.  No cluster, no barrier, no ticket.
template <bool FUSED, bool CLUSTER, bool PARTIAL = false>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_kernel(const unsigned short* __restrict__ q,
                                                                      unsigned short* __restrict__ k_cache,
                                                                      unsigned short* __restrict__ v_cache,
                                                                      unsigned short* __restrict__ out, float* __restrict__ scratch,
                                                                      unsigned* __restrict__ tickets, int q_heads, int kv_heads,
                                                                      int length, int max_positions, float scale, int dtype,
                                                                      const NewToken nt) {
  constexpr int D = 128;
  const int head = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = q_heads / kv_heads, kvh = head / group;
  const unsigned short* kbase = k_cache + (size_t)kvh * max_positions * D + lane * 4;
  const unsigned short* vbase = v_cache + (size_t)kvh * max_positions * D + lane * 4;
  const int chunk = (length + splits - 1) / splits;
  const int p0 = split * chunk, p1 = min(length, p0 + chunk);
  const int newest = length - 1;  // FUSED: the token being decoded, not in the cache yet
  // a CTA's shared memory may be written by the others of its cluster only once it is running:
  // every thread arrives here and waits just before the exchange, far from the critical path
  if (CLUSTER) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  __shared__ __align__(8) unsigned short sm_new[3][D];  // rotated q, rotated k, v of the new token
  // A warp takes kAttnBatch positions at a time with all their loads in flight; the first batch
  // is requested before the q/k prologue so that the two round trips overlap.
  uint2 kr[kAttnBatch], vr[kAttnBatch];
  auto fetch = [&](int base) {
#pragma unroll
    for (int j = 0; j < kAttnBatch; ++j) {
      const int pos = min(base + j, p1 - 1);
      if (base < p1 && !(FUSED && pos == newest)) {
        kr[j] = *reinterpret_cast<const uint2*>(kbase + (size_t)pos * D);
        vr[j] = *reinterpret_cast<const uint2*>(vbase + (size_t)pos * D);
      } else {
        kr[j] = vr[j] = make_uint2(0u, 0u);
      }
    }
  };
  // FUSED: the cache rows of EARLIER positions are requested before the wait on the preceding
  // launch, so that their HBM round trip overlaps that launch's tail.  This is ordered because
  // this kernel (like the LM-head kernel) releases its own dependents only after its wait: when a
  // launch that follows one of them starts, everything before that one has completed, so the rows
  // written by the attention launches of earlier steps are in place as soon as one such launch
  // (or any launch without programmatic dependency) lies between the writer and this kernel.
  // The unfused form reads the newest row, written by the launch just before it, and must wait first.
  HeadConstants hc = {};
  if (FUSED) {
    if (warp < 2) hc = load_head_constants(warp == 0 ? nt.q_weight : nt.k_weight, nt.cosv, nt.sinv, dtype, lane);  // constants of the decode
    fetch(p0 + warp * kAttnBatch);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!FUSED) fetch(p0 + warp * kAttnBatch);
  float qv[4];
  if (FUSED) {
    if (warp == 0) norm_rope_head(nt.q + (size_t)head * D, hc, nt.eps, dtype, lane, sm_new[0]);
    if (warp == 1) norm_rope_head(nt.k + (size_t)kvh * D, hc, nt.eps, dtype, lane, sm_new[1]);
    if (warp == 2) *reinterpret_cast<uint2*>(&sm_new[2][lane * 4]) = *reinterpret_cast<const uint2*>(nt.v + (size_t)kvh * D + lane * 4);
    __syncthreads();
    if (head % group == 0 && split == splits - 1 && warp < 2) {  // the cache row of the new token
      unsigned short* row = (warp == 0 ? k_cache : v_cache) + ((size_t)kvh * max_positions + newest) * D;
      *reinterpret_cast<uint2*>(row + lane * 4) = *reinterpret_cast<const uint2*>(&sm_new[1 + warp][lane * 4]);
    }
    unpack4(*reinterpret_cast<const uint2*>(&sm_new[0][lane * 4]), dtype, qv);
  } else {
    unpack4(*reinterpret_cast<const uint2*>(q + (size_t)head * D + lane * 4), dtype, qv);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) qv[i] *= scale;
  float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int base = p0 + warp * kAttnBatch; base < p1; base += kAttnWarps * kAttnBatch) {
    if (base != p0 + warp * kAttnBatch) fetch(base);
    if (FUSED) {
#pragma unroll
      for (int j = 0; j < kAttnBatch; ++j)
        if (min(base + j, p1 - 1) == newest) {
          kr[j] = *reinterpret_cast<const uint2*>(&sm_new[1][lane * 4]);
          vr[j] = *reinterpret_cast<const uint2*>(&sm_new[2][lane * 4]);
        }
    }
    float s[kAttnBatch];
#pragma unroll
    for (int j = 0; j < kAttnBatch; ++j) {
      float kf[4];
      unpack4(kr[j], dtype, kf);
      s[j] = qv[0] * kf[0] + qv[1] * kf[1] + qv[2] * kf[2] + qv[3] * kf[3];
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
#pragma unroll
      for (int j = 0; j < kAttnBatch; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], d);
    }
    // Online softmax a batch at a time: the batch's maximum first, then every exponential and
    // product independently (no chain through the running maximum from position to position).
    float batch_max = -INFINITY;
#pragma unroll
    for (int j = 0; j < kAttnBatch; ++j)
      if (base + j < p1) batch_max = fmaxf(batch_max, s[j]);
    const float m_new = fmaxf(m, batch_max);
    const float correction = __expf(m - m_new);
    float psum = 0.f, pv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < kAttnBatch; ++j) {
      const float pj = base + j < p1 ? __expf(s[j] - m_new) : 0.f;
      float vf[4];
      unpack4(vr[j], dtype, vf);
      psum += pj;
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] += pj * vf[i];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = acc[i] * correction + pv[i];
    l = l * correction + psum;
    m = m_new;
  }
  __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps], sm_acc[kAttnWarps][D];
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) sm_acc[warp][lane * 4 + i] = acc[i];
  __syncthreads();
  // CLUSTER: the CTAs of one head form a thread-block cluster; every CTA stores its (output, max,
  // sum) into the first CTA's shared memory and one cluster barrier hands them over, instead of
  // a global scratch slot, a fence, a ticket and a round of loads.
  __shared__ __align__(16) float cl_part[CLUSTER ? kAttnMaxSplits : 1][kAttnSlot];
  if (CLUSTER) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // all CTAs of the head have started
  float* slot = scratch + ((size_t)head * kAttnMaxSplits + split) * kAttnSlot;
  float my_m = -INFINITY, my_l = 0.f;
  float4 part[kAttnMaxSplits];
  if (warp == 0) {
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) gm = fmaxf(gm, sm_m[w]);
    float total = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - gm);
      total = fmaf(sm_l[w], f, total);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = fmaf(sm_acc[w][lane * 4 + i], f, o[i]);
    }
    if (PARTIAL) {
      *reinterpret_cast<float4*>(slot + lane * 4) = make_float4(o[0], o[1], o[2], o[3]);
      if (lane == 0) *reinterpret_cast<float2*>(slot + 128) = make_float2(gm, total);
      return;
    }
    if (!CLUSTER && splits == 1) {  // nothing to merge: no scratch round trip
      const float inv1 = 1.f / total;
      uint2 direct;
      direct.x = (uint32_t)to_bits(o[0] * inv1, dtype) | ((uint32_t)to_bits(o[1] * inv1, dtype) << 16);
      direct.y = (uint32_t)to_bits(o[2] * inv1, dtype) | ((uint32_t)to_bits(o[3] * inv1, dtype) << 16);
      *reinterpret_cast<uint2*>(out + (size_t)head * D + lane * 4) = direct;
      return;
    }
    if (CLUSTER) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(&cl_part[split][0])), "r"(0));
      asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + lane * 16), "f"(o[0]), "f"(o[1]), "f"(o[2]), "f"(o[3]) : "memory");
      if (lane == 0) {
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 512), "f"(gm) : "memory");
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 516), "f"(total) : "memory");
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) slot[lane * 4 + i] = o[i];
      if (lane == 0) {
        slot[128] = gm;
        slot[129] = total;
      }
      __threadfence();
      __syncwarp();
      unsigned prior = 0;
      if (lane == 0) prior = atomicAdd(&tickets[head], 1u);
      prior = __shfl_sync(0xffffffffu, prior, 0);
      if (prior != (unsigned)splits - 1u) return;
      __threadfence();
    }
  } else if (!CLUSTER) {
    return;
  }
  if (CLUSTER) {
    // every thread of every CTA of the cluster arrives: release the stores above, acquire the others'
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (split != 0 || warp != 0) return;
    my_m = lane < splits ? cl_part[lane][128] : -INFINITY;
    my_l = lane < splits ? cl_part[lane][129] : 0.f;
#pragma unroll
    for (int sp = 0; sp < kAttnMaxSplits; ++sp)
      part[sp] = sp < splits ? *reinterpret_cast<const float4*>(&cl_part[sp][lane * 4]) : make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    // Merge of the splits by one warp with every load in flight at once: lane sp fetches the
    // (max, sum) of split sp, the rescaling factors come from shuffles, and each lane fetches its
    // four output dims of all splits before the first use.  Sums run in ascending split order.
    const float* base_slot = scratch + (size_t)head * kAttnMaxSplits * kAttnSlot;
    my_m = lane < splits ? __ldcg(base_slot + lane * kAttnSlot + 128) : -INFINITY;
    my_l = lane < splits ? __ldcg(base_slot + lane * kAttnSlot + 129) : 0.f;
#pragma unroll
    for (int sp = 0; sp < kAttnMaxSplits; ++sp)
      part[sp] = sp < splits ? __ldcg(reinterpret_cast<const float4*>(base_slot + sp * kAttnSlot + lane * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float gm = my_m;
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, d));
  const float my_f = my_m == -INFINITY ? 0.f : __expf(my_m - gm);
  float total = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int sp = 0; sp < kAttnMaxSplits; ++sp) {
    // explicit fused multiply-adds: fb_w3_gemv_attn_merge repeats this merge and must round alike
    const float f = __shfl_sync(0xffffffffu, my_f, sp);
    total = fmaf(__shfl_sync(0xffffffffu, my_l, sp), f, total);
    o[0] = fmaf(part[sp].x, f, o[0]);
    o[1] = fmaf(part[sp].y, f, o[1]);
    o[2] = fmaf(part[sp].z, f, o[2]);
    o[3] = fmaf(part[sp].w, f, o[3]);
  }
  const float inv = 1.f / total;
  uint2 packed;
  packed.x = (uint32_t)to_bits(o[0] * inv, dtype) | ((uint32_t)to_bits(o[1] * inv, dtype) << 16);
  packed.y = (uint32_t)to_bits(o[2] * inv, dtype) | ((uint32_t)to_bits(o[3] * inv, dtype) << 16);
  *reinterpret_cast<uint2*>(out + (size_t)head * D + lane * 4) = packed;
  if (!CLUSTER && lane == 0) tickets[head] = 0u;
}

__global__ void silu_mul_kernel(const unsigned short* __restrict__ gate, const unsigned short* __restrict__ up,
                                unsigned short* __restrict__ out, int n, int dtype) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = bits_to_float(gate[i], dtype);
  const float s = round_to(g / (1.f + __expf(-g)), dtype);  // silu in the activation dtype, as torch does
  out[i] = to_bits(s * bits_to_float(up[i], dtype), dtype);
}

// Receiving half of the tensor-parallel push: every rank's GEMV stores {fp32 value, mark = 1} as
// ONE 64-bit store into this rank's exchange buffer [world][n] (a scalar 8-byte access is
// single-copy atomic, so the mark never becomes visible without its value).  A thread polls the
// `world` slots of its element until all carry the mark (bounded by `wait_ns`), sums the values
// in ascending rank order (the same on every rank), and clears the slots for the next use: no
// fence, no counter, no collective call.  A rank cannot write a slot again before it has received
// this rank's NEXT contribution, which this rank sends only after this kernel: the clear is safe.
// On expiry the status word is set to 4; the slots are cleared all the same, so the buffer is
// clean for the next use once the late stores (if any) have been dealt with by the host.
__global__ void tp_reduce_kernel(unsigned long long* parts, int world, const unsigned short* __restrict__ residual,
                                 unsigned short* __restrict__ out, int n, int dtype, unsigned* status, unsigned long long wait_ns) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long start = global_timer_ns();
  float total = 0.f;
  bool expired = false;
  for (int r = 0; r < world; ++r) {
    unsigned long long* slot = parts + (size_t)r * n + i;
    unsigned long long got;
    for (;;) {
      asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(got) : "l"(slot) : "memory");
      if ((unsigned)(got >> 32) == 1u) break;
      if (expired || global_timer_ns() - start > wait_ns) {
        expired = true;
        break;
      }
    }
    total += __uint_as_float((unsigned)got);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(slot), "l"(0ull) : "memory");
  }
  if (expired) atomicExch(status, 4u);
  float value = round_to(total, dtype);
  if (residual) value += bits_to_float(residual[i], dtype);
  out[i] = to_bits(value, dtype);
}

// Up to 80 positions per CTA (one round of loads), the split count a power of two and at most 8:
// the CTAs of a head form a thread-block cluster, and clusters beyond the portable size of 8
// measured slower than the longer walk they would save.
inline int attention_splits(int length) {
  int splits = 1;
  while (splits < 8 && splits * 80 < length) splits *= 2;
  return splits;
}

// Attention launch: with more than one split the CTAs of a head (grid.y of them) form one
// thread-block cluster, which merges the splits in distributed shared memory.  Clusters of more
// than 8 CTAs need the non-portable size attribute, set once per kernel and device.
template <class Kernel, class... Args>
int launch_attention(Kernel kernel, Kernel cluster_kernel, dim3 grid, cudaStream_t stream, const char* what, Args... args) {
  if (grid.y == 1) return launch_pdl(kernel, grid, dim3(kAttnWarps * 32), 0, stream, what, args...);
  if (grid.y > 8) {  // per kernel and device; the two kernels share this function's instantiation
    static std::mutex lock;
    static const void* done[64][4] = {};
    int device = 0;
    cudaGetDevice(&device);
    std::lock_guard<std::mutex> guard(lock);
    bool ready = false;
    if (device >= 0 && device < 64)
      for (const void* seen : done[device]) ready = ready || seen == reinterpret_cast<const void*>(cluster_kernel);
    if (!ready) {
      cudaError_t err = cudaFuncSetAttribute(cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(non-portable cluster size)");
      if (device >= 0 && device < 64)
        for (const void*& seen : done[device])
          if (!seen) {
            seen = reinterpret_cast<const void*>(cluster_kernel);
            break;
          }
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(kAttnWarps * 32);
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = grid.y;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl_allowed() ? 2 : 1;
  cudaError_t err = cudaLaunchKernelEx(&config, cluster_kernel, args...);
  if (err != cudaSuccess) return cuda_fail(err, what);
  return FB_OK;
}

inline const unsigned short* u16(const void* p) { return static_cast<const unsigned short*>(p); }
inline unsigned short* u16(void* p) { return static_cast<unsigned short*>(p); }

}  // namespace

extern "C" int fb_qknorm_rope_cache(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                                    const void* cosv, const void* sinv, void* q_out, void* k_cache, void* v_cache, int q_heads,
                                    int kv_heads, int head_dim, int position, int max_positions, float eps, int dtype,
                                    fb_stream_t stream) {
  if (!q || !k || !v || !q_weight || !k_weight || !cosv || !sinv || !q_out || !k_cache || !v_cache) return fail(FB_EINVAL, "fb_qknorm_rope_cache: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_qknorm_rope_cache: dtype must be FB_F16 or FB_BF16");
  if (q_heads < 1 || kv_heads < 1 || head_dim < 2 || head_dim % 2 || head_dim > 1024) return fail(FB_ELIMIT, "fb_qknorm_rope_cache: head geometry outside bounds");
  if (position < 0 || position >= max_positions) return fail(FB_ELIMIT, "fb_qknorm_rope_cache: position %d outside the cache of %d", position, max_positions);
  const int heads = q_heads + 2 * kv_heads;
  return launch_pdl(qknorm_rope_cache_kernel, dim3((heads + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream), "qknorm_rope_cache launch",
                    u16(q), u16(k), u16(v), u16(q_weight), u16(k_weight), u16(cosv), u16(sinv), u16(q_out), u16(k_cache), u16(v_cache),
                    q_heads, kv_heads, head_dim, position, max_positions, eps, dtype);
}

extern "C" size_t fb_attn_decode_scratch_bytes(int q_heads) {
  if (q_heads < 1) return 0;
  return (size_t)q_heads * kAttnMaxSplits * kAttnSlot * sizeof(float) + (size_t)q_heads * sizeof(unsigned);
}

extern "C" int fb_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, int q_heads, int kv_heads,
                              int head_dim, int length, int max_positions, float scale, int dtype, void* scratch,
                              size_t scratch_bytes, fb_stream_t stream) {
  if (!q || !k_cache || !v_cache || !out) return fail(FB_EINVAL, "fb_attn_decode: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_attn_decode: dtype must be FB_F16 or FB_BF16");
  if (head_dim != 128) return fail(FB_ELIMIT, "fb_attn_decode: head_dim must be 128");
  if (q_heads < 1 || kv_heads < 1 || q_heads % kv_heads) return fail(FB_ELIMIT, "fb_attn_decode: q_heads must be a multiple of kv_heads");
  if (length < 1 || length > max_positions) return fail(FB_ELIMIT, "fb_attn_decode: length %d outside 1..%d", length, max_positions);
  if (!aligned(q, 8) || !aligned(k_cache, 8) || !aligned(v_cache, 8) || !aligned(out, 8)) return fail(FB_EINVAL, "fb_attn_decode: tensors must be 8-byte aligned");
  const size_t need = fb_attn_decode_scratch_bytes(q_heads);
  if (!scratch || scratch_bytes < need || !aligned(scratch, 16)) return fail(FB_ESCRATCH, "fb_attn_decode: 16-byte aligned scratch of %zu bytes needed", need);
  const int splits = attention_splits(length);
  float* partial = static_cast<float*>(scratch);
  unsigned* tickets = reinterpret_cast<unsigned*>(partial + (size_t)q_heads * kAttnMaxSplits * kAttnSlot);
  return launch_attention(attn_decode_kernel<false, false>, attn_decode_kernel<false, true>, dim3(q_heads, splits), static_cast<cudaStream_t>(stream), "attn_decode launch",
                    u16(q), const_cast<unsigned short*>(u16(k_cache)), const_cast<unsigned short*>(u16(v_cache)), u16(out), partial, tickets,
                    q_heads, kv_heads, length, max_positions, scale, dtype, NewToken{});
}

extern "C" int fb_attn_decode_fused(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                                    const void* cosv, const void* sinv, void* k_cache, void* v_cache, void* out, int q_heads,
                                    int kv_heads, int head_dim, int position, int max_positions, float eps, float scale, int dtype,
                                    void* scratch, size_t scratch_bytes, fb_stream_t stream) {
  if (!q || !k || !v || !q_weight || !k_weight || !cosv || !sinv || !k_cache || !v_cache || !out) return fail(FB_EINVAL, "fb_attn_decode_fused: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_attn_decode_fused: dtype must be FB_F16 or FB_BF16");
  if (head_dim != 128) return fail(FB_ELIMIT, "fb_attn_decode_fused: head_dim must be 128");
  if (q_heads < 1 || kv_heads < 1 || q_heads % kv_heads) return fail(FB_ELIMIT, "fb_attn_decode_fused: q_heads must be a multiple of kv_heads");
  if (position < 0 || position >= max_positions) return fail(FB_ELIMIT, "fb_attn_decode_fused: position %d outside the cache of %d", position, max_positions);
  if (!aligned(q, 8) || !aligned(k, 8) || !aligned(v, 8) || !aligned(k_cache, 8) || !aligned(v_cache, 8) || !aligned(out, 8))
    return fail(FB_EINVAL, "fb_attn_decode_fused: tensors must be 8-byte aligned");
  const size_t need = fb_attn_decode_scratch_bytes(q_heads);
  if (!scratch || scratch_bytes < need || !aligned(scratch, 16)) return fail(FB_ESCRATCH, "fb_attn_decode_fused: 16-byte aligned scratch of %zu bytes needed", need);
  const int length = position + 1;
  const int splits = attention_splits(length);
  float* partial = static_cast<float*>(scratch);
  unsigned* tickets = reinterpret_cast<unsigned*>(partial + (size_t)q_heads * kAttnMaxSplits * kAttnSlot);
  const NewToken nt = {u16(q), u16(k), u16(v), u16(q_weight), u16(k_weight), u16(cosv), u16(sinv), eps};
  return launch_attention(attn_decode_kernel<true, false>, attn_decode_kernel<true, true>, dim3(q_heads, splits), static_cast<cudaStream_t>(stream), "attn_decode_fused launch",
                    static_cast<const unsigned short*>(nullptr), u16(k_cache), u16(v_cache), u16(out), partial, tickets, q_heads, kv_heads, length,
                    max_positions, scale, dtype, nt);
}

extern "C" int fb_attn_decode_splits(int length) { return length < 1 ? 0 : attention_splits(length); }

extern "C" int fb_attn_decode_partial(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                                      const void* cosv, const void* sinv, void* k_cache, void* v_cache, int q_heads, int kv_heads,
                                      int head_dim, int position, int max_positions, float eps, float scale, int dtype,
                                      void* partials, size_t partial_bytes, fb_stream_t stream) {
  if (!q || !k || !v || !q_weight || !k_weight || !cosv || !sinv || !k_cache || !v_cache) return fail(FB_EINVAL, "fb_attn_decode_partial: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_attn_decode_partial: dtype must be FB_F16 or FB_BF16");
  if (head_dim != 128) return fail(FB_ELIMIT, "fb_attn_decode_partial: head_dim must be 128");
  if (q_heads < 1 || kv_heads < 1 || q_heads % kv_heads) return fail(FB_ELIMIT, "fb_attn_decode_partial: q_heads must be a multiple of kv_heads");
  if (position < 0 || position >= max_positions) return fail(FB_ELIMIT, "fb_attn_decode_partial: position %d outside the cache of %d", position, max_positions);
  if (!aligned(q, 8) || !aligned(k, 8) || !aligned(v, 8) || !aligned(k_cache, 8) || !aligned(v_cache, 8))
    return fail(FB_EINVAL, "fb_attn_decode_partial: tensors must be 8-byte aligned");
  const size_t need = fb_attn_decode_scratch_bytes(q_heads);
  if (!partials || partial_bytes < need || !aligned(partials, 16)) return fail(FB_ESCRATCH, "fb_attn_decode_partial: 16-byte aligned buffer of %zu bytes needed", need);
  const int length = position + 1;
  const NewToken nt = {u16(q), u16(k), u16(v), u16(q_weight), u16(k_weight), u16(cosv), u16(sinv), eps};
  return launch_pdl(attn_decode_kernel<true, false, true>, dim3(q_heads, attention_splits(length)), dim3(kAttnWarps * 32), 0,
                    static_cast<cudaStream_t>(stream), "attn_decode_partial launch", static_cast<const unsigned short*>(nullptr), u16(k_cache),
                    u16(v_cache), static_cast<unsigned short*>(nullptr), static_cast<float*>(partials), static_cast<unsigned*>(nullptr), q_heads,
                    kv_heads, length, max_positions, scale, dtype, nt);
}

extern "C" int fb_silu_mul(const void* gate, const void* up, void* out, int n, int dtype, fb_stream_t stream) {
  if (!gate || !up || !out) return fail(FB_EINVAL, "fb_silu_mul: null pointer");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_silu_mul: dtype must be FB_F16 or FB_BF16");
  if (n < 1) return fail(FB_ELIMIT, "fb_silu_mul: n must be positive");
  return launch_pdl(silu_mul_kernel, dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), "silu_mul launch",
                    u16(gate), u16(up), u16(out), n, dtype);
}

extern "C" int fb_tp_reduce(void* parts, int world, const void* residual, void* out, int n, int dtype, unsigned* status,
                            uint64_t wait_ns, fb_stream_t stream) {
  if (!parts || !out || !status) return fail(FB_EINVAL, "fb_tp_reduce: null pointer");
  if (!aligned(parts, 8)) return fail(FB_EINVAL, "fb_tp_reduce: the exchange buffer must be 8-byte aligned");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_tp_reduce: dtype must be FB_F16 or FB_BF16");
  if (world < 1 || world > 8 || n < 1) return fail(FB_ELIMIT, "fb_tp_reduce: world 1..8 and n >= 1");
  if (wait_ns > 60000000000ull) return fail(FB_ELIMIT, "fb_tp_reduce: wait limit above 60 s");
  const unsigned long long limit = wait_ns ? wait_ns : 10000000000ull;  // default ten seconds: ranks may be skewed by host work
  return launch_pdl(tp_reduce_kernel, dim3((n + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), "tp_reduce launch",
                    static_cast<unsigned long long*>(parts), world, u16(residual), u16(out), n, dtype, status, limit);
}
