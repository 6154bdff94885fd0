// LM head of the decode step: logits = W . x over a dense 16-bit weight [V,K] with the greedy
// choice (argmax) taken in the same launch, and the small kernels around it.
//
// The reference keeps the LM head as a dense 16-bit Linear followed by torch.argmax and names it the
// next thing to optimise (docs/performance/NONLINEAR_FUSION.md:100).  At batch one it is pure HBM
// streaming: 1.245 GB for Qwen3's 151936 x 4096 head.  Here
//   * the final RMSNorm of the hidden state is applied while x is staged into shared memory (every
//     CTA norms the few KB itself, with the arithmetic and summation order of fb_rmsnorm);
//   * a warp owns whole rows: 16-byte loads, eight in flight per lane, fp32 accumulation, one
//     shuffle reduction per row;
//   * the logit is rounded to the 16-bit dtype (what a 16-bit Linear returns) and compared as an
//     order-preserving 64-bit key {rounded value, ~row}: ties go to the lowest row, as
//     torch.argmax resolves them; one atomicMax per CTA, and the CTA that arrives last publishes
//     the index, resets the two control words and (optionally) copies the embedding row of the
//     next token into the hidden-state buffer, so that the next step needs no gather launch;
//   * the 300 KB of logits are written only when the caller asks for them.
#include <mutex>

#include "fb_common.cuh"

namespace {

using namespace fb;

constexpr int kHeadThreads = 256;
constexpr int kHeadCtasPerSm = 3;

struct HeadParams {
  const unsigned short* x;        // [K] hidden state (before the final norm when norm_weight != null)
  const unsigned short* norm_weight;  // [K] or null
  const unsigned short* weight;   // [V,K]
  unsigned short* logits;         // [V] or null
  unsigned long long* state;      // [0] best key so far, [1] arrival ticket; both zero between launches
  long long* best;                // [1] the chosen row
  const long long* forced_next;   // optional: the token whose embedding row is copied (else the chosen row)
  const unsigned short* embedding;  // [V,K] or null
  unsigned short* next_hidden;    // [K] or null
  float eps;
  int V, K, dtype;
  // Vocabulary shard of a tensor-parallel rank: `weight` holds rows row_base .. row_base + V - 1 of the
  // whole matrix, keys carry the global row, and instead of publishing its choice the last CTA stores
  // the shard's best key into slot `push_rank` of every rank's key array (plain 8-byte peer stores).
  int row_base;
  unsigned long long* push_keys[8];
  int push_world, push_rank;
};

__device__ __forceinline__ unsigned ordered_bits(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <bool BF16>
__device__ __forceinline__ void widen8(const uint4& raw, float (&f)[8]) {
  const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (BF16) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    } else {
      const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      f[2 * j] = pair.x;
      f[2 * j + 1] = pair.y;
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(kHeadThreads, kHeadCtasPerSm) lm_head_kernel(const HeadParams p) {
  extern __shared__ __align__(16) float xs[];  // [K] the (normed) activations, widened
  __shared__ float part[kHeadThreads / 32];
  __shared__ unsigned long long warp_best[kHeadThreads / 32];
  __shared__ int is_last;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int dtype = BF16 ? FB_BF16 : FB_F16;

  const int warps_total = gridDim.x * (kHeadThreads / 32);
  int row = blockIdx.x * (kHeadThreads / 32) + warp;
  // The weights never change: the first row's loads go out before the wait on the previous kernel.
  constexpr int kInFlight = 8;
  const int steps = (p.K + 255) / 256;  // 256 elements (32 lanes x 16 bytes) per step
  uint4 ahead[kInFlight];
#pragma unroll
  for (int u = 0; u < kInFlight; ++u) {
    ahead[u] = make_uint4(0u, 0u, 0u, 0u);
    const int k0 = (u * 32 + lane) * 8;
    if (row < p.V && k0 < p.K) ahead[u] = __ldcs(reinterpret_cast<const uint4*>(p.weight + (size_t)row * p.K + k0));
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Dependents are released only after the wait: a launch that follows this one then starts with
  // everything before this one complete (the decode attention relies on that for its early reads
  // of the cache); nothing is lost, this kernel fills every SM until it ends.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- stage x (optionally RMS-normed, with fb_rmsnorm's summation order) ----
  float inv = 1.f;
  if (p.norm_weight) {
    float ss = 0.f;
    for (int i = t; i < p.K; i += kHeadThreads) {
      const float v = bits_to_float(p.x[i], dtype);
      ss += v * v;
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < kHeadThreads / 32; ++w) ss += part[w];
    inv = rsqrtf(ss / (float)p.K + p.eps);
  }
  for (int i = t; i < p.K; i += kHeadThreads) {
    float v = bits_to_float(p.x[i], dtype);
    if (p.norm_weight) v = round_to(bits_to_float(p.norm_weight[i], dtype) * round_to(v * inv, dtype), dtype);
    xs[i] = v;
  }
  __syncthreads();

  // ---- rows of this warp: row, row + warps_total, ... ----
  unsigned long long best_key = 0ull;
  for (; row < p.V; row += warps_total) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s0 = 0; s0 < steps; s0 += kInFlight) {
      // the batch after this one: the rest of this row, or the start of this warp's next row
      const bool same_row = s0 + kInFlight < steps;
      const int next_row = same_row ? row : row + warps_total;
      const int next_s0 = same_row ? s0 + kInFlight : 0;
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const uint4 cur = ahead[u];
        // refill this register set at once: eight 16-byte loads stay in flight per lane
        const int kn = ((next_s0 + u) * 32 + lane) * 8;
        ahead[u] = make_uint4(0u, 0u, 0u, 0u);
        if (next_row < p.V && kn < p.K) ahead[u] = __ldcs(reinterpret_cast<const uint4*>(p.weight + (size_t)next_row * p.K + kn));
        const int k0 = ((s0 + u) * 32 + lane) * 8;
        if (k0 < p.K) {
          float w8[8];
          widen8<BF16>(cur, w8);
          const float4 xa = *reinterpret_cast<const float4*>(xs + k0);
          const float4 xb = *reinterpret_cast<const float4*>(xs + k0 + 4);
          acc[0] = fmaf(w8[0], xa.x, acc[0]);
          acc[1] = fmaf(w8[1], xa.y, acc[1]);
          acc[2] = fmaf(w8[2], xa.z, acc[2]);
          acc[3] = fmaf(w8[3], xa.w, acc[3]);
          acc[0] = fmaf(w8[4], xb.x, acc[0]);
          acc[1] = fmaf(w8[5], xb.y, acc[1]);
          acc[2] = fmaf(w8[6], xb.z, acc[2]);
          acc[3] = fmaf(w8[7], xb.w, acc[3]);
        }
      }
    }
    float total = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
    const float logit = round_to(total, dtype);
    if (lane == 0 && p.logits) p.logits[row] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(total)) : __half_as_ushort(__float2half_rn(total));
    const unsigned long long key = ((unsigned long long)ordered_bits(logit) << 32) | (unsigned long long)(0xffffffffu - (unsigned)(p.row_base + row));
    best_key = key > best_key ? key : best_key;
  }

  // ---- merge: warps -> CTA -> one atomicMax; the last CTA publishes ----
  if (lane == 0) warp_best[warp] = best_key;
  __syncthreads();
  if (t == 0) {
    unsigned long long cta_best = 0ull;
#pragma unroll
    for (int w = 0; w < kHeadThreads / 32; ++w) cta_best = warp_best[w] > cta_best ? warp_best[w] : cta_best;
    atomicMax(&p.state[0], cta_best);
    __threadfence();
    const unsigned long long ticket = atomicAdd(&p.state[1], 1ull);
    is_last = ticket == (unsigned long long)(gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const unsigned long long final_key = *reinterpret_cast<volatile unsigned long long*>(&p.state[0]);
  if (p.push_world > 0) {  // a key is never zero (its low word is 2^32 - 1 - row), so a non-zero slot is a delivered one
    if (t < p.push_world) asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p.push_keys[t] + p.push_rank), "l"(final_key) : "memory");
    if (t == 0) {
      p.state[0] = 0ull;
      p.state[1] = 0ull;
    }
    return;
  }
  const long long chosen = (long long)(0xffffffffu - (unsigned)(final_key & 0xffffffffull));
  if (p.embedding && p.next_hidden) {
    const long long token = p.forced_next ? *p.forced_next : chosen;
    if (token >= 0 && token < p.V)
      for (int i = t; i < p.K; i += kHeadThreads) p.next_hidden[i] = p.embedding[(size_t)token * p.K + i];
  }
  if (t == 0) {
    *p.best = chosen;
    p.state[0] = 0ull;
    p.state[1] = 0ull;
  }
}

__global__ void embed_row_kernel(const unsigned short* __restrict__ embedding, const long long* __restrict__ token, unsigned short* __restrict__ out,
                                 int V, int K) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long row = *token;
  if (row < 0 || row >= V) return;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < K; i += gridDim.x * blockDim.x) out[i] = embedding[(size_t)row * K + i];
}

}  // namespace

extern "C" size_t fb_lm_head_scratch_bytes(void) { return 256; }

namespace {
int run_head(const void* x, const void* norm_weight, float eps, const void* weight, int vocab, int in_features, int dtype, void* logits,
             int64_t* best, const int64_t* forced_next, const void* embedding, void* next_hidden, void* scratch, size_t scratch_bytes,
             fb_stream_t stream, int row_base, const fb_w3_push_t* keys, int rank) {
  if (!x || !weight || !best) return fail(FB_EINVAL, "fb_lm_head_argmax: x, weight and best must be non-null");
  if (dtype != FB_F16 && dtype != FB_BF16) return fail(FB_EINVAL, "fb_lm_head_argmax: dtype must be FB_F16 or FB_BF16");
  if (vocab < 1 || vocab > (1 << 30) || in_features < 8 || in_features % 8 || in_features > 49152)
    return fail(FB_ELIMIT, "fb_lm_head_argmax: vocab=%d K=%d outside bounds (K a multiple of 8, at most 49152)", vocab, in_features);
  if (!aligned(weight, 16) || !aligned(x, 2) || !aligned(best, 8) || !aligned(logits, 2) || !aligned(norm_weight, 2) ||
      !aligned(embedding, 2) || !aligned(next_hidden, 2) || !aligned(forced_next, 8))
    return fail(FB_EINVAL, "fb_lm_head_argmax: weight must be 16-byte aligned, best 8-byte, 16-bit tensors 2-byte");
  if ((embedding == nullptr) != (next_hidden == nullptr)) return fail(FB_EINVAL, "fb_lm_head_argmax: embedding and next_hidden go together");
  if (!scratch || scratch_bytes < fb_lm_head_scratch_bytes() || !aligned(scratch, 16))
    return fail(FB_ESCRATCH, "fb_lm_head_argmax: 16-byte aligned scratch of %zu bytes needed", fb_lm_head_scratch_bytes());
  const size_t x_bytes = (size_t)in_features * 2;
  if (next_hidden && overlaps(next_hidden, x_bytes, weight, (size_t)vocab * in_features * 2))
    return fail(FB_EALIAS, "fb_lm_head_argmax: next_hidden overlaps the weight");
  const DeviceInfo* info = device_info();
  if (!info) return FB_ECUDA;
  HeadParams p;
  p.x = static_cast<const unsigned short*>(x);
  p.norm_weight = static_cast<const unsigned short*>(norm_weight);
  p.weight = static_cast<const unsigned short*>(weight);
  p.logits = static_cast<unsigned short*>(logits);
  p.state = static_cast<unsigned long long*>(scratch);
  p.best = reinterpret_cast<long long*>(best);
  p.forced_next = reinterpret_cast<const long long*>(forced_next);
  p.embedding = static_cast<const unsigned short*>(embedding);
  p.next_hidden = static_cast<unsigned short*>(next_hidden);
  p.eps = eps;
  p.V = vocab;
  p.K = in_features;
  p.dtype = dtype;
  p.row_base = row_base;
  p.push_world = keys ? keys->world : 0;
  p.push_rank = rank;
  for (int r = 0; r < 8; ++r) p.push_keys[r] = keys && r < keys->world ? static_cast<unsigned long long*>(keys->data[r]) : nullptr;
  const size_t smem = (size_t)in_features * sizeof(float);
  static std::mutex lock;
  static bool ready[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
  if (device < 0 || device >= 64) return fail(FB_ELIMIT, "device ordinal %d outside 0..63", device);
  {
    std::lock_guard<std::mutex> guard(lock);
    if (!ready[device]) {
      err = cudaFuncSetAttribute(lm_head_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152 * 4);
      if (err == cudaSuccess) err = cudaFuncSetAttribute(lm_head_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152 * 4);
      if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(lm_head_kernel)");
      ready[device] = true;
    }
  }
  int ctas = info->sm_count * kHeadCtasPerSm;
  const int by_rows = (vocab + kHeadThreads / 32 - 1) / (kHeadThreads / 32);
  if (ctas > by_rows) ctas = by_rows;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FB_BF16) return launch_pdl(lm_head_kernel<true>, dim3(ctas), dim3(kHeadThreads), smem, s, "lm_head_kernel launch", p);
  return launch_pdl(lm_head_kernel<false>, dim3(ctas), dim3(kHeadThreads), smem, s, "lm_head_kernel launch", p);
}
}  // namespace

extern "C" int fb_lm_head_argmax(const void* x, const void* norm_weight, float eps, const void* weight, int vocab, int in_features,
                                 int dtype, void* logits, int64_t* best, const int64_t* forced_next, const void* embedding,
                                 void* next_hidden, void* scratch, size_t scratch_bytes, fb_stream_t stream) {
  return run_head(x, norm_weight, eps, weight, vocab, in_features, dtype, logits, best, forced_next, embedding, next_hidden, scratch,
                  scratch_bytes, stream, 0, nullptr, 0);
}

namespace {
// Receiving half of the vocabulary-split LM head: one CTA polls the `world` keys that the ranks'
// shards delivered (bounded), takes the largest (ties: the lowest row, as torch.argmax), zeroes the
// slots, publishes the choice and copies the embedding row of the next token into the hidden state.
__global__ void __launch_bounds__(256) tp_argmax_kernel(unsigned long long* keys, int world, long long* best, const long long* forced_next,
                                                        const unsigned short* embedding, unsigned short* next_hidden, int V, int K,
                                                        unsigned* status, unsigned long long wait_ns) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // after the wait: see the attention kernel's ordering rule
  __shared__ unsigned long long chosen_key;
  const int t = threadIdx.x;
  if (t < 32) {
    unsigned long long key = 0ull;
    if (t < world) {
      const unsigned long long start = global_timer_ns();
      for (;;) {
        asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(key) : "l"(keys + t) : "memory");
        if (key != 0ull || global_timer_ns() - start > wait_ns) break;
      }
      if (key == 0ull) atomicExch(status, 6u);
      asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(keys + t), "l"(0ull) : "memory");
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, d);
      key = other > key ? other : key;
    }
    if (t == 0) chosen_key = key;
  }
  __syncthreads();
  const long long chosen = (long long)(0xffffffffu - (unsigned)(chosen_key & 0xffffffffull));
  if (embedding && next_hidden) {
    const long long token = forced_next ? *forced_next : chosen;
    if (token >= 0 && token < V)
      for (int i = t; i < K; i += 256) next_hidden[i] = embedding[(size_t)token * K + i];
  }
  if (t == 0) *best = chosen;
}
}  // namespace

extern "C" int fb_lm_head_shard(const void* x, const void* norm_weight, float eps, const void* weight, int vocab_rows, int row_base,
                                int in_features, int dtype, void* logits, const fb_w3_push_t* keys, int rank, void* scratch,
                                size_t scratch_bytes, fb_stream_t stream) {
  if (!keys || keys->world < 1 || keys->world > 8 || rank < 0 || rank >= keys->world)
    return fail(FB_EINVAL, "fb_lm_head_shard: key arrays of 1..8 ranks and a rank among them");
  for (int r = 0; r < keys->world; ++r)
    if (!keys->data[r] || !aligned(keys->data[r], 8)) return fail(FB_EINVAL, "fb_lm_head_shard: key array of rank %d missing or not 8-byte aligned", r);
  if (row_base < 0 || vocab_rows < 1 || (long long)row_base + vocab_rows > (1ll << 30)) return fail(FB_ELIMIT, "fb_lm_head_shard: rows outside 0..2^30");
  int64_t unused = 0;
  return run_head(x, norm_weight, eps, weight, vocab_rows, in_features, dtype, logits, &unused, nullptr, nullptr, nullptr, scratch, scratch_bytes,
                  stream, row_base, keys, rank);
}

extern "C" int fb_tp_argmax(void* keys, int world, int64_t* best, const int64_t* forced_next, const void* embedding, void* next_hidden,
                            int vocab, int in_features, unsigned* status, uint64_t wait_ns, fb_stream_t stream) {
  if (!keys || !best || !status) return fail(FB_EINVAL, "fb_tp_argmax: null pointer");
  if (world < 1 || world > 8) return fail(FB_ELIMIT, "fb_tp_argmax: world outside 1..8");
  if (!aligned(keys, 8) || !aligned(best, 8) || !aligned(forced_next, 8)) return fail(FB_EINVAL, "fb_tp_argmax: keys, best and forced_next must be 8-byte aligned");
  if ((embedding == nullptr) != (next_hidden == nullptr)) return fail(FB_EINVAL, "fb_tp_argmax: embedding and next_hidden go together");
  if (embedding && (vocab < 1 || in_features < 1)) return fail(FB_ELIMIT, "fb_tp_argmax: empty embedding table");
  if (wait_ns > 60000000000ull) return fail(FB_ELIMIT, "fb_tp_argmax: wait limit above 60 s");
  return launch_pdl(tp_argmax_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), "tp_argmax launch",
                    static_cast<unsigned long long*>(keys), world, reinterpret_cast<long long*>(best), reinterpret_cast<const long long*>(forced_next),
                    static_cast<const unsigned short*>(embedding), static_cast<unsigned short*>(next_hidden), vocab, in_features, status,
                    (unsigned long long)(wait_ns ? wait_ns : 10000000000ull));
}

extern "C" int fb_embed_row(const void* embedding, const int64_t* token, void* out, int vocab, int in_features, fb_stream_t stream) {
  if (!embedding || !token || !out) return fail(FB_EINVAL, "fb_embed_row: null pointer");
  if (vocab < 1 || in_features < 1) return fail(FB_ELIMIT, "fb_embed_row: empty table");
  if (!aligned(token, 8) || !aligned(embedding, 2) || !aligned(out, 2)) return fail(FB_EINVAL, "fb_embed_row: misaligned pointer");
  return launch_pdl(embed_row_kernel, dim3((in_features + 1023) / 1024), dim3(256), 0, static_cast<cudaStream_t>(stream), "embed_row_kernel launch",
                    static_cast<const unsigned short*>(embedding), reinterpret_cast<const long long*>(token), static_cast<unsigned short*>(out),
                    vocab, in_features);
}
