// W3 (GPTQ 3-bit, group 128, planar layout) small-batch GEMM for B200 (sm_100a):
//   y[M,O] = x[M,K] . W^T,  M = 1..16, on the fifth-generation tensor cores (tcgen05 + TMEM).
//
// Where the M = 1 kernel (fb_w3_gemv.cu) replaces multiplications by table lookups, whose cost
// grows with every extra activation row, this kernel dequantises each weight ONCE into a
// shared-memory operand tile and lets one tcgen05.mma apply it to all rows of the batch:
//   * a CTA owns 128 output rows and a contiguous range of K groups (split-K over CTAs);
//   * the three bit planes of (group, 128 rows) arrive by one tiled TMA copy (6 KB);
//   * 256 threads turn them into a 128 x 128 tile of 16-bit weights T((code - zero) * T(scale)):
//     a plane byte (8 inputs) indexes a 256-entry table that spreads its bits over the eight
//     nibbles of a word; the three planes' words add up to eight 3-bit codes, which one logic
//     instruction per pair drops into the mantissas of two 16-bit floats (1024 + code, or
//     128 + code for bf16); a packed subtract removes the bias and the zero point exactly and a
//     packed multiply applies the scale with its single rounding.  Tiles are written straight in
//     the K-major "core matrix" order that the MMA's shared-memory descriptor walks (8 rows x 16
//     bytes per core matrix, no swizzle): one 16-byte store per 8 weights;
//   * the activations of the group (M rows padded to N = 16) are stored the same way;
//   * warp-specialised: eight warps dequantise, the elected lane of a ninth issues the plane
//     copies and 8 x tcgen05.mma (128 x 16 x 16 each) per group, accumulating in 16 TMEM columns
//     over all groups of the CTA; tiles are double-buffered and the two sides meet on mbarriers
//     only (tile complete: 256 arrivals; buffer free: the MMAs' commit), never on a CTA barrier;
//   * the 128 x 16 fp32 result is read back with tcgen05.ld and either written (one split) or
//     combined across splits with the 64-bit fixed-point atomic of the M = 1 kernel.
// Every wait on an mbarrier is bounded; on expiry the CTA records a status, frees its TMEM
// columns and leaves.
//
// The weights still cross HBM exactly once, so the bound is the same as for M = 1; the reference
// has no packed path for M > 1 at all (csrc/w3_lut.cu:195 rejects it) and falls back to a dense
// matmul of the restored weight (w3_lut_deployment.py:343-359), which is the oracle here.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <type_traits>

#include "fb_common.cuh"

namespace {

using namespace fb;

constexpr int kTileRows = 128;
constexpr int kN = 16;            // activation rows presented to the MMA (M padded)
constexpr int kProducers = 256;       // eight warps that dequantise
constexpr int kThreads = kProducers + 32;  // and one warp whose elected lane issues the copies and the MMAs
constexpr int kATile = kTileRows * 128 * 2;  // 32 KB: 128 rows x 128 k, 16-bit
constexpr int kBTile = kN * 128 * 2;         // 4 KB
constexpr int kPlaneTile = 3 * kTileRows * 16;  // 6 KB: three planes of 128 rows
constexpr int kPlaneStages = 4;  // groups whose planes are in flight or staged: HBM latency is longer than one tile's dequantisation
constexpr int kMaxSplits = 16;
constexpr int kTmemCols = 32;
constexpr size_t kCombineOffset = 16384;

struct MmaParams {
  alignas(64) CUtensorMap plane_map;  // planes as uint32 [G*3][O/32][128], box 3 x 4 x 128
  const void* x;
  const unsigned short* scales;
  const uint8_t* zeros;
  const int16_t* perm;
  void* out;
  unsigned long long* combine;
  unsigned* status;
  int M, O, K, G;
  int groups_per_split, splits;
  int act_dtype, scale_dtype;
};

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes;
// `lbo` = byte distance between core matrices adjacent in K, `sbo` = between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t address, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((address >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) |
         (1ull << 46);
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 2) w3_mma_kernel(const __grid_constant__ MmaParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* const a_tiles = smem;                           // 2 x 32 KB
  unsigned char* const b_tiles = smem + 2 * kATile;              // 2 x 4 KB
  unsigned char* const planes_s = b_tiles + 2 * kBTile;          // 2 x 6 KB
  // barriers: mma_done[2] at 0, all_done at 2, tile_full[2] at 3, plane_full[kPlaneStages] at 5
  uint64_t* const bars = reinterpret_cast<uint64_t*>(planes_s + kPlaneStages * kPlaneTile);
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 5 + kPlaneStages);
  // Spread table: entry b (a plane byte, bit i = input i of the chunk) -> a word whose nibble for
  // input i holds that bit; input 2j sits in nibble j of the low half, input 2j + 1 in nibble j of
  // the high half, so that shifting by 4j and masking with 0x000f000f leaves inputs 2j and 2j + 1 in
  // the two 16-bit lanes of a word.  Sixteen copies side by side (entry stride 64 B, copy stride
  // 4 B): lane l reads copy l % 16, so two lanes at most share a bank group.
  unsigned char* const spread = planes_s + kPlaneStages * kPlaneTile + 128;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int g_begin = split * p.groups_per_split, g_end = min(p.G, g_begin + p.groups_per_split);
  const int ng = g_end - g_begin;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid < 5 + kPlaneStages) {
    mbar_init(smem_u32(&bars[tid]), tid == 3 || tid == 4 ? kProducers : 1);  // a finished tile: every producer thread arrives
    mbar_init_fence();
  }
  if (tid < kProducers) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {  // 256 entries x 16 copies, written in address order
      const uint32_t index = (uint32_t)tid + 256u * j, byte = index >> 4;
      uint32_t word = 0u;
#pragma unroll
      for (int i = 0; i < 8; ++i) word |= ((byte >> i) & 1u) << ((i & 1) * 16 + (i >> 1) * 4);
      reinterpret_cast<uint32_t*>(spread)[index] = word;
    }
  }
  if (warp == 0) {  // TMEM columns for the 128 x 16 fp32 accumulator
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  auto issue_planes = [&](int gi) {  // one elected thread: the three planes of group gi, 128 rows
    const uint32_t bar = smem_u32(&bars[5 + gi % kPlaneStages]);
    mbar_expect_tx(bar, (uint32_t)kPlaneTile);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(planes_s + (size_t)(gi % kPlaneStages) * kPlaneTile)),
        "l"(&p.plane_map), "r"(0), "r"(tile * (kTileRows / 32)), "r"(3 * (g_begin + gi)), "r"(bar)
        : "memory");
  };
  const bool issuer = tid == kProducers;  // lane 0 of the ninth warp
  if (issuer) {  // weights never change: staged before the wait on the previous kernel
    for (int gi = 0; gi < kPlaneStages && gi < ng; ++gi) issue_planes(gi);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // instruction descriptor: D fp32, A and B in the activation dtype, both K-major, N = 16, M = 128
  const uint32_t format = p.act_dtype == FB_BF16 ? 1u : 0u;
  const uint32_t idesc = (1u << 4) | (format << 7) | (format << 10) | ((uint32_t)(kN >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);

  const int row_in_tile = tid & 127, khalf = (tid >> 7) & 1;  // dequantisation: one row, 8 of its 16 chunks
  const int row = tile * kTileRows + row_in_tile;
  const int xn = tid >> 4, xc = tid & 15;  // activation tile: row of the batch, chunk of 8 inputs
  bool dead = false;

  // Per-group operands that come straight from global memory (scale and zero point of this
  // thread's row, eight activations of this thread's batch row) are requested one group ahead.
  // (volatile requests: they must stay a whole group ahead of their first use)
  uint32_t scale_bits_next = 0, zero_bits_next = 4;
  uint4 x_next = make_uint4(0u, 0u, 0u, 0u);
  auto fetch_group = [&](int g) {
    scale_bits_next = 0;
    zero_bits_next = 4;
    x_next = make_uint4(0u, 0u, 0u, 0u);
    if (row < p.O) {  // rows past O contribute zero weights (scale 0)
      asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(scale_bits_next) : "l"(p.scales + (size_t)g * p.O + row));
      if (p.zeros) asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(zero_bits_next) : "l"(p.zeros + (size_t)g * p.O + row));
    }
    if (xn < p.M) {
      const int kbase = g * 128 + xc * 8;
      const unsigned short* xrow = reinterpret_cast<const unsigned short*>(p.x) + (size_t)xn * p.K;
      if (p.perm) {  // gathered through the column order
        unsigned short v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = xrow[p.perm[kbase + j]];
        x_next = make_uint4(v[0] | (uint32_t)v[1] << 16, v[2] | (uint32_t)v[3] << 16, v[4] | (uint32_t)v[5] << 16, v[6] | (uint32_t)v[7] << 16);
      } else {
        asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(x_next.x), "=r"(x_next.y), "=r"(x_next.z), "=r"(x_next.w)
                     : "l"(xrow + kbase));
      }
    }
  };
  // ---- the issuing lane: for every group, wait for its tile, run the eight MMAs, signal the
  // buffer free through the MMAs' completion, and stage the planes kPlaneStages groups ahead (every
  // producer has read this buffer's planes once the tile is complete).  No CTA-wide barrier in
  // the loop: producers and issuer meet on mbarriers only. ----
  if (issuer) {
    for (int gi = 0; gi < ng; ++gi) {
      const int buf = gi & 1;
      if (!mbar_wait_bounded(smem_u32(&bars[3 + buf]), (uint32_t)((gi >> 1) & 1))) {
        dead = true;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_base = smem_u32(a_tiles + (size_t)buf * kATile), b_base = smem_u32(b_tiles + (size_t)buf * kBTile);
#pragma unroll
      for (int j = 0; j < 8; ++j)  // K = 16 per instruction: two chunks
        mma_f16(tmem_base, smem_desc(a_base + j * 2 * 2048, 2048, 128), smem_desc(b_base + j * 2 * 256, 256, 128), idesc,
                (gi > 0 || j > 0) ? 1u : 0u);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[buf])) : "memory");
      if (gi + kPlaneStages < ng) issue_planes(gi + kPlaneStages);  // every producer has read this stage: its tile is complete
    }
    if (!dead) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[2])) : "memory");
  }

  if (tid < kProducers && ng > 0) fetch_group(g_begin);

  for (int gi = 0; gi < ng && tid < kProducers; ++gi) {
    const int buf = gi & 1;
    const float scale = row < p.O ? bits_to_float((unsigned short)scale_bits_next, p.scale_dtype) : 0.f;
    const float zero = (float)zero_bits_next;
    const uint4 xraw = x_next;
    if (gi + 1 < ng) fetch_group(g_begin + gi + 1);
    // the tiles of this buffer were last read by the MMAs issued two groups ago
    bool ok = true;
    if (gi >= 2) ok = mbar_wait_bounded(smem_u32(&bars[buf]), (uint32_t)(((gi >> 1) - 1) & 1));
    ok = ok && mbar_wait_bounded(smem_u32(&bars[5 + gi % kPlaneStages]), (uint32_t)((gi / kPlaneStages) & 1));
    if (!ok) {
      dead = true;
      break;
    }
    // ---- activation tile: core matrix (chunk, 8 batch rows) at chunk * 256 + (n / 8) * 128 ----
    *reinterpret_cast<uint4*>(b_tiles + (size_t)buf * kBTile + xc * 256 + (xn >> 3) * 128 + (xn & 7) * 16) = xraw;
    // ---- weight tile: core matrix (chunk, 8 rows) at chunk * 2048 + (row / 8) * 128 ----
    {
      const unsigned char* pl = planes_s + (size_t)(gi % kPlaneStages) * kPlaneTile + row_in_tile * 16 + khalf * 8;
      const uint2 w0 = *reinterpret_cast<const uint2*>(pl), w1 = *reinterpret_cast<const uint2*>(pl + kTileRows * 16),
                  w2 = *reinterpret_cast<const uint2*>(pl + 2 * kTileRows * 16);
      // weight = T((code - zero) * T(scale)) in packed 16-bit arithmetic.  The three planes' spread
      // words add up to code' = b0 + 2 b1 + 4 b2' per nibble (the high plane is stored inverted, so
      // code = code' ^ 4).  For the pair of inputs (2j, 2j + 1): shift by 4j, keep the two nibbles,
      // flip their bit 2 and set the exponent bits of 1024 (fp16) or 128 (bf16) in ONE three-input
      // logic instruction: the two lanes now hold bias + code exactly.  A packed subtract of
      // bias + zero leaves code - zero, a packed multiply applies the scale with a single rounding,
      // as the reference's dense fallback rounds.
      using Pair = typename std::conditional<BF16, __nv_bfloat162, __half2>::type;
      auto as_pair = [](uint32_t bits) { return *reinterpret_cast<const Pair*>(&bits); };
      auto as_bits = [](Pair v) { return *reinterpret_cast<const uint32_t*>(&v); };
      Pair bias_zero2, scale2;  // bias + zero (an integer below 2048 / 256: exact), scale
      if (BF16) {
        const __nv_bfloat162 o2 = __float2bfloat162_rn(128.f + zero), s2 = __float2bfloat162_rn(scale);
        bias_zero2 = *reinterpret_cast<const Pair*>(&o2);
        scale2 = *reinterpret_cast<const Pair*>(&s2);
      } else {
        const __half2 o2 = __float2half2_rn(1024.f + zero), s2 = __float2half2_rn(scale);
        bias_zero2 = *reinterpret_cast<const Pair*>(&o2);
        scale2 = *reinterpret_cast<const Pair*>(&s2);
      }
      constexpr uint32_t kMagic = (BF16 ? 0x43004300u : 0x64006400u) | 0x00040004u;  // exponent bits, and the flip of bit 2
      const uint32_t table = smem_u32(spread) + (uint32_t)((lane & 15) * 4);
      auto spread_of = [&](uint32_t word, int byte) {  // the table word of byte `byte` of `word`
        uint32_t v;
        const uint32_t index = (word >> (8 * byte)) & 0xffu;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(table + index * 64u));
        return v;
      };
      unsigned char* const a_row = a_tiles + (size_t)buf * kATile + (row_in_tile >> 3) * 128 + (row_in_tile & 7) * 16;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t p0 = c < 4 ? w0.x : w0.y, p1 = c < 4 ? w1.x : w1.y, p2 = c < 4 ? w2.x : w2.y;
        // nibbles never carry: b0 + 2 b1 + 4 b2' <= 7
        const uint32_t codes = spread_of(p0, c & 3) + 2u * spread_of(p1, c & 3) + 4u * spread_of(p2, c & 3);
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t biased;  // (shifted & 0x000f000f) ^ 0x00040004 | exponent bits == mask ? shifted ^ magic : magic
          asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(biased) : "r"(codes >> (4 * j)), "r"(0x000f000fu), "r"(kMagic));
          packed[j] = as_bits(__hmul2(__hsub2(as_pair(biased), bias_zero2), scale2));
        }
        *reinterpret_cast<uint4*>(a_row + (size_t)(khalf * 8 + c) * 2048) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
    // generic-proxy stores must be visible to the tensor core's (async proxy) reads; then this
    // thread's part of the tile is done
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars[3 + buf])) : "memory");
  }

  // ---- all MMAs done: read the accumulator back ----
  // (a thread whose bounded wait expired arrives here with `dead` set; the others' waits expire in turn)
  {
    const bool ok = !dead && (ng == 0 || mbar_wait_bounded(smem_u32(&bars[2]), 0u));
    if (__syncthreads_or(!ok)) dead = true;
  }
  if (dead) {
    if (tid == 0) atomicExch(p.status, 3u);
  } else if (warp < 4 && ng > 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t acc[16];
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]), "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7]), "=r"(acc[8]),
          "=r"(acc[9]), "=r"(acc[10]), "=r"(acc[11]), "=r"(acc[12]), "=r"(acc[13]), "=r"(acc[14]), "=r"(acc[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    const int out_row = tile * kTileRows + warp * 32 + lane;  // TMEM lane = row of the tile
    if (out_row < p.O) {
      if (p.splits == 1) {
#pragma unroll
        for (int n = 0; n < kN; ++n)
          if (n < p.M) store_act(p.out, p.act_dtype, n * p.O + out_row, __uint_as_float(acc[n]));
      } else {
        // same combine as the M = 1 kernel: fixed point in bits 12..63, arrivals in bits 0..5,
        // non-finite / out-of-range contributions counted in bits 6..11.  All adds of a thread are
        // issued before the first answer is looked at: one round trip, not one per batch row.
        unsigned long long add[kN], old[kN];
#pragma unroll
        for (int n = 0; n < kN; ++n) {
          const float v = __uint_as_float(acc[n]);
          const bool fits = fabsf(v) < 2097152.f;
          add[n] = fits ? ((unsigned long long)__float2ll_rn(v * 67108864.f) << 12) + 1ull : 65ull;
          old[n] = 0ull;
          if (n < p.M)
            asm volatile("atom.add.relaxed.gpu.global.u64 %0, [%1], %2;"
                         : "=l"(old[n])
                         : "l"(p.combine + (size_t)n * p.O + out_row), "l"(add[n])
                         : "memory");
        }
#pragma unroll
        for (int n = 0; n < kN; ++n) {
          if (n < p.M && (int)(old[n] & 63ull) == p.splits - 1) {
            const unsigned long long total = old[n] + add[n];
            float value = __ll2float_rn((long long)total >> 12) * 1.4901161193847656e-08f;
            if ((total >> 6) & 63ull) value = __int_as_float(0x7fc00000);
            store_act(p.out, p.act_dtype, n * p.O + out_row, value);
            p.combine[(size_t)n * p.O + out_row] = 0ull;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

}  // namespace

extern "C" size_t fb_w3_gemm_small_scratch_bytes(int m, int out_features, int in_features) {
  if (m < 1 || m > kN || out_features < 32 || in_features < 128) return 0;
  return kCombineOffset + (size_t)m * out_features * sizeof(unsigned long long);
}

extern "C" int fb_w3_gemm_small(const void* x, int act_dtype, int m, const uint8_t* planes, const void* scales, int scale_dtype,
                                const uint8_t* zeros, const int16_t* perm, void* out, int out_features, int in_features,
                                void* scratch, size_t scratch_bytes, fb_stream_t stream) {
  const int O = out_features, K = in_features;
  if (!x || !planes || !scales || !out) return fail(FB_EINVAL, "fb_w3_gemm_small: x, planes, scales and out must be non-null");
  if ((act_dtype != FB_F16 && act_dtype != FB_BF16) || (scale_dtype != FB_F16 && scale_dtype != FB_BF16))
    return fail(FB_EINVAL, "fb_w3_gemm_small: dtype tags must be FB_F16 or FB_BF16");
  if (m < 1 || m > kN) return fail(FB_ELIMIT, "fb_w3_gemm_small: M=%d outside 1..%d", m, kN);
  if (K < 128 || K % 128 || K / 128 > 255) return fail(FB_ELIMIT, "fb_w3_gemm_small: K=%d must be a multiple of 128 with at most 255 groups", K);
  if (O < 32 || O > 65536 || O % 32) return fail(FB_ELIMIT, "fb_w3_gemm_small: O=%d must be a multiple of 32 in 32..65536", O);
  if (!aligned(planes, 16) || !aligned(scales, 2) || !aligned(out, 2) || !aligned(perm, 2))
    return fail(FB_EINVAL, "fb_w3_gemm_small: planes must be 16-byte aligned, 16-bit tensors 2-byte aligned");
  if (!perm && !aligned(x, 16)) return fail(FB_EINVAL, "fb_w3_gemm_small: x must be 16-byte aligned");
  const int G = K / 128;
  const size_t x_bytes = (size_t)m * K * 2, out_bytes = (size_t)m * O * 2;
  if (overlaps(out, out_bytes, x, x_bytes) || overlaps(out, out_bytes, planes, (size_t)G * 3 * O * 16) ||
      overlaps(out, out_bytes, scales, (size_t)G * O * 2))
    return fail(FB_EALIAS, "fb_w3_gemm_small: out overlaps an input");
  const size_t need = fb_w3_gemm_small_scratch_bytes(m, O, K);
  if (!scratch || scratch_bytes < need) return fail(FB_ESCRATCH, "fb_w3_gemm_small: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  if (!aligned(scratch, 256)) return fail(FB_EINVAL, "fb_w3_gemm_small: scratch must be 256-byte aligned");
  if (overlaps(scratch, need, out, out_bytes) || overlaps(scratch, need, x, x_bytes)) return fail(FB_EALIAS, "fb_w3_gemm_small: scratch overlaps x or out");

  const DeviceInfo* info = device_info();
  if (!info) return FB_ECUDA;
  MmaParams p;
  if (!plane_tensor_map(planes, O, G, kTileRows / 32, 3, &p.plane_map)) return FB_ECUDA;
  p.x = x;
  p.scales = static_cast<const unsigned short*>(scales);
  p.zeros = zeros;
  p.perm = perm;
  p.out = out;
  p.status = reinterpret_cast<unsigned*>(scratch);
  p.combine = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(scratch) + kCombineOffset);
  p.M = m;
  p.O = O;
  p.K = K;
  p.G = G;
  p.act_dtype = act_dtype;
  p.scale_dtype = scale_dtype;
  const int tiles = (O + kTileRows - 1) / kTileRows;
  int splits = 2 * info->sm_count / tiles;
  if (splits < 1) splits = 1;
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits > G) splits = G;
  p.groups_per_split = (G + splits - 1) / splits;
  p.splits = (G + p.groups_per_split - 1) / p.groups_per_split;

  const size_t smem = 2 * (size_t)kATile + 2 * kBTile + kPlaneStages * kPlaneTile + 128 + 16384;  // tiles, barriers, spread table
  static std::mutex lock;
  static bool ready[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  {
    std::lock_guard<std::mutex> guard(lock);
    if (device >= 0 && device < 64 && !ready[device]) {
      cudaError_t err = cudaFuncSetAttribute(w3_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err == cudaSuccess) err = cudaFuncSetAttribute(w3_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(w3_mma_kernel)");
      ready[device] = true;
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(tiles, p.splits);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl_allowed() ? 1 : 0;
  cudaError_t err = act_dtype == FB_BF16 ? cudaLaunchKernelEx(&config, w3_mma_kernel<true>, p) : cudaLaunchKernelEx(&config, w3_mma_kernel<false>, p);
  if (err != cudaSuccess) return cuda_fail(err, "w3_mma_kernel launch");
  return FB_OK;
}
