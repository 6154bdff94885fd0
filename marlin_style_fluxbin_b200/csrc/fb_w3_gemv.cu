// GPTQ W3 group-128 planar GEMV for M = 1..4 rows of activations (batch-1 decode).
//
// HBM-bound byte work: every packed weight byte is read exactly once.  The design:
//
//  * K is cut into blocks of two groups (256 inputs = 32 chunks of 8).  For a K block a
//    CTA holds 32 activation lookup tables (one per chunk, 256 subset sums each) in
//    shared memory, laid out entry-major: entry p of table t lives at byte p*128 + t*4
//    (M = 1), so the BANK of a lookup is the table number, never the weight byte.
//  * A warp processes a unit of 32 output rows x one K block; lane = row, so no
//    cross-lane reduction is needed.  Lanes walk the 32 chunks in a rotated order
//    (half / word / byte rotation from the lane number) such that at every step the 32
//    lanes address 32 different tables: all table lookups are bank-conflict free by
//    construction, whatever the weights are.  The same rotation makes the reads of the
//    staged weight words conflict free.
//  * The three bit planes of a unit (6 runs of 512 bytes: group half x plane) are staged into
//    shared memory by ONE tiled bulk copy (cp.async.bulk.tensor + mbarrier).  Every warp owns a
//    private ring of staged units and refills a slot as soon as it has read it, so warps never
//    wait for one another between table builds.
//  * Two CTAs of 8 warps per SM (together the whole register file; 110 KB of shared memory each
//    with M = 1): each K super-block is served by floor(2 SMs / super-blocks) CTAs that split its
//    rows.  Two smaller CTAs beat one of 16 warps: when the first of a pair leaves, CTAs of the
//    next kernel in the stream move in and stage weights beside the one still running.
//  * A warp whose rows are a single unit carries its sum across the K blocks its CTA walks
//    (K > 4096) in registers; otherwise the running sums go through an L2-resident scratch.
//  * M = 1: scales and zero points of a unit ride with its planes (two more small tiled copies
//    into the same ring slot), so HBM latency never sits between a unit's lookups and its
//    result.  M > 1 (no room in the ring): coalesced global loads requested one task ahead.
//  * Fused producers of x (M = 1): RMSNorm, the SwiGLU gate, or the merge of the attention
//    launch's per-split pieces.  Every thread transforms ONE of the K block's 256 activations and
//    shares it through shared memory; the tables are built from the shared values.
//  * Two lookups are accumulated by one packed fp32x2 add or multiply-add (an even-step and an
//    odd-step partial sum share a 64-bit register pair; the plane weights 1, 2, -4 ride in the
//    multiply-add), which halves the arithmetic of the main loop and leaves four accumulators.
//  * Launched with programmatic dependent launch: barrier set-up and the first weight copies
//    come before griddepcontrol.wait; everything that reads activations or touches scratch
//    comes after it, and the later ring stages are requested after the first table build (their
//    issue would otherwise sit in front of it on the critical path).
//  * Split-K is combined inside the kernel with ONE 64-bit atomic add per contribution: the
//    partial sum in fixed point (2^-26 units) plus an arrival count in the low bits.  Integer
//    addition is associative, so the result is independent of arrival order (deterministic,
//    repeat-exact); the contributor that reads back the last count writes the output.  A K
//    longer than 16 K blocks is walked in turn by the same CTA (at most 16 contributions).
//
// Arithmetic follows the reference kernel (csrc/w3_lut.cu:38-139): per group
// dot = a0 + 2*a1 - 4*a2 over the stored planes (plane 2 inverted), times the group
// scale, fp32 accumulation; tables hold ascending-order subset sums as in
// csrc/lut8_unsigned.cuh:12-27.  Extension over the reference: fp16 or bf16 scales and
// an optional per-(group,row) zero point, y += scale*(4-zero)*sum(x_group); the rounding
// correction of the dequantised-weight arithmetic (csrc/w3_lut.cu:105-122) is extended to zero
// points 3 and 4, the two for which +/-3 are the only inexact products.
#include <mutex>
#include <type_traits>

#include "fb_common.cuh"

namespace {

using namespace fb;

constexpr int kUnitRows = 32;
constexpr int kPlaneTile = kUnitRows * 16;      // 512 B: one plane of one group for a unit
constexpr int kUnitBytes = 2 * 3 * kPlaneTile;  // 3072 B of planes staged per unit
// CTA shape by activation rows: with the tables of one or two rows (32 / 64 KB) two CTAs of eight
// warps share an SM, so that one CTA's build and tail overlap the other's lookups; the 128 KB of
// tables for three or four rows leave room for one CTA, which then runs sixteen warps.
constexpr int warps_for(int m) { return m <= 2 ? 8 : 16; }
constexpr int ctas_per_sm_for(int m) { return m <= 2 ? 2 : 1; }
constexpr int kMaxM = 4;
constexpr int kMaxSplits = 16;  // partial sums per output (one arrival count of 6 bits, 52-bit fixed-point sum)
constexpr int kMaxMatrices = 4;

// One weight matrix of a launch.  Several matrices that share x and K (q/k/v, gate/up) are
// served by one launch: their rows are concatenated, 32-row unit by unit.
struct W3Matrix {
  const uint8_t* planes;
  const unsigned short* scales;
  const uint8_t* zeros;
  void* out;             // [M,O] 16-bit, or fp32 [G,O] group partials when group_partials != 0
  const void* residual;  // optional [M,O] 16-bit, added to the rounded result
  int O;
  int ru_begin;          // first 32-row unit of this matrix in the concatenated row space
};

struct W3Params {
  // One tiled-copy descriptor per matrix: the planes seen as uint32 [G*3][O/32][128], so that a
  // box of 6 x 1 x 128 is the six 512-byte runs of one unit (two groups x three planes).
  alignas(64) CUtensorMap plane_maps[kMaxMatrices];
  // Scales and zero points as [G][O] tensors, box = 32 rows x 2 groups: the 128 + 64 bytes a unit
  // needs of them are staged beside its planes.  Groups beyond G read as zero, which drops the
  // empty half of the last K block of an odd G without any test in the kernel.
  CUtensorMap scale_maps[kMaxMatrices];
  CUtensorMap zero_maps[kMaxMatrices];
  const void* x;
  W3Matrix mats[kMaxMatrices];
  int n_mats;
  const int16_t* perm;
  const void* prologue_arg;  // RMSNorm weight [K] (kind 1), the `up` vector [K] (kind 2), attention partials (kind 3)
  int prologue;              // 0 none, 1 RMSNorm of x, 2 x = silu(x) * up, 3 x = merged attention splits  (M = 1, identity order)
  int attn_splits;           // kind 3: splits per head (1..8)
  float eps;
  // Tensor-parallel push (M = 1, one matrix): instead of writing `out`, the final fp32 value of a
  // row goes, together with a valid mark in the same 8-byte store, to slot `row` of a buffer on
  // every rank (peer pointers over NVLink, this rank's own buffer included).  No fence and no
  // counter: the receiver polls each slot for its mark.
  unsigned long long* push_data[8];
  int push_world;  // 0 = no push
  float* partials;  // [nSB, M, O]
  unsigned long long* combine;  // [M, O] split-K accumulators, zero between launches
  unsigned* status;
  int O, K, G, nKB, nRU;
  int act_dtype, scale_dtype;
  int S, nSB;          // K blocks per super-block (one CTA walks them in turn), super-blocks
  int units_per_slice, units_extra;  // nRU / slices and nRU % slices
  int group_partials;  // write scale-multiplied per-group sums instead of reducing
  int same_input;      // FB_W3_SAME_INPUT: no wait at the start, one before the end
};

// Shared-memory geometry.  Entry p of table t for activation row m lives at byte
//   p * kStride + m * 128 + t * 4,   kStride = 128 * (M rounded up to a power of two),
// so with M = 1 the 32 tables of a K block take 32 KB and the bank of a lookup is the table
// number.  The ring holds three staged units per warp with M = 1, two otherwise (M = 2 then still
// fits two CTAs per SM).
template <int M>
struct Geom {
  static constexpr int kWarps = warps_for(M);
  static constexpr int kCtasPerSm = ctas_per_sm_for(M);
  static constexpr int kStrideLog = 7 + (M == 1 ? 0 : (M == 2 ? 1 : 2));
  static constexpr int kStride = 1 << kStrideLog;
  static constexpr int kLutBytes = 256 << kStrideLog;
  static constexpr int kStages = M == 1 ? 3 : 2;
  // a staged unit: its planes, then (M = 1 only: with larger tables two CTAs per SM leave no room)
  // its scales at +3072 (2 groups x 64 B) and its zero points at +3200 (2 groups x 32 B)
  static constexpr bool kStageAux = M == 1;
  static constexpr int kSlotBytes = kUnitBytes + (kStageAux ? 256 : 0);
  static constexpr int kRingOffset = kLutBytes;
  static constexpr int kBarOffset = kRingOffset + kWarps * kStages * kSlotBytes;
  static constexpr int kSmemBytes = kBarOffset + kWarps * kStages * 8;
};

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// acc + {table entry at a0, table entry at a1}: the two loads land in the halves of one 64-bit
// register pair, which the packed add consumes as it is.
__device__ __forceinline__ uint64_t add2_lds(uint64_t acc, uint32_t a0, uint32_t a1) {
  uint64_t r;
  asm volatile(
      "{\n\t.reg .f32 lo, hi;\n\t.reg .b64 both;\n\t"
      "ld.shared.f32 lo, [%2];\n\t"
      "ld.shared.f32 hi, [%3];\n\t"
      "mov.b64 both, {lo, hi};\n\t"
      "add.rn.f32x2 %0, %1, both;\n\t}"
      : "=l"(r)
      : "l"(acc), "r"(a0), "r"(a1));
  return r;
}
// acc + w * {table entry at a0, table entry at a1} with w = {2, 2} or {-4, -4}: the plane weights of
// code - 4 = b0 + 2 b1 - 4 b2' applied as the entries are accumulated (products by 2 and 4 are exact).
__device__ __forceinline__ uint64_t fma2_lds(uint64_t acc, uint32_t a0, uint32_t a1, uint64_t w) {
  uint64_t r;
  asm volatile(
      "{\n\t.reg .f32 lo, hi;\n\t.reg .b64 both;\n\t"
      "ld.shared.f32 lo, [%2];\n\t"
      "ld.shared.f32 hi, [%3];\n\t"
      "mov.b64 both, {lo, hi};\n\t"
      "fma.rn.f32x2 %0, both, %4, %1;\n\t}"
      : "=l"(r)
      : "l"(acc), "r"(a0), "r"(a1), "l"(w));
  return r;
}
// Shared-memory load at a 32-bit address plus a compile-time offset (folded into the instruction).
template <int OFFSET>
__device__ __forceinline__ float lds_at(uint32_t address) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(address), "n"(OFFSET));
  return v;
}
__device__ __forceinline__ float sum2(uint64_t v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo + hi;
}

// Matrix that owns 32-row unit `ru` of the concatenated row space.
__device__ __forceinline__ int locate_unit(const W3Params& p, int ru) {
  int j = 0;
  while (j + 1 < p.n_mats && ru >= p.mats[j + 1].ru_begin) ++j;
  return j;
}

// Final value of one output element: rounded to the 16-bit dtype, then the optional residual is
// added and the sum rounded again (what separate Linear and add kernels produce); or, for the
// tensor-parallel push, one 8-byte store {value, mark = 1} into every rank's exchange buffer.
// Reached once per output row: kept out of line, away from the main loop's registers and code.
__device__ __forceinline__ void emit_row(const W3Params& p, int m, int ru, int lane, float value) {
  const W3Matrix& mat = p.mats[locate_unit(p, ru)];
  const int lrow = (ru - mat.ru_begin) * kUnitRows + lane;
  if (p.push_world > 0) {
    const unsigned long long slot = (1ull << 32) | (unsigned long long)__float_as_uint(value);
    for (int r = 0; r < p.push_world; ++r)
      asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p.push_data[r] + lrow), "l"(slot) : "memory");
    return;
  }
  if (mat.residual) value = round_to(value, p.act_dtype) + load_act(mat.residual, p.act_dtype, m * mat.O + lrow);
  store_act(mat.out, p.act_dtype, m * mat.O + lrow, value);
}

// The contributor that read back the last arrival count: fixed point to float, NaN if any partial
// had no fixed-point form, emit, and leave the combine word zero for the next launch.
__device__ __forceinline__ void emit_combined(const W3Params& p, int m, int ru, int lane, unsigned long long total) {
  float value = __ll2float_rn((long long)total >> 12) * 1.4901161193847656e-08f;  // 2^-26
  if ((total >> 6) & 63ull) value = __int_as_float(0x7fc00000);
  emit_row(p, m, ru, lane, value);
  p.combine[(size_t)m * p.O + ru * kUnitRows + lane] = 0ull;
}

template <int M, bool CORRECT>
__global__ void __launch_bounds__(Geom<M>::kWarps * 32, Geom<M>::kCtasPerSm) w3_gemv_kernel(const __grid_constant__ W3Params p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  using G_ = Geom<M>;
  constexpr int kStages = G_::kStages, kWarps = G_::kWarps;
  // the warp index through a shuffle: the compiler then knows that it, and everything derived from it (ring
  // addresses, unit counters, copy coordinates), is the same in all lanes and keeps it in uniform registers
  const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  unsigned char* const lut = smem;
  // Every warp owns a private ring of kStages staged units, [stage][group half * 3 + plane][32 rows
  // x 16 B], and one mbarrier per stage: warps never wait for one another between table builds.
  const uint32_t ring_u32 = smem_u32(smem + G_::kRingOffset) + (uint32_t)(warp * kStages * G_::kSlotBytes);
  const uint32_t bars_u32 = smem_u32(smem + G_::kBarOffset) + (uint32_t)(warp * kStages * 8);

  // Release of the next kernel in the stream.  A launch that waits for the one ahead of it releases
  // its dependents only AFTER that wait (further down): whatever follows it in the stream then
  // starts with everything before this launch complete.  That is what allows a launch whose inputs
  // were ready before the launch ahead began (FB_W3_SAME_INPUT: k_proj behind q_proj, up_proj
  // behind gate_proj) to skip the wait at its start: it begins at once, releases at once, and waits
  // for the launch ahead only before it ends, so that stream order holds for what comes after.
  if (p.same_input) pdl_launch_dependents();

  if (threadIdx.x < kWarps * kStages) {
    mbar_init(smem_u32(smem + G_::kBarOffset) + threadIdx.x * 8, 1);  // the issuing lane's expect_tx
    mbar_init_fence();
  }
  __syncthreads();

  // Work of this CTA: super-block blockIdx.y (K blocks sb*S ..), the row units [first, first + count)
  // of slice blockIdx.x.  The first nRU % slices slices take one unit more.
  const int sb = (int)blockIdx.y;
  const int cta_first = (int)blockIdx.x * p.units_per_slice + min((int)blockIdx.x, p.units_extra);
  const int cta_count = p.units_per_slice + ((int)blockIdx.x < p.units_extra ? 1 : 0);
  auto locate = [&](int ru) { return locate_unit(p, ru); };
  auto emit = [&](int m, int ru, float value) { emit_row(p, m, ru, lane, value); };

  // Lane rotation (byte, half, word): at every step the 32 lanes hit 32 different tables.
  const int rb = lane & 3, rh = (lane >> 2) & 1, rw = (lane >> 3) & 3;
  // Per-lane constants of the rotated walk, all as 32-bit shared-memory addresses / offsets so
  // that the hot loop does no 64-bit pointer arithmetic.  A lookup is: one 4-way byte dot product
  // (entry * stride + table address), the shared-memory load, and half a packed add.
  const uint32_t lut_u32 = smem_u32(lut);
  uint32_t sel[4], xl[2][4][4], woff[2][4];
#pragma unroll
  for (int b = 0; b < 4; ++b) sel[b] = 128u << (8 * ((b + rb) & 3));  // weight 128 at byte (b+rb)%4
#pragma unroll
  for (int jh = 0; jh < 2; ++jh)
#pragma unroll
    for (int jw = 0; jw < 4; ++jw) {
      woff[jh][jw] = (uint32_t)(((jh ^ rh) * 3) * kPlaneTile + ((jw + rw) & 3) * 4 + lane * 16);
#pragma unroll
      for (int b = 0; b < 4; ++b) xl[jh][jw][b] = lut_u32 + 64u * (jh ^ rh) + 16u * ((jw + rw) & 3) + 4u * ((b + rb) & 3);
    }
  // entry * stride + table address in ONE instruction: a 4-way byte dot product whose only
  // non-zero weight (the stride, 128 for M = 1) sits at the wanted byte of the staged word
  auto lookup_address = [&](uint32_t word, int b, uint32_t table) {
    uint32_t address;
    if (G_::kStride <= 128) {
      asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(address) : "r"(word), "r"(sel[b]), "r"(table));
    } else {  // the stride does not fit a byte weight: dot product with weight 128, then scale
      uint32_t entry128;
      asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(entry128) : "r"(word), "r"(sel[b]), "r"(0u));
      address = entry128 * (G_::kStride / 128) + table;
    }
    return address;
  };

  // This CTA walks the K blocks kb_begin .. kb_begin + nS - 1 over the same rows.  Warp w takes
  // the units cta_first + w, + kWarps, ...; its tasks are numbered K block * my_count + unit.
  const int kb_begin = sb * p.S, nS = min(p.S, p.nKB - kb_begin);
  const int my_count = cta_count > warp ? (cta_count - warp + kWarps - 1) / kWarps : 0;
  const int my_tasks = nS * my_count;
  const int my_first = cta_first + warp, my_end = cta_first + cta_count;
  // Staging of this warp's tasks, in task order, into its ring: lane 0 announces the bytes of a unit
  // and issues ONE tiled copy that brings its six plane runs (and two small ones for its scales and
  // zero points).  A slot is refilled only after the
  // warp has finished reading it (all lanes pass a __syncwarp first).  The matrix a unit belongs
  // to changes rarely: its descriptor and bounds are cached.
  int pf_left = my_tasks, pf_slot = 0, pf_kb = kb_begin, pf_ru = my_first;  // the next task to stage
  int pf_j = 0, pf_begin = 0, pf_end = -1;
  bool pf_zeros = false;
  auto issue_next = [&]() {
    if (pf_ru < pf_begin || pf_ru >= pf_end) {
      pf_j = locate(pf_ru);
      pf_begin = p.mats[pf_j].ru_begin;
      pf_end = pf_j + 1 < p.n_mats ? p.mats[pf_j + 1].ru_begin : p.nRU;
      pf_zeros = p.mats[pf_j].zeros != nullptr;
    }
    if (lane == 0) {
      const uint32_t bar = bars_u32 + (uint32_t)(pf_slot * 8);
      const uint32_t dst = ring_u32 + (uint32_t)(pf_slot * G_::kSlotBytes);
      const int lru = pf_ru - pf_begin;
      // the boxes are always whole: what lies beyond G reads as zero and still counts as bytes
      mbar_expect_tx(bar, (uint32_t)(kUnitBytes + (G_::kStageAux ? 128 + (pf_zeros ? 64 : 0) : 0)));
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
          "l"(&p.plane_maps[pf_j]), "r"(0), "r"(lru), "r"(6 * pf_kb), "r"(bar)
          : "memory");
      if (G_::kStageAux) {
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                         dst + (uint32_t)kUnitBytes),
                     "l"(&p.scale_maps[pf_j]), "r"(lru * kUnitRows), "r"(2 * pf_kb), "r"(bar)
                     : "memory");
        if (pf_zeros)
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                           dst + (uint32_t)(kUnitBytes + 128)),
                       "l"(&p.zero_maps[pf_j]), "r"(lru * kUnitRows), "r"(2 * pf_kb), "r"(bar)
                       : "memory");
      }
    }
    --pf_left;
    pf_slot = pf_slot + 1 == kStages ? 0 : pf_slot + 1;
    pf_ru += kWarps;
    if (pf_ru >= my_end) {
      pf_ru = my_first;
      ++pf_kb;
    }
  };
  // Weights never change, so staging needs no wait.  Only one unit per warp goes out before the
  // wait on the previous kernel: requests are served in order, and a whole grid's worth of weights
  // ahead of the wait slows the tail of the kernel still running and the small activation loads
  // that follow the wait.
  if (pf_left > 0) issue_next();

  // Without room in the ring (M > 1) the scales and zero points of a task come straight from global
  // memory (one coalesced run per group), requested ONE TASK AHEAD of their use so that HBM latency
  // never sits between a unit's lookups and its result.  Half jh of a lane's walk covers group
  // 2*kb + (jh ^ rh).
  uint32_t nx_scale[2] = {0u, 0u}, nx_zero[2] = {4u, 4u};
  int ax_j = 0, ax_begin = 0, ax_end = -1;
  bool any_zeros = false;
  for (int j = 0; j < p.n_mats; ++j) any_zeros = any_zeros || p.mats[j].zeros != nullptr;
  auto request_aux = [&](int kb_, int ru) {
    if (ru < ax_begin || ru >= ax_end) {  // entering another matrix of the launch: rare
      ax_j = locate(ru);
      ax_begin = p.mats[ax_j].ru_begin;
      ax_end = ax_j + 1 < p.n_mats ? p.mats[ax_j + 1].ru_begin : p.nRU;
    }
    const W3Matrix& mat = p.mats[ax_j];
    const int lrow = (ru - ax_begin) * kUnitRows + lane;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int g = min(2 * kb_ + (jh ^ rh), p.G - 1);  // an odd G: the empty half reads a valid address, its term is dropped
      const int at = g * mat.O + lrow;                  // G * O < 2^24
      asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(nx_scale[jh]) : "l"(mat.scales + at));
      nx_zero[jh] = 4u;
      if (mat.zeros) asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(nx_zero[jh]) : "l"(mat.zeros + at));
    }
  };
  if (!G_::kStageAux && my_tasks > 0) request_aux(kb_begin, my_first);  // constant data: may precede the wait as well
  // staged form: this lane's scale / zero point of walk half 0 within a slot; half 1 is the other group
  const uint32_t aux_scale0 = (uint32_t)(kUnitBytes + rh * 64 + lane * 2), aux_zero0 = (uint32_t)(kUnitBytes + 128 + rh * 32 + lane);
  // the walk constants are computed here, while the launch waits for the previous kernel anyway
#pragma unroll
  for (int jh = 0; jh < 2; ++jh)
#pragma unroll
    for (int jw = 0; jw < 4; ++jw) {
      asm volatile("" : "+r"(woff[jh][jw]));
#pragma unroll
      for (int b = 0; b < 4; ++b) asm volatile("" : "+r"(xl[jh][jw][b]));
    }

  // Everything below reads activations and writes scratch / outputs of this stream.
  if (!p.same_input) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
  }

  // Raw 16-bit activations of one lane's table (8 values); the next K block's are fetched while
  // the current one is being computed.
  const bool fast_x = M == 1 && !p.perm;
  auto fetch_x = [&](int kb_, uint4& raw) {
    const int g = 2 * kb_ + (lane >> 4);
    raw = make_uint4(0u, 0u, 0u, 0u);
    if (g < p.G) raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.x) + g * 128 + (lane & 15) * 8);
  };
  // With a fused input transform every thread owns ONE of the K block's 256 activations: it loads
  // the raw value and the operand, transforms them once and shares the result through shared
  // memory, instead of every warp transforming all 256 for itself.
  const bool shared_x = fast_x && p.prologue != 0;
  __shared__ __align__(16) float xs[M == 1 ? 256 : 4];
  uint32_t el_raw = 0u, el_op = 0u;
  auto fetch_el = [&](int kb_) {
    const int e = kb_ * 256 + (int)threadIdx.x;
    el_raw = el_op = 0u;
    if (p.prologue != 3 && threadIdx.x < 256 && e < p.K) {
      el_raw = reinterpret_cast<const unsigned short*>(p.x)[e];
      el_op = reinterpret_cast<const unsigned short*>(p.prologue_arg)[e];
    }
  };
  // requested before the RMS reduction below, so that the two round trips overlap
  uint4 raw_next = make_uint4(0u, 0u, 0u, 0u);
  if (shared_x)
    fetch_el(kb_begin);
  else if (fast_x)
    fetch_x(kb_begin, raw_next);

  // Optional fused input transform.  For RMSNorm every CTA reduces the whole activation row
  // itself (K 16-bit values: a few KB out of L2), which costs far less than a separate launch.
  float inv_rms = 1.f;
  if (p.prologue == 1) {
    float ss = 0.f;
    constexpr int kStep = kWarps * 32 * 8, kAhead = 4;  // four 16-byte loads of a thread in flight: one round trip for K <= 8192
    for (int i0 = threadIdx.x * 8; i0 < p.K; i0 += kAhead * kStep) {
      uint4 raws[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int i = i0 + u * kStep;
        raws[u] = make_uint4(0u, 0u, 0u, 0u);  // zeros past the end add nothing to the sum
        if (i < p.K) raws[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.x) + i);
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const uint32_t words[4] = {raws[u].x, raws[u].y, raws[u].z, raws[u].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = bits_to_float((unsigned short)((words[j >> 1] >> (16 * (j & 1))) & 0xffffu), p.act_dtype);
          ss += v * v;
        }
      }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    __shared__ float warp_sums[kWarps];
    if (lane == 0) warp_sums[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) ss += warp_sums[w];
    inv_rms = rsqrtf(ss / (float)p.K + p.eps);
  }

  if (kStages > 1 && pf_left > 0) issue_next();  // the second ring stage, behind the activation loads

  // ---- build the 32 tables of K block kb_: lane = table; warp w owns the entries of
  // 16 / kWarps low nibbles (2w and 2w + 1 with eight warps), so that the walk over the high nibble unrolls with constant offsets.  sx[m][jh]: the sum of the activations of the group this lane walks in half jh. ----
  auto build = [&](int kb_, float (&sx)[M][2]) {
    const int g = 2 * kb_ + (lane >> 4);
    const int kbase = g * 128 + (lane & 15) * 8;
    unsigned char* const tables = lut;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v8[8];
      if (shared_x && p.prologue == 3) {
        // x = the attention output, still in pieces: every split of a head left (output[128], max, sum) in
        // its slot; merge them as the attention kernel's own last step does (ascending split order, the
        // same fused multiply-adds) and round to the activation dtype.
        if (threadIdx.x < 256) {
          const int e = kb_ * 256 + (int)threadIdx.x;
          float value = 0.f;
          if (e < p.K) {
            const float* slots = static_cast<const float*>(p.prologue_arg) + (size_t)(e >> 7) * (16 * 132);
            float ms[8], ls[8], as[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
              ms[sp] = -INFINITY, ls[sp] = 0.f, as[sp] = 0.f;
              if (sp < p.attn_splits) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(slots + sp * 132 + 128));
                ms[sp] = ml.x, ls[sp] = ml.y;
                as[sp] = __ldcg(slots + sp * 132 + (e & 127));
              }
            }
            float gm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) gm = fmaxf(gm, ms[sp]);
            float total = 0.f, o = 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
              const float f = ms[sp] == -INFINITY ? 0.f : __expf(ms[sp] - gm);
              total = fmaf(ls[sp], f, total);
              o = fmaf(as[sp], f, o);
            }
            value = round_to(o * (1.f / total), p.act_dtype);
          }
          xs[M == 1 ? threadIdx.x : 0] = value;
        }
        __syncthreads();
        const float4 lo = *reinterpret_cast<const float4*>(&xs[M == 1 ? (lane >> 4) * 128 + (lane & 15) * 8 : 0]);
        const float4 hi4 = *reinterpret_cast<const float4*>(&xs[M == 1 ? (lane >> 4) * 128 + (lane & 15) * 8 + 4 : 0]);
        v8[0] = lo.x, v8[1] = lo.y, v8[2] = lo.z, v8[3] = lo.w;
        v8[4] = hi4.x, v8[5] = hi4.y, v8[6] = hi4.z, v8[7] = hi4.w;
      } else if (shared_x) {
        if (threadIdx.x < 256) {
          // same roundings as the separate kernels: RMSNorm casts before the weight multiply,
          // SwiGLU rounds silu(gate) before the product
          const float v = bits_to_float((unsigned short)el_raw, p.act_dtype), other = bits_to_float((unsigned short)el_op, p.act_dtype);
          xs[M == 1 ? threadIdx.x : 0] = p.prologue == 1 ? round_to(other * round_to(v * inv_rms, p.act_dtype), p.act_dtype)
                                                           : round_to(round_to(v / (1.f + __expf(-v)), p.act_dtype) * other, p.act_dtype);
        }
        if (kb_ + 1 < kb_begin + nS) fetch_el(kb_ + 1);
        __syncthreads();
        const float4 lo = *reinterpret_cast<const float4*>(&xs[M == 1 ? (lane >> 4) * 128 + (lane & 15) * 8 : 0]);
        const float4 hi4 = *reinterpret_cast<const float4*>(&xs[M == 1 ? (lane >> 4) * 128 + (lane & 15) * 8 + 4 : 0]);
        v8[0] = lo.x, v8[1] = lo.y, v8[2] = lo.z, v8[3] = lo.w;
        v8[4] = hi4.x, v8[5] = hi4.y, v8[6] = hi4.z, v8[7] = hi4.w;
      } else if (fast_x) {
        const uint32_t words[4] = {raw_next.x, raw_next.y, raw_next.z, raw_next.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v8[j] = bits_to_float((unsigned short)((words[j >> 1] >> (16 * (j & 1))) & 0xffffu), p.act_dtype);
        if (kb_ + 1 < kb_begin + nS) fetch_x(kb_ + 1, raw_next);
      } else if (g < p.G) {
        if (p.perm) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v8[j] = load_act(p.x, p.act_dtype, m * p.K + p.perm[kbase + j]);
        } else {
          const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.x) + (size_t)m * p.K + kbase);
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int j = 0; j < 8; ++j)
            v8[j] = bits_to_float((unsigned short)((words[j >> 1] >> (16 * (j & 1))) & 0xffffu), p.act_dtype);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v8[j] = 0.f;
      }
      // Every entry is the ascending-order subset sum of its activations (as the reference's
      // tables are): first the low nibble's, then one add per step of the high nibble's tree.
      unsigned char* const column = tables + m * 128 + lane * 4;
#pragma unroll
      for (int qq = 0; qq < 16 / kWarps; ++qq) {
        const int q = warp * (16 / kWarps) + qq;
        float hi[16];
        hi[0] = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if ((q >> b) & 1) hi[0] += v8[b];
#pragma unroll
        for (int h = 1; h < 16; ++h) {
          const int top = h >= 8 ? 3 : (h >= 4 ? 2 : (h >= 2 ? 1 : 0));
          hi[h] = hi[h & ~(1 << top)] + v8[4 + top];
        }
        unsigned char* const at = column + (size_t)q * G_::kStride;
#pragma unroll
        for (int h = 0; h < 16; ++h) *reinterpret_cast<float*>(at + (size_t)h * 16 * G_::kStride) = hi[h];
      }
      float total = 0.f;
#pragma unroll
      for (int b = 0; b < 8; ++b) total += v8[b];
#pragma unroll
      for (int d = 8; d >= 1; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
      // lanes 0..15 hold the first group's sum, lanes 16..31 the second's; half jh of this lane's
      // walk is group (jh ^ rh)
      sx[m][0] = __shfl_sync(0xffffffffu, total, 16 * rh);
      sx[m][1] = __shfl_sync(0xffffffffu, total, 16 * (rh ^ 1));
    }
  };

  // Split-K combine.  A contribution is ONE 64-bit atomic add: the partial sum in fixed point
  // (units of 2^-26) in bits 12..63, an arrival count in bits 0..5, a count of non-finite or
  // out-of-range partials in bits 6..11.  Integer addition is associative, so the result does
  // not depend on arrival order (repeat- and replay-exact); whoever reads back the last count
  // converts, writes the output and zeroes the word.  The answer of an add is only needed one
  // unit later, so its round trip hides behind the next unit's lookups.
  unsigned long long pend_old[M], pend_add[M];
  int pend_ru = -1;
  auto settle = [&]() {
    if (pend_ru < 0) return;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      if (((unsigned)pend_old[m] & 63u) == (unsigned)(p.nSB - 1))  // rare: one contribution in nSB
        emit_combined(p, m, pend_ru, lane, pend_old[m] + pend_add[m]);
    }
    pend_ru = -1;
  };
  auto contribute = [&](int m, int ru, float v) {
    if (m == 0) settle();  // the previous unit's answers have long arrived
    const bool fits = fabsf(v) < 2097152.f;  // 2^21: sixteen of them stay inside 52 bits
    pend_add[m] = fits ? ((unsigned long long)__float2ll_rn(v * 67108864.f) << 12) + 1ull : 65ull;
    asm volatile("atom.add.relaxed.gpu.global.u64 %0, [%1], %2;"
                 : "=l"(pend_old[m])
                 : "l"(p.combine + (size_t)m * p.O + ru * kUnitRows + lane), "l"(pend_add[m])
                 : "memory");
    pend_ru = ru;
  };

  // What becomes of a unit's sum over one K block (decided once):
  //   0 group partials to the fp32 workspace   1 final (a single K block): emit
  //   2 carried in registers over the K blocks (a warp with one unit), then combined
  //   3 running sum through the L2-resident partials (several units and several K blocks)
  //   4 one K block per CTA: combined at once
  const int mode = p.group_partials ? 0 : (p.nKB == 1 ? 1 : (nS == 1 ? 4 : (my_count == 1 ? 2 : 3)));
  float carried[M];
#pragma unroll
  for (int m = 0; m < M; ++m) carried[m] = 0.f;
  int c_slot = 0;
  uint32_t c_phase = 0;
  bool dead = false;
  float sx_cur[M][2];

  // ---- the units of this warp for K block kb = kb_begin + s ----
  auto run_block = [&](int s) {
    const int kb = kb_begin + s;
    const bool last_block = s + 1 == nS;
    // an odd G leaves the second group of the last K block empty
    const bool has[2] = {2 * kb + rh < p.G, 2 * kb + (rh ^ 1) < p.G};
    int cu_begin = 0, cu_end = -1;
    bool cu_zeros = false;
    for (int ru = my_first; ru < my_end; ru += kWarps) {
      // unstaged form: this task's scales and zero points were requested a task ago; now request the next task's
      uint32_t sbits[2] = {nx_scale[0], nx_scale[1]}, zp[2] = {nx_zero[0], nx_zero[1]};
      if (!G_::kStageAux) {
        const bool wraps = ru + kWarps >= my_end;
        if (!wraps || !last_block) request_aux(wraps ? kb + 1 : kb, wraps ? my_first : ru + kWarps);
      }
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bars_u32 + (uint32_t)(c_slot * 8), c_phase))) {
        if (lane == 0) atomicExch(p.status, 1u);  // the copy never landed: give up, keep the barriers
        dead = true;
        return;
      }
      const uint32_t wbase = ring_u32 + (uint32_t)(c_slot * G_::kSlotBytes);
      if (G_::kStageAux) {
        // the slot's low address bits are zero (slots are multiples of 256 bytes), so the other
        // group's entry is one flipped bit away
        const uint32_t as = wbase + aux_scale0, az = wbase + aux_zero0;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sbits[0]) : "r"(as));
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sbits[1]) : "r"(as ^ 64u));
        if (any_zeros && (ru < cu_begin || ru >= cu_end)) {  // entering another matrix of the launch: rare
          const int j = locate(ru);
          cu_begin = p.mats[j].ru_begin;
          cu_end = j + 1 < p.n_mats ? p.mats[j + 1].ru_begin : p.nRU;
          cu_zeros = p.mats[j].zeros != nullptr;
        }
        if (cu_zeros) {  // a matrix without zero points stages none: they stay 4
          asm volatile("ld.shared.u8 %0, [%1];" : "=r"(zp[0]) : "r"(az));
          asm volatile("ld.shared.u8 %0, [%1];" : "=r"(zp[1]) : "r"(az ^ 32u));
        }
      }
      // per activation row and group half: an (even byte step, odd byte step) pair of sums of
      // entry(plane 0) + 2 entry(plane 1) - 4 entry(plane 2)
      uint64_t acc[M][2];
      float corr[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
          corr[m][jh] = 0.f;
          acc[m][jh] = 0ull;
        }
      const uint64_t two2 = 0x4000000040000000ull, minus_four2 = 0xc0800000c0800000ull;  // {2.f, 2.f}, {-4.f, -4.f}
      {
        // the rounding correction needs the zero points during the lookups (code - zero = +/-3 is
        // code 7 / 1 at zero point 4 and code 6 / 0 at zero point 3)
        uint32_t flip[2] = {0u, 0u};
        if (CORRECT) {
          flip[0] = zp[0] == 3u ? 0xffffffffu : 0u;
          flip[1] = zp[1] == 3u ? 0xffffffffu : 0u;
        }
        // staged words are fetched one (half, word) step ahead of their use, into two register
        // sets used in turn
        auto fetch = [&](int step, uint32_t (&dst)[3]) {
          const uint32_t wa = wbase + woff[step >> 2][step & 3];
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(dst[0]) : "r"(wa));
          asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(dst[1]) : "r"(wa), "n"(kPlaneTile));
          asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(dst[2]) : "r"(wa), "n"(2 * kPlaneTile));
        };
        auto walk = [&](int step, const uint32_t (&w)[3]) {
          const int jh = step >> 2, jw = step & 3;
          uint32_t plus3 = 0, minus3 = 0;
          if (CORRECT) {
            const uint32_t low = w[0] ^ flip[jh];
            plus3 = low & w[1] & ~w[2];   // code - zero = +3 (the stored high plane is inverted)
            minus3 = low & ~w[1] & w[2];  // code - zero = -3
          }
#pragma unroll
          for (int bp = 0; bp < 2; ++bp) {  // byte steps 2bp (even) and 2bp + 1 (odd) make one packed add
#pragma unroll
            for (int pl = 0; pl < 3; ++pl) {
              const uint32_t a0 = lookup_address(w[pl], 2 * bp, xl[jh][jw][2 * bp]);
              const uint32_t a1 = lookup_address(w[pl], 2 * bp + 1, xl[jh][jw][2 * bp + 1]);
#pragma unroll
              for (int m = 0; m < M; ++m) {  // activation row m sits m * 128 bytes further
                const uint32_t b0 = a0 + (uint32_t)(m * 128), b1 = a1 + (uint32_t)(m * 128);
                acc[m][jh] = pl == 0 ? add2_lds(acc[m][jh], b0, b1) : fma2_lds(acc[m][jh], b0, b1, pl == 1 ? two2 : minus_four2);
              }
            }
            if (CORRECT) {
#pragma unroll
              for (int b = 2 * bp; b < 2 * bp + 2; ++b) {
                const uint32_t ap = lookup_address(plus3, b, xl[jh][jw][b]);
                const uint32_t am = lookup_address(minus3, b, xl[jh][jw][b]);
#pragma unroll
                for (int m = 0; m < M; ++m) corr[m][jh] += lds_at<0>(ap + (uint32_t)(m * 128)) - lds_at<0>(am + (uint32_t)(m * 128));
              }
            }
          }
        };
        uint32_t wa[3], wb[3];
        fetch(0, wa);
#pragma unroll
        for (int step = 0; step < 8; step += 2) {
          fetch(step + 1, wb);
          walk(step, wa);
          if (step + 2 < 8) fetch(step + 2, wa);
          walk(step + 1, wb);
        }
      }

      // all lanes are done with the staged bytes: the slot takes this warp's task kStages ahead
      __syncwarp();
      if (pf_left > 0) issue_next();
      if (++c_slot == kStages) {
        c_slot = 0;
        c_phase ^= 1u;
      }

      const float sc[2] = {G_::kStageAux || has[0] ? bits_to_float((unsigned short)sbits[0], p.scale_dtype) : 0.f,
                           G_::kStageAux || has[1] ? bits_to_float((unsigned short)sbits[1], p.scale_dtype) : 0.f};
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float term[2];
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
          float d = sum2(acc[m][jh]);
          if (any_zeros) d += (4.f - (float)zp[jh]) * sx_cur[m][jh];
          term[jh] = d * sc[jh];
          if (CORRECT) {
            // rounding of scale*(+/-3) in the scale's dtype: the only inexact products
            const float r3 = round_to(3.f * sc[jh], p.scale_dtype);
            term[jh] += corr[m][jh] * (r3 - 3.f * sc[jh]);
          }
        }
        const float both = term[0] + term[1];
        if (mode == 4) {
          contribute(m, ru, both);
        } else if (mode == 2) {
          carried[m] += both;
          if (last_block) contribute(m, ru, carried[m]);
        } else if (mode == 3) {
          // later K blocks of the super-block add to the partial this same thread stored before
          float* slot = &p.partials[((size_t)sb * M + m) * p.O + ru * kUnitRows + lane];
          const float v = (s > 0 ? __ldcg(slot) : 0.f) + both;
          if (last_block)
            contribute(m, ru, v);
          else
            *slot = v;
        } else if (mode == 1) {
          emit(m, ru, both);
        } else {
          const W3Matrix& mat = p.mats[locate(ru)];
          float* ws_out = reinterpret_cast<float*>(mat.out);
          const int lrow = (ru - mat.ru_begin) * kUnitRows + lane;
#pragma unroll
          for (int jh = 0; jh < 2; ++jh)
            if (has[jh]) ws_out[(size_t)(2 * kb + (jh ^ rh)) * mat.O + lrow] = term[jh];
        }
      }
    }
  };
  build(kb_begin, sx_cur);
  for (int t = 2; t < kStages && pf_left > 0; ++t) issue_next();  // the rest of the ring
  __syncthreads();
  for (int s = 0; s < nS; ++s) {
    if (!dead) run_block(s);
    if (s + 1 < nS) {
      __syncthreads();  // everyone has finished reading the tables
      build(kb_begin + s + 1, sx_cur);
      __syncthreads();
    }
  }
  settle();
  if (p.same_input) pdl_wait_prior_grid();  // stream order for everything that comes after this launch
}

struct Plan {
  int slices, S, nSB;
  size_t smem;
};

size_t smem_bytes(int m) {
  switch (m) {
    case 1: return Geom<1>::kSmemBytes;
    case 2: return Geom<2>::kSmemBytes;
    case 3: return Geom<3>::kSmemBytes;
    default: return Geom<4>::kSmemBytes;
  }
}

// ctas_per_sm_for(m) CTAs per SM.  At most kMaxSplits partial sums per output: beyond 16 K blocks one CTA walks
// several K blocks of its rows in turn.  The SMs are dealt over the super-blocks; the CTAs of a
// super-block split its row units.
Plan make_plan(int m, int nKB, int nRU, const DeviceInfo& info) {
  Plan plan;
  plan.S = (nKB + kMaxSplits - 1) / kMaxSplits;
  plan.nSB = (nKB + plan.S - 1) / plan.S;
  int c = ctas_per_sm_for(m) * info.sm_count / plan.nSB;
  if (c < 1) c = 1;
  if (c > nRU) c = nRU;
  plan.slices = c;
  plan.smem = smem_bytes(m);
  return plan;
}

template <int M, bool CORRECT>
int launch(const W3Params& p, const Plan& plan, bool pdl, cudaStream_t stream) {
  // Raising the dynamic shared memory limit is a per-device, per-kernel setting; do it once.
  static std::mutex lock;
  static bool ready[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
  if (device < 0 || device >= 64) return fail(FB_ELIMIT, "device ordinal %d outside 0..63", device);
  {
    std::lock_guard<std::mutex> guard(lock);
    if (!ready[device]) {
      err = cudaFuncSetAttribute(w3_gemv_kernel<M, CORRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
      if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(w3_gemv_kernel)");
      ready[device] = true;
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan.slices, plan.nSB);
  config.blockDim = dim3(Geom<M>::kWarps * 32);
  config.dynamicSmemBytes = plan.smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl && pdl_allowed() ? 1 : 0;
  err = cudaLaunchKernelEx(&config, w3_gemv_kernel<M, CORRECT>, p);
  if (err != cudaSuccess) return cuda_fail(err, "w3_gemv_kernel launch");
  return FB_OK;
}

// Scratch layout, identical for every problem size so that one scratch can serve calls of
// different shapes: [0,256) status word; from byte 16384 the split-K combine words (one 64-bit
// word per activation row and output row, 2 MiB for the largest launch), which are zero between
// calls; after them the fp32 partials that a CTA walking several K blocks keeps between them.
constexpr size_t kCombineOffset = 16384;
constexpr size_t kPartialsOffset = kCombineOffset + (size_t)kMaxM * 65536 * sizeof(unsigned long long);

size_t partial_bytes(int m, int O, int K) {
  const int nKB = (K / 128 + 1) / 2;
  const int S = (nKB + kMaxSplits - 1) / kMaxSplits, nSB = (nKB + S - 1) / S;
  return S > 1 ? (size_t)nSB * m * O * sizeof(float) : 0;
}

}  // namespace

extern "C" size_t fb_w3_gemv_scratch_bytes(int m, int out_features, int in_features) {
  if (m < 1 || m > kMaxM || out_features < 1 || in_features < 128) return 0;
  return kPartialsOffset + partial_bytes(m, out_features, in_features);
}

namespace {

int run_multi(const void* x, int act_dtype, int m, const fb_w3_matrix_t* matrices, int n_matrices, int scale_dtype,
              const int16_t* perm, int in_features, void* scratch, size_t scratch_bytes, unsigned flags,
              fb_stream_t stream, int prologue, const void* prologue_arg, float eps, const fb_w3_push_t* push = nullptr) {
  const int K = in_features;
  if (push) {
    if (m != 1 || n_matrices != 1 || (flags & FB_W3_GROUP_PARTIALS) || matrices[0].residual)
      return fail(FB_EINVAL, "fb_w3_gemv_push: one matrix, M = 1, no residual and no group partials");
    if (push->world < 1 || push->world > 8) return fail(FB_ELIMIT, "fb_w3_gemv_push: world=%d outside 1..8", push->world);
    for (int r = 0; r < push->world; ++r)
      if (!push->data[r] || !aligned(push->data[r], 8))
        return fail(FB_EINVAL, "fb_w3_gemv_push: exchange pointer of rank %d missing or not 8-byte aligned", r);
  }
  if (prologue < 0 || prologue > 3) return fail(FB_EINVAL, "fb_w3_gemv: unknown input transform %d", prologue);
  if (prologue == 3 && (K % 128 || eps < 1.f || eps > 8.f)) return fail(FB_ELIMIT, "fb_w3_gemv_attn_merge: 1..8 splits per head");
  if (prologue != 0 && (m != 1 || perm || !prologue_arg || !aligned(prologue_arg, 16)))
    return fail(FB_EINVAL, "fb_w3_gemv: a fused input transform needs M = 1, identity column order and a 16-byte aligned operand");
  const bool group_partials = (flags & FB_W3_GROUP_PARTIALS) != 0;
  if (!x || !matrices) return fail(FB_EINVAL, "fb_w3_gemv: x and the matrix list must be non-null");
  if (n_matrices < 1 || n_matrices > kMaxMatrices) return fail(FB_ELIMIT, "fb_w3_gemv: %d matrices given, 1..%d supported", n_matrices, kMaxMatrices);
  if ((act_dtype != FB_F16 && act_dtype != FB_BF16) || (scale_dtype != FB_F16 && scale_dtype != FB_BF16))
    return fail(FB_EINVAL, "fb_w3_gemv: dtype tags must be FB_F16 or FB_BF16");
  if (m < 1 || m > kMaxM) return fail(FB_ELIMIT, "fb_w3_gemv: M=%d outside 1..%d", m, kMaxM);
  if (K < 128 || K % 128 || K / 128 > 255) return fail(FB_ELIMIT, "fb_w3_gemv: K=%d must be a multiple of 128 with at most 255 groups", K);
  if (!aligned(x, 16) && !perm) return fail(FB_EINVAL, "fb_w3_gemv: x must be 16-byte aligned");
  if (!aligned(x, 2) || (perm && !aligned(perm, 2))) return fail(FB_EINVAL, "fb_w3_gemv: 16-bit tensors must be 2-byte aligned");
  if (flags & ~(FB_W3_DECODED_BF16 | FB_W3_NO_PDL | FB_W3_GROUP_PARTIALS | FB_W3_SAME_INPUT)) return fail(FB_EINVAL, "fb_w3_gemv: unknown flag bits 0x%x", flags);
  if ((flags & FB_W3_SAME_INPUT) && (prologue != 0 || push || (flags & FB_W3_NO_PDL)))
    return fail(FB_EINVAL, "fb_w3_gemv: FB_W3_SAME_INPUT goes with a plain programmatic launch (no fused input, no push)");
  if (group_partials && (m != 1 || n_matrices != 1)) return fail(FB_EINVAL, "fb_w3_gemv: group partials need M = 1 and a single matrix");
  const int G = K / 128;
  const size_t x_bytes = (size_t)m * K * 2;

  W3Params p;
  p.x = x;
  p.perm = perm;
  p.prologue = prologue;
  p.attn_splits = prologue == 3 ? (int)eps : 0;
  p.prologue_arg = prologue_arg;
  p.eps = eps;
  p.push_world = push ? push->world : 0;
  for (int r = 0; r < 8; ++r) p.push_data[r] = push && r < push->world ? static_cast<unsigned long long*>(push->data[r]) : nullptr;
  p.n_mats = n_matrices;
  long long total = 0;
  for (int j = 0; j < kMaxMatrices; ++j) {
    W3Matrix& mat = p.mats[j];
    if (j >= n_matrices) {
      mat = W3Matrix{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0};
      p.plane_maps[j] = p.plane_maps[0];
      p.scale_maps[j] = p.scale_maps[0];
      p.zero_maps[j] = p.zero_maps[0];
      continue;
    }
    const fb_w3_matrix_t& in = matrices[j];
    const int O = in.out_features;
    if (!in.planes || !in.scales || !in.out) return fail(FB_EINVAL, "fb_w3_gemv: planes, scales and out must be non-null");
    if (O < 32 || O > 65536 || O % 32) return fail(FB_ELIMIT, "fb_w3_gemv: O=%d must be a multiple of 32 in 32..65536", O);
    if (!aligned(in.planes, 16) || !aligned(in.scales, 16) || !aligned(in.zeros, 16))
      return fail(FB_EINVAL, "fb_w3_gemv: planes, scales and zeros must be 16-byte aligned");
    if (!aligned(in.scales, 2) || !aligned(in.out, group_partials ? 4 : 2) || !aligned(in.residual, 2))
      return fail(FB_EINVAL, "fb_w3_gemv: 16-bit tensors must be 2-byte aligned");
    const size_t out_bytes = group_partials ? (size_t)G * O * 4 : (size_t)m * O * 2;
    if (overlaps(in.out, out_bytes, x, x_bytes) || overlaps(in.out, out_bytes, in.planes, (size_t)G * 3 * O * 16) ||
        overlaps(in.out, out_bytes, in.scales, (size_t)G * O * 2))
      return fail(FB_EALIAS, "fb_w3_gemv: out overlaps an input");
    if (scratch && overlaps(scratch, scratch_bytes, in.out, out_bytes)) return fail(FB_EALIAS, "fb_w3_gemv: scratch overlaps out");
    if (!plane_tensor_map(in.planes, O, G, 1, 6, &p.plane_maps[j])) return FB_ECUDA;
    if (m == 1) {  // the M = 1 kernel stages scales and zero points with the planes
      if (!group_row_tensor_map(in.scales, 2, O, G, &p.scale_maps[j])) return FB_ECUDA;
      if (in.zeros && !group_row_tensor_map(in.zeros, 1, O, G, &p.zero_maps[j])) return FB_ECUDA;
      if (!in.zeros) p.zero_maps[j] = p.scale_maps[j];
    } else {
      p.scale_maps[j] = p.plane_maps[j];
      p.zero_maps[j] = p.plane_maps[j];
    }
    mat.planes = in.planes;
    mat.scales = static_cast<const unsigned short*>(in.scales);
    mat.zeros = in.zeros;
    mat.out = in.out;
    mat.residual = in.residual;
    mat.O = O;
    mat.ru_begin = (int)(total / kUnitRows);
    total += O;
  }
  if (total > 65536) return fail(FB_ELIMIT, "fb_w3_gemv: %lld output rows in one launch, at most 65536", total);
  const size_t need = fb_w3_gemv_scratch_bytes(m, (int)total, K);
  if (!scratch || scratch_bytes < need) return fail(FB_ESCRATCH, "fb_w3_gemv: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  if (!aligned(scratch, 256)) return fail(FB_EINVAL, "fb_w3_gemv: scratch must be 256-byte aligned");
  if (overlaps(scratch, need, x, x_bytes)) return fail(FB_EALIAS, "fb_w3_gemv: scratch overlaps x");

  const DeviceInfo* info = device_info();
  if (!info) return FB_ECUDA;
  p.O = (int)total;
  p.K = K;
  p.G = G;
  p.nKB = (G + 1) / 2;
  p.nRU = (int)(total / kUnitRows);
  p.act_dtype = act_dtype;
  p.scale_dtype = scale_dtype;
  unsigned char* base = static_cast<unsigned char*>(scratch);
  p.status = reinterpret_cast<unsigned*>(base);
  p.combine = reinterpret_cast<unsigned long long*>(base + kCombineOffset);
  p.partials = reinterpret_cast<float*>(base + kPartialsOffset);
  const Plan plan = make_plan(m, p.nKB, p.nRU, *info);
  p.S = plan.S;
  p.units_per_slice = p.nRU / plan.slices;
  p.units_extra = p.nRU % plan.slices;
  p.nSB = plan.nSB;
  p.group_partials = group_partials ? 1 : 0;
  p.same_input = (flags & FB_W3_SAME_INPUT) ? 1 : 0;
  if (plan.smem > (size_t)info->max_smem_optin) return fail(FB_ELIMIT, "fb_w3_gemv: plan needs %zu bytes of shared memory", plan.smem);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool correct = (flags & FB_W3_DECODED_BF16) != 0;
  const bool pdl = (flags & FB_W3_NO_PDL) == 0;
#define FB_DISPATCH(MM) \
  case MM:              \
    return correct ? launch<MM, true>(p, plan, pdl, s) : launch<MM, false>(p, plan, pdl, s);
  switch (m) {
    FB_DISPATCH(1)
    FB_DISPATCH(2)
    FB_DISPATCH(3)
    FB_DISPATCH(4)
  }
#undef FB_DISPATCH
  return fail(FB_ELIMIT, "fb_w3_gemv: unsupported M");
}
}  // namespace

extern "C" int fb_w3_gemv_multi(const void* x, int act_dtype, int m, const fb_w3_matrix_t* matrices, int n_matrices,
                                int scale_dtype, const int16_t* perm, int in_features, void* scratch,
                                size_t scratch_bytes, unsigned flags, fb_stream_t stream) {
  return run_multi(x, act_dtype, m, matrices, n_matrices, scale_dtype, perm, in_features, scratch, scratch_bytes, flags, stream,
                   0, nullptr, 0.f);
}

extern "C" int fb_w3_gemv_fused_input(const void* x, int act_dtype, int transform, const void* operand, float eps,
                                      const fb_w3_matrix_t* matrices, int n_matrices, int scale_dtype, int in_features,
                                      void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream) {
  if (transform != FB_W3_INPUT_RMSNORM && transform != FB_W3_INPUT_SILU_MUL)
    return fail(FB_EINVAL, "fb_w3_gemv_fused_input: transform must be FB_W3_INPUT_RMSNORM or FB_W3_INPUT_SILU_MUL");
  return run_multi(x, act_dtype, 1, matrices, n_matrices, scale_dtype, nullptr, in_features, scratch, scratch_bytes, flags, stream,
                   transform, operand, eps);
}

extern "C" int fb_w3_gemv_attn_merge(const void* partials, int splits, int act_dtype, const fb_w3_matrix_t* matrices, int n_matrices,
                                     int scale_dtype, int in_features, void* scratch, size_t scratch_bytes, unsigned flags,
                                     fb_stream_t stream) {
  if (splits < 1 || splits > 8) return fail(FB_ELIMIT, "fb_w3_gemv_attn_merge: %d splits per head, 1..8 supported", splits);
  // the partials stand in for x (head h, split s at float offset (16 h + s) * 132) and are the transform's operand
  return run_multi(partials, act_dtype, 1, matrices, n_matrices, scale_dtype, nullptr, in_features, scratch, scratch_bytes, flags, stream,
                   3, partials, (float)splits);
}

extern "C" int fb_w3_gemv_push(const void* x, int act_dtype, int transform, const void* operand, float eps,
                               const fb_w3_matrix_t* matrix, int scale_dtype, int in_features, const fb_w3_push_t* push,
                               void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream) {
  if (!push || !matrix) return fail(FB_EINVAL, "fb_w3_gemv_push: matrix and push descriptor must be non-null");
  if (transform != 0 && transform != FB_W3_INPUT_RMSNORM && transform != FB_W3_INPUT_SILU_MUL && transform != FB_W3_INPUT_ATTN_PIECES)
    return fail(FB_EINVAL, "fb_w3_gemv_push: unknown input transform %d", transform);
  if (transform == FB_W3_INPUT_ATTN_PIECES) operand = x;  // the pieces are both the activations and the transform's operand
  return run_multi(x, act_dtype, 1, matrix, 1, scale_dtype, nullptr, in_features, scratch, scratch_bytes, flags, stream, transform,
                   operand, eps, push);
}

extern "C" int fb_w3_gemv(const void* x, int act_dtype, int m, const uint8_t* planes, const void* scales,
                          int scale_dtype, const uint8_t* zeros, const int16_t* perm, void* out,
                          int out_features, int in_features, void* scratch, size_t scratch_bytes,
                          unsigned flags, fb_stream_t stream) {
  fb_w3_matrix_t one = {planes, scales, zeros, out, nullptr, out_features};
  return fb_w3_gemv_multi(x, act_dtype, m, &one, 1, scale_dtype, perm, in_features, scratch, scratch_bytes, flags, stream);
}

namespace {
__global__ void w3_finish_kernel(const float* __restrict__ partials, int splits, int O, void* out, int dtype) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= O) return;
  float total = 0.f;
  for (int s = 0; s < splits; ++s) total += partials[(size_t)s * O + o];
  fb::store_act(out, dtype, o, total);
}
}  // namespace

extern "C" int fb_w3_finish(const float* partials, int splits, int out_features, void* out, int out_dtype,
                            fb_stream_t stream) {
  using namespace fb;
  if (!partials || !out) return fail(FB_EINVAL, "fb_w3_finish: null pointer");
  if (out_dtype != FB_F16 && out_dtype != FB_BF16) return fail(FB_EINVAL, "fb_w3_finish: out dtype must be FB_F16 or FB_BF16");
  if (splits < 1 || splits > 255 || out_features < 1 || out_features > 65536) return fail(FB_ELIMIT, "fb_w3_finish: dimensions outside bounds");
  if (overlaps(out, (size_t)out_features * 2, partials, (size_t)splits * out_features * 4)) return fail(FB_EALIAS, "fb_w3_finish: out overlaps partials");
  w3_finish_kernel<<<(out_features + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(partials, splits, out_features, out, out_dtype);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_fail(err, "w3_finish_kernel launch");
  return FB_OK;
}
