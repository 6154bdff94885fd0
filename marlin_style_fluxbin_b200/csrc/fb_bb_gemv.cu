// Two-base binary-basis GEMV, M = 1:  W ~ sum_b diag(row_b) * B_b * diag(col_b), B_b in {-1,+1},
// packed one bit per weight per base, in groups of 128 inputs.
//
// Same skeleton as the W3 GEMV (HBM-bound byte work, see fb_w3_gemv.cu): a K block is TWO groups
// (one for matrices of fewer than 128 row units);
// a CTA holds 32 signed activation tables per group (2 bases x 16 chunks of 8 inputs, entries are
// sums of +/- x*col in ascending order) laid out entry-major so that the bank of a lookup is the
// table number; lane = output row; lanes walk the 32 (base, chunk) pairs of a group in a
// lane-rotated order so that lookups and staged-word reads are bank-conflict free; a warp's rows
// are, per group, one contiguous run of 32-byte code rows, staged by a bulk copy; the split over
// the K blocks is combined in the kernel by one 64-bit fixed-point atomic add per contribution
// (order-independent, repeat-exact).  Two groups per unit halve the fixed cost per byte of a unit
// (staging, scale loads, the returning atomic) and the atomics per output row.
//
// Two scale conventions:
//  * group mode (the reference's hybrid g128-s8 payload, deployment.py:23-27, kernel
//    csrc/m1_v5.cu:27-104): fp32 row scales per (group,row,base), fp32 column scales per
//    (group,input,base), plus a two-base refinement on 8 selected columns per group (two more
//    tables).  Codes may be planar [G,O,2,16] or interleaved [G,O,32].
//  * global mode (matrix-wide fp16 scales r_b[O], c_b[K], planar codes, and `n_sal` dense bf16
//    residual columns): the per-base sums are kept separate through the K split and the row
//    scales and the residual are applied once, by whoever reduces a row.
#include <mutex>

#include "fb_common.cuh"

namespace {

using namespace fb;

constexpr int kUnitRows = 32;
constexpr int kGroupBytes = kUnitRows * 32;  // 1 KB of codes per unit and group
constexpr int kWarps = 8;
constexpr int kCtasPerSm = 2;
constexpr int kMaxSlots = 4;                // staged units per warp: at most 4 KB in flight per warp
constexpr int kGroupLutBytes = 32768;       // 256 entries x 32 tables x 4 B
constexpr int kGroupSparseBytes = 2048;     // 2 tables x 256 entries

struct BBParams {
  const void* x;
  const uint8_t* codes;
  const float* rows;
  const float* cols;
  const uint8_t* sparse;
  const float* srows;
  const float* scols;
  const int16_t* indices;
  const __half* grow;
  const __half* gcol;
  const int32_t* sal_idx;
  const __nv_bfloat16* sal;
  void* out;
  unsigned long long* combine;  // [O] split-K accumulators, zero between launches
  unsigned* status;
  int O, K, G, nKB, nRU;
  int act_dtype, interleaved, global_mode, n_sal;
  int slots, ctas_per_kb;
};

// one base's eight sign bits out of sixteen interleaved bits (reference csrc/lut8.cuh:10-15)
__device__ __forceinline__ uint32_t compact_even(uint32_t word) {
  word &= 0x5555u;
  word = (word | (word >> 1)) & 0x3333u;
  word = (word | (word >> 2)) & 0x0f0fu;
  return (word | (word >> 4)) & 0xffu;
}

template <bool INTERLEAVED, bool GLOBAL, int GPB>
__global__ void __launch_bounds__(kWarps * 32, kCtasPerSm) bb_gemv_kernel(const BBParams p) {
  constexpr int kBlockGroups = GPB;
  constexpr int kUnitBytes = GPB * kGroupBytes;  // staged per unit
  constexpr int kLutBytes = GPB * kGroupLutBytes, kSparseLutBytes = GPB * kGroupSparseBytes;
  extern __shared__ __align__(1024) unsigned char smem[];
  // the warp index through a shuffle, so that the compiler knows it is the same in all lanes (uniform registers)
  const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int S = p.slots;
  unsigned char* const lut = smem;
  float* const sparse_lut = reinterpret_cast<float*>(smem + kLutBytes);
  unsigned char* const stage_base = smem + kLutBytes + kSparseLutBytes + (size_t)warp * S * kUnitBytes;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(smem + kLutBytes + kSparseLutBytes + (size_t)kWarps * S * kUnitBytes) + warp * (kMaxSlots + 1);
  const uint32_t stage_u32 = smem_u32(stage_base);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int nV = p.nKB * p.ctas_per_kb;
  if ((int)blockIdx.x >= nV) return;

  if (lane == 0)
    for (int s = 0; s <= kMaxSlots; ++s) mbar_init(smem_u32(&bars[s]), 1);
  mbar_init_fence();
  __syncwarp();

  auto share = [&](int v, int& kb, int& first, int& count) {
    kb = v / p.ctas_per_kb;
    const int slice = v - kb * p.ctas_per_kb;
    const int ua = (int)((long long)slice * p.nRU / p.ctas_per_kb);
    const int ub = (int)((long long)(slice + 1) * p.nRU / p.ctas_per_kb);
    const int n = ub - ua, q = n / kWarps, r = n - q * kWarps;
    first = ua + warp * q + min(warp, r);
    count = q + (warp < r ? 1 : 0);
  };
  // n units from `first` into slots slot.., one bulk copy per unit and group; rows past O in the
  // last unit are never copied (the copy is clipped) and never stored
  auto stage_units = [&](int kb, int first, int n, int slot, int bar_index) {
    if (lane == 0) {
      const int ngroups = min(kBlockGroups, p.G - kBlockGroups * kb);
      const uint32_t bar = smem_u32(&bars[bar_index]);
      int total = 0;
      for (int u = 0; u < n; ++u) total += min(kUnitRows, p.O - (first + u) * kUnitRows) * 32 * ngroups;
      mbar_expect_tx(bar, (uint32_t)total);
      for (int u = 0; u < n; ++u) {
        const int rows = min(kUnitRows, p.O - (first + u) * kUnitRows);
        for (int gi = 0; gi < ngroups; ++gi)
          bulk_g2s(stage_u32 + (uint32_t)((slot + u) * kUnitBytes + gi * kGroupBytes),
                   p.codes + ((size_t)(kBlockGroups * kb + gi) * p.O + (size_t)(first + u) * kUnitRows) * 32, (uint32_t)(rows * 32), bar);
      }
    }
  };

  const int rb = lane & 3, rw = (lane >> 2) & 3, rh = (lane >> 4) & 1;
  // Lookups use 32-bit shared-window addresses: entry * 128 + table offset is ONE dp4a (a byte
  // dot product whose only non-zero weight, 128, sits at the wanted byte of the staged word).
  const uint32_t lut_u32 = smem_u32(lut);
  uint32_t sel[4];
#pragma unroll
  for (int b = 0; b < 4; ++b) sel[b] = 128u << (8 * ((b + rb) & 3));
  auto lookup = [&](uint32_t word, int b, uint32_t table) {
    uint32_t address;
    float value;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(address) : "r"(word), "r"(sel[b]), "r"(table));
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(value) : "r"(address));
    return value;
  };
  uint32_t chunk_parity = 0, slot_parity = 0;
  bool dead = false, first_pass = true;
  int kb, my_first, my_count;
  share((int)blockIdx.x, kb, my_first, my_count);
  if (my_count > 0) stage_units(kb, my_first, min(S, my_count), 0, kMaxSlots);

  asm volatile("griddepcontrol.wait;" ::: "memory");

  // Split over the K blocks: every contribution is ONE 64-bit atomic add carrying the scaled
  // partial sum in fixed point (steps of 2^-26, bits 16..63), an arrival count (bits 0..7) and a
  // count of partials that are not finite or too large for the format (bits 8..15).  Integer
  // adds commute, so the result is independent of arrival order; whoever reads back the last
  // count converts, writes the output and zeroes the word.  The answer is looked at one unit
  // later, so its round trip hides behind the next unit's lookups.
  unsigned long long pend_old = 0ull, pend_add = 0ull;
  int pend_row = -1;
  auto settle = [&]() {
    if (pend_row < 0) return;
    if (((unsigned)pend_old & 255u) == (unsigned)(p.nKB - 1)) {
      const unsigned long long total = pend_old + pend_add;
      float value = __ll2float_rn((long long)total >> 16) * 1.4901161193847656e-08f;  // 2^-26
      if ((total >> 8) & 255ull) value = __int_as_float(0x7fc00000);
      store_act(p.out, p.act_dtype, pend_row, value);
      p.combine[pend_row] = 0ull;
    }
    pend_row = -1;
  };

  for (int v = (int)blockIdx.x; v < nV; v += (int)gridDim.x) {
    if (!first_pass) {
      __syncthreads();  // everyone has finished reading the previous tables
      share(v, kb, my_first, my_count);
      if (!dead && my_count > 0) stage_units(kb, my_first, min(S, my_count), 0, kMaxSlots);
    }
    first_pass = false;
    const int ngroups = min(kBlockGroups, p.G - kBlockGroups * kb);

    float sal_x[kBlockGroups] = {};
    // ---- 32 signed tables per group: lane = table (base = lane/16, chunk = lane%16), warp = 32 entries ----
#pragma unroll
    for (int gi = 0; gi < kBlockGroups; ++gi) {
      const int g = kBlockGroups * kb + gi;
      const int base = lane >> 4, chunk = lane & 15;
      float v8[8];
      if (gi < ngroups) {
        // eight activations (and, with matrix-wide scales, eight fp16 column scales) in one 16-byte load each
        const int k0 = g * 128 + chunk * 8;
        const uint4 xr = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.x) + k0);
        const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w};
        uint32_t cw[4] = {0u, 0u, 0u, 0u};
        if (GLOBAL) {
          const uint4 cr = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.gcol) + (size_t)base * p.K + k0);
          cw[0] = cr.x, cw[1] = cr.y, cw[2] = cr.z, cw[3] = cr.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xv = bits_to_float((unsigned short)((xw[j >> 1] >> (16 * (j & 1))) & 0xffffu), p.act_dtype);
          const float cv = GLOBAL ? __half2float(__ushort_as_half((unsigned short)((cw[j >> 1] >> (16 * (j & 1))) & 0xffffu)))
                                  : p.cols[(size_t)(k0 + j) * 2 + base];
          v8[j] = __fmul_rn(xv, cv);
        }
      } else {  // an odd number of groups: the second half of the last K block is empty
#pragma unroll
        for (int j = 0; j < 8; ++j) v8[j] = 0.f;
      }
      // the salient input this group's contribution carries (matrix-wide scales): fetched once per group
      if (GLOBAL && gi < ngroups && g < p.n_sal) sal_x[gi] = load_act(p.x, p.act_dtype, p.sal_idx[g]);
      // entry(p) = sum_b (bit b of p ? +v_b : -v_b) = low-nibble part + high-nibble part.  Warp w
      // owns the entries whose low nibble is 2w or 2w+1; the sixteen high-nibble parts come from
      // a tree (one add each), so an entry costs one add and one store.
      unsigned char* const column = lut + gi * kGroupLutBytes + lane * 4;
      float hi[16];
      hi[0] = ((-v8[4] - v8[5]) - v8[6]) - v8[7];
#pragma unroll
      for (int h = 1; h < 16; ++h) {
        const int top = h >= 8 ? 3 : (h >= 4 ? 2 : (h >= 2 ? 1 : 0));
        hi[h] = hi[h & ~(1 << top)] + 2.f * v8[4 + top];
      }
#pragma unroll
      for (int qq = 0; qq < 16 / kWarps; ++qq) {
        const int q = warp * (16 / kWarps) + qq;
        float lo = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) lo += ((q >> b) & 1) ? v8[b] : -v8[b];
#pragma unroll
        for (int h = 0; h < 16; ++h) *reinterpret_cast<float*>(column + (size_t)(h * 16 + q) * 128) = lo + hi[h];
      }
      if (!GLOBAL && gi < ngroups) {
        // two refinement tables over the group's 8 selected columns; warp w fills entries 32w..32w+31
        const int pp = warp * 32 + lane;
#pragma unroll
        for (int base2 = 0; base2 < 2; ++base2) {
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int idx = p.indices[g * 8 + j];
            const float sv = __fmul_rn(load_act(p.x, p.act_dtype, g * 128 + idx), p.scols[(size_t)(g * 8 + j) * 2 + base2]);
            sum += ((pp >> j) & 1) ? sv : -sv;
          }
          sparse_lut[gi * 512 + base2 * 256 + pp] = sum;
        }
      }
    }
    __syncthreads();

    const int chunk_units = min(S, my_count);
    for (int i = 0; i < my_count; ++i) {
      const int slot = i % S;
      const int ru = my_first + i;
      const int row = ru * kUnitRows + lane;
      const bool live = row < p.O;
      float2 rs[kBlockGroups], srs[kBlockGroups];
      unsigned sp[kBlockGroups] = {};
      uint32_t g0bits = 0, g1bits = 0;
      uint32_t sal_bits[kBlockGroups] = {};
#pragma unroll
      for (int gi = 0; gi < kBlockGroups; ++gi) {
        const int g = kBlockGroups * kb + gi;
        rs[gi] = make_float2(0.f, 0.f);
        srs[gi] = make_float2(0.f, 0.f);
        if (GLOBAL && live && gi < ngroups && g < p.n_sal)
          asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(sal_bits[gi]) : "l"(p.sal + (size_t)row * p.n_sal + g));
        if (!GLOBAL && live && gi < ngroups) {
          rs[gi] = *reinterpret_cast<const float2*>(p.rows + ((size_t)g * p.O + row) * 2);
          srs[gi] = *reinterpret_cast<const float2*>(p.srows + ((size_t)g * p.O + row) * 2);
          sp[gi] = *reinterpret_cast<const unsigned short*>(p.sparse + ((size_t)g * p.O + row) * 2);
        }
      }
      if (GLOBAL && live) {
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(g0bits) : "l"(p.grow + row));
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(g1bits) : "l"(p.grow + (size_t)p.O + row));
      }

      bool ok = false;
      if (!dead) {
        if (i < chunk_units)
          ok = mbar_wait_bounded(smem_u32(&bars[kMaxSlots]), chunk_parity);
        else
          ok = mbar_wait_bounded(smem_u32(&bars[slot]), (slot_parity >> slot) & 1u);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && !dead) {
        dead = true;
        if (lane == 0) atomicExch(p.status, 1u);
      }
      if (i >= chunk_units) slot_parity ^= 1u << slot;

      float d0[kBlockGroups] = {}, d1[kBlockGroups] = {};
      if (!dead) {
#pragma unroll
        for (int gi = 0; gi < kBlockGroups; ++gi) {
          if (gi >= ngroups) break;  // nothing was staged for an empty second group
          const unsigned char* const buf = stage_base + slot * kUnitBytes + gi * kGroupBytes + lane * 32;
          const uint32_t buf_u32 = stage_u32 + (uint32_t)(slot * kUnitBytes + gi * kGroupBytes + lane * 32);
          const uint32_t group_lut = lut_u32 + (uint32_t)(gi * kGroupLutBytes);
          if (!INTERLEAVED) {
            // row = [base 0: 16 bytes][base 1: 16 bytes]; steps with jh = 0 serve base rh
            float acc[2] = {0.f, 0.f};
#pragma unroll
            for (int jh = 0; jh < 2; ++jh) {
              const int h = jh ^ rh;
#pragma unroll
              for (int jw = 0; jw < 4; ++jw) {
                const int ws = (jw + rw) & 3;
                uint32_t w;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(buf_u32 + (uint32_t)(h * 16 + ws * 4)));
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[jh] += lookup(w, b, group_lut + (uint32_t)(64 * h + 16 * ws + 4 * ((b + rb) & 3)));
              }
            }
            d0[gi] = rh ? acc[1] : acc[0];
            d1[gi] = rh ? acc[0] : acc[1];
          } else {
            // row = 16 little-endian 16-bit words, word c holds chunk c of both bases, bits
            // interleaved.  A 32-bit read gives chunks 2w and 2w+1; sub-step b picks
            // (chunk half, base) = ((b+rb)&1, (b+rb)>>1 & 1).
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int jh = 0; jh < 2; ++jh) {
#pragma unroll
              for (int jw = 0; jw < 4; ++jw) {
                const int w8 = 4 * (jh ^ rh) + ((jw + rw) & 3);
                const uint32_t w = *reinterpret_cast<const uint32_t*>(buf + w8 * 4);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const int combo = (b + rb) & 3, half = combo & 1, base = combo >> 1;
                  const uint32_t entry = compact_even((w >> (16 * half)) >> base);
                  acc[b] += *reinterpret_cast<const float*>(lut + gi * kGroupLutBytes + entry * 128 + 4 * (16 * base + 2 * w8 + half));
                }
              }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              if ((((b + rb) & 3) >> 1) == 0) d0[gi] += acc[b]; else d1[gi] += acc[b];
            }
          }
        }
      }

      __syncwarp();
      if (!dead && i + S < my_count) stage_units(kb, my_first + i + S, 1, slot, slot);

      settle();  // the previous unit's answer has long arrived
      if (!dead && live) {
        float value = 0.f;
        if (GLOBAL) {
          asm volatile("" : "+r"(g0bits), "+r"(g1bits));  // first use: after the lookups
          const float r0 = __half2float(__ushort_as_half((unsigned short)g0bits)), r1 = __half2float(__ushort_as_half((unsigned short)g1bits));
#pragma unroll
          for (int gi = 0; gi < kBlockGroups; ++gi) {
            if (gi >= ngroups) break;
            const int g = kBlockGroups * kb + gi;
            value = __fmaf_rn(r0, d0[gi], value);
            value = __fmaf_rn(r1, d1[gi], value);
            // the dense residual columns are dealt round-robin over the groups' contributions
            if (g < p.n_sal) {
              asm volatile("" : "+r"(sal_bits[gi]));
              value = __fmaf_rn(__uint_as_float(sal_bits[gi] << 16), sal_x[gi], value);
            }
            for (int sidx = g + p.G; sidx < p.n_sal; sidx += p.G)  // more salient columns than groups: rare
              value = __fmaf_rn(__bfloat162float(p.sal[(size_t)row * p.n_sal + sidx]), load_act(p.x, p.act_dtype, p.sal_idx[sidx]), value);
          }
        } else {
#pragma unroll
          for (int gi = 0; gi < kBlockGroups; ++gi) {
            if (gi >= ngroups) break;
            const uint32_t p0 = INTERLEAVED ? compact_even(sp[gi]) : (sp[gi] & 0xffu);
            const uint32_t p1 = INTERLEAVED ? compact_even(sp[gi] >> 1) : (sp[gi] >> 8);
            value = __fmaf_rn(rs[gi].x, d0[gi], value);
            value = __fmaf_rn(rs[gi].y, d1[gi], value);
            value = __fmaf_rn(srs[gi].x, sparse_lut[gi * 512 + p0], value);
            value = __fmaf_rn(srs[gi].y, sparse_lut[gi * 512 + 256 + p1], value);
          }
        }
        if (p.nKB == 1) {
          store_act(p.out, p.act_dtype, row, value);
        } else {
          const bool fits = fabsf(value) < 8192.f;  // 255 of them stay inside 48 bits
          pend_add = fits ? ((unsigned long long)__float2ll_rn(value * 67108864.f) << 16) + 1ull : 257ull;
          asm volatile("atom.add.relaxed.gpu.global.u64 %0, [%1], %2;" : "=l"(pend_old) : "l"(p.combine + row), "l"(pend_add) : "memory");
          pend_row = row;
        }
      }
    }
    if (my_count > 0) chunk_parity ^= 1u;
  }

  settle();
}

constexpr size_t kCombineOffset = 16384;  // after the status block: one 64-bit word per output row

template <bool INTERLEAVED, bool GLOBAL, int GPB>
int launch(const BBParams& p, int grid, size_t smem, int max_smem, bool pdl, cudaStream_t stream) {
  static std::mutex lock;
  static bool ready[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  {
    std::lock_guard<std::mutex> guard(lock);
    if (!ready[device]) {
      cudaError_t err = cudaFuncSetAttribute(bb_gemv_kernel<INTERLEAVED, GLOBAL, GPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
      if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute(bb_gemv_kernel)");
      ready[device] = true;
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kWarps * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = pdl && pdl_allowed() ? 1 : 0;
  cudaError_t err = cudaLaunchKernelEx(&config, bb_gemv_kernel<INTERLEAVED, GLOBAL, GPB>, p);
  if (err != cudaSuccess) return cuda_fail(err, "bb_gemv_kernel launch");
  return FB_OK;
}

int run(BBParams& p, void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream, const char* who) {
  const size_t need = kCombineOffset + (size_t)p.O * sizeof(unsigned long long);
  if (!scratch || scratch_bytes < need) return fail(FB_ESCRATCH, "%s: scratch of %zu bytes needed, %zu given", who, need, scratch_bytes);
  if (!aligned(scratch, 256)) return fail(FB_EINVAL, "%s: scratch must be 256-byte aligned", who);
  const DeviceInfo* info = device_info();
  if (!info) return FB_ECUDA;
  unsigned char* base = static_cast<unsigned char*>(scratch);
  p.status = reinterpret_cast<unsigned*>(base);
  p.combine = reinterpret_cast<unsigned long long*>(base + kCombineOffset);
  p.nRU = (p.O + kUnitRows - 1) / kUnitRows;
  // Two groups per K block halve the per-byte cost of a unit; with few row units the second table
  // build on the critical path costs more than that saves.
  const int gpb = p.nRU >= 128 && p.G >= 2 ? 2 : 1;
  p.nKB = (p.G + gpb - 1) / gpb;
  int c = kCtasPerSm * info->sm_count / p.nKB;
  if (c < 1) c = 1;
  if (c > p.nRU) c = p.nRU;
  p.ctas_per_kb = c;
  const int nV = p.nKB * c;
  const int grid = nV < kCtasPerSm * info->sm_count ? nV : kCtasPerSm * info->sm_count;
  const int per_warp = ((p.nRU + c - 1) / c + kWarps - 1) / kWarps;
  const int max_slots = kMaxSlots / gpb;
  p.slots = per_warp < max_slots ? (per_warp < 1 ? 1 : per_warp) : max_slots;
  const size_t smem = (size_t)gpb * (kGroupLutBytes + kGroupSparseBytes) + (size_t)kWarps * p.slots * gpb * kGroupBytes + (size_t)kWarps * (kMaxSlots + 1) * 8;
  const bool pdl = (flags & FB_W3_NO_PDL) == 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (gpb == 2) {
    if (p.global_mode) return launch<false, true, 2>(p, grid, smem, info->max_smem_optin, pdl, s);
    if (p.interleaved) return launch<true, false, 2>(p, grid, smem, info->max_smem_optin, pdl, s);
    return launch<false, false, 2>(p, grid, smem, info->max_smem_optin, pdl, s);
  }
  if (p.global_mode) return launch<false, true, 1>(p, grid, smem, info->max_smem_optin, pdl, s);
  if (p.interleaved) return launch<true, false, 1>(p, grid, smem, info->max_smem_optin, pdl, s);
  return launch<false, false, 1>(p, grid, smem, info->max_smem_optin, pdl, s);
}

int check_common(const char* who, const void* x, int act_dtype, const uint8_t* codes, void* out, int O, int K) {
  if (!x || !codes || !out) return fail(FB_EINVAL, "%s: x, codes and out must be non-null", who);
  if (act_dtype != FB_F16 && act_dtype != FB_BF16) return fail(FB_EINVAL, "%s: activation dtype must be FB_F16 or FB_BF16", who);
  if (K < 128 || K % 128 || K / 128 > 255) return fail(FB_ELIMIT, "%s: K=%d must be a multiple of 128 with at most 255 groups", who, K);
  if (O < 1 || O > 65536) return fail(FB_ELIMIT, "%s: O=%d outside 1..65536", who, O);
  if (!aligned(codes, 16)) return fail(FB_EINVAL, "%s: codes must be 16-byte aligned", who);
  if (overlaps(out, (size_t)O * 2, x, (size_t)K * 2) || overlaps(out, (size_t)O * 2, codes, (size_t)(K / 128) * O * 32))
    return fail(FB_EALIAS, "%s: out overlaps an input", who);
  return FB_OK;
}

}  // namespace

extern "C" size_t fb_bb_gemv_scratch_bytes(int out_features, int in_features, int global_scales) {
  if (out_features < 1 || in_features < 128) return 0;
  (void)global_scales;
  return kCombineOffset + (size_t)out_features * sizeof(unsigned long long);
}

extern "C" int fb_bb_gemv(const void* x, int act_dtype, const uint8_t* codes, int planar, const float* rows,
                          const float* cols, const uint8_t* sparse_codes, const float* sparse_rows,
                          const float* sparse_cols, const int16_t* indices, void* out, int out_features,
                          int in_features, void* scratch, size_t scratch_bytes, unsigned flags, fb_stream_t stream) {
  int rc = check_common("fb_bb_gemv", x, act_dtype, codes, out, out_features, in_features);
  if (rc) return rc;
  if (!rows || !cols || !sparse_codes || !sparse_rows || !sparse_cols || !indices)
    return fail(FB_EINVAL, "fb_bb_gemv: every payload tensor must be non-null");
  if (!aligned(rows, 8) || !aligned(sparse_rows, 8) || !aligned(sparse_codes, 2) || !aligned(cols, 4) || !aligned(sparse_cols, 4))
    return fail(FB_EINVAL, "fb_bb_gemv: scale tensors are misaligned");
  if (flags & ~FB_W3_NO_PDL) return fail(FB_EINVAL, "fb_bb_gemv: unknown flag bits 0x%x", flags);
  BBParams p = {};
  p.x = x; p.codes = codes; p.rows = rows; p.cols = cols; p.sparse = sparse_codes; p.srows = sparse_rows;
  p.scols = sparse_cols; p.indices = indices; p.out = out; p.O = out_features; p.K = in_features;
  p.G = in_features / 128; p.act_dtype = act_dtype; p.interleaved = planar ? 0 : 1; p.global_mode = 0;
  return run(p, scratch, scratch_bytes, flags, stream, "fb_bb_gemv");
}

extern "C" int fb_bb_global_gemv(const void* x, int act_dtype, const uint8_t* codes, const void* row_scales,
                                 const void* col_scales, const int32_t* salient_idx, const void* salient,
                                 int n_salient, void* out, int out_features, int in_features, void* scratch,
                                 size_t scratch_bytes, unsigned flags, fb_stream_t stream) {
  int rc = check_common("fb_bb_global_gemv", x, act_dtype, codes, out, out_features, in_features);
  if (rc) return rc;
  if (!row_scales || !col_scales) return fail(FB_EINVAL, "fb_bb_global_gemv: scales must be non-null");
  if (n_salient < 0 || n_salient > 256 || (n_salient > 0 && (!salient_idx || !salient)))
    return fail(FB_EINVAL, "fb_bb_global_gemv: salient columns: 0..256 with index and value tensors");
  if (flags & ~FB_W3_NO_PDL) return fail(FB_EINVAL, "fb_bb_global_gemv: unknown flag bits 0x%x", flags);
  BBParams p = {};
  p.x = x; p.codes = codes; p.grow = static_cast<const __half*>(row_scales); p.gcol = static_cast<const __half*>(col_scales);
  p.sal_idx = salient_idx; p.sal = static_cast<const __nv_bfloat16*>(salient); p.n_sal = n_salient; p.out = out;
  p.O = out_features; p.K = in_features; p.G = in_features / 128; p.act_dtype = act_dtype; p.global_mode = 1;
  return run(p, scratch, scratch_bytes, flags, stream, "fb_bb_global_gemv");
}
