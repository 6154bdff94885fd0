/*
 * CPU oracle for the batch-1 packed-Linear decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference project's Python
 * reference functions and CUDA kernels for this path.  It is the checker that the
 * parity tests, the smoke test and the CPU-baseline leg of the benchmark call; the
 * product (the CUDA library) never links, loads or calls it.
 *
 * Parity is pinned: tests/test_oracle_golden.py checks every function below against
 * fixtures produced by running the reference's own Python code
 * (tests/golden/make_golden.py) and against the known answers the reference's tests
 * hold (10-1-10-1-10 boundary word layout, the two-base byte 0b11100100, the 65 536
 * interleaved patterns).
 *
 * Half-precision values cross this ABI as raw 16-bit patterns (uint16_t) together
 * with a dtype tag: FBO_F16 = 0, FBO_BF16 = 1, FBO_F32 = 2 (float storage).
 *
 * Each function cites the reference file:line it follows (paths are relative to the
 * reference project's root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FBO_F16 0
#define FBO_BF16 1
#define FBO_F32 2
#define FBO_GROUP 128

/* ------------------------------------------------------------------ scalars */

static inline float bf16_bits_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16_bits(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float f16_bits_to_f32(uint16_t b) {
  _Float16 h;
  memcpy(&h, &b, 2);
  return (float)h;
}

static inline uint16_t f32_to_f16_bits(float f) {
  _Float16 h = (_Float16)f; /* round to nearest even */
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}

static inline float half_to_f32(uint16_t b, int dtype) {
  return dtype == FBO_BF16 ? bf16_bits_to_f32(b) : f16_bits_to_f32(b);
}

static inline uint16_t f32_to_half(float f, int dtype) {
  return dtype == FBO_BF16 ? f32_to_bf16_bits(f) : f32_to_f16_bits(f);
}

/* value of x rounded to the 16-bit dtype, as a float */
static inline float round_to(float f, int dtype) {
  if (dtype == FBO_F32) return f;
  return half_to_f32(f32_to_half(f, dtype), dtype);
}

int fbo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the parallel loops (a launcher may have exported OMP_NUM_THREADS=1). */
void fbo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void fbo_convert_to_f32(const uint16_t* src, int dtype, int64_t n, float* dst) {
  for (int64_t i = 0; i < n; ++i) dst[i] = half_to_f32(src[i], dtype);
}

void fbo_convert_from_f32(const float* src, int dtype, int64_t n, uint16_t* dst) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_half(src[i], dtype);
}

/* ------------------------------------------------- GPTQ 10-1-10-1-10 words */

/* 32 three-bit codes <-> three 32-bit words.  Code 10 straddles words 0/1 (two low
 * bits in bits 30..31 of word 0, its high bit in bit 0 of word 1); code 21 straddles
 * words 1/2 (its low bit in bit 31 of word 1, two high bits in bits 0..1 of word 2).
 * Follows gptq_deployment.py:25-32 (shift table) and :42-72 (_unpack_10_1_10_1_10),
 * and the packer :331-348 (pack_gptq_w3_codes). */
static void unpack32(const uint32_t w[3], uint8_t c[32]) {
  for (int i = 0; i < 10; ++i) c[i] = (w[0] >> (3 * i)) & 7u;
  c[10] = (uint8_t)(((w[0] >> 30) & 3u) | ((w[1] & 1u) << 2));
  for (int i = 0; i < 10; ++i) c[11 + i] = (w[1] >> (1 + 3 * i)) & 7u;
  c[21] = (uint8_t)(((w[1] >> 31) & 1u) | ((w[2] & 3u) << 1));
  for (int i = 0; i < 10; ++i) c[22 + i] = (w[2] >> (2 + 3 * i)) & 7u;
}

static void pack32(const uint8_t c[32], uint32_t w[3]) {
  w[0] = w[1] = w[2] = 0;
  for (int i = 0; i < 10; ++i) w[0] |= (uint32_t)(c[i] & 7u) << (3 * i);
  w[0] |= (uint32_t)(c[10] & 3u) << 30;
  w[1] |= (uint32_t)((c[10] >> 2) & 1u);
  for (int i = 0; i < 10; ++i) w[1] |= (uint32_t)(c[11 + i] & 7u) << (1 + 3 * i);
  w[1] |= (uint32_t)(c[21] & 1u) << 31;
  w[2] |= (uint32_t)((c[21] >> 1) & 3u);
  for (int i = 0; i < 10; ++i) w[2] |= (uint32_t)(c[22 + i] & 7u) << (2 + 3 * i);
}

/* qweight int32 [3K/32, O]  ->  codes uint8 [K, O]  (gptq_deployment.py:75-78). */
int fbo_gptq_w3_unpack_rows(const int32_t* words, int64_t packed_rows, int64_t cols,
                            uint8_t* codes) {
  if (packed_rows % 3) return -1;
  for (int64_t blk = 0; blk < packed_rows / 3; ++blk)
    for (int64_t o = 0; o < cols; ++o) {
      uint32_t w[3];
      uint8_t c[32];
      for (int j = 0; j < 3; ++j) w[j] = (uint32_t)words[(blk * 3 + j) * cols + o];
      unpack32(w, c);
      for (int i = 0; i < 32; ++i) codes[(blk * 32 + i) * cols + o] = c[i];
    }
  return 0;
}

/* codes uint8 [K, O] -> qweight int32 [3K/32, O]  (gptq_deployment.py:331-348). */
int fbo_gptq_w3_pack_rows(const uint8_t* codes, int64_t k, int64_t cols, int32_t* words) {
  if (k % 32) return -1;
  for (int64_t i = 0; i < k * cols; ++i)
    if (codes[i] > 7) return -2;
  for (int64_t blk = 0; blk < k / 32; ++blk)
    for (int64_t o = 0; o < cols; ++o) {
      uint32_t w[3];
      uint8_t c[32];
      for (int i = 0; i < 32; ++i) c[i] = codes[(blk * 32 + i) * cols + o];
      pack32(c, w);
      for (int j = 0; j < 3; ++j) words[(blk * 3 + j) * cols + o] = (int32_t)w[j];
    }
  return 0;
}

/* qzeros int32 [G, 3O/32] -> zeros uint8 [G, O]; format 1 stores zero-1
 * (gptq_deployment.py:81-93). */
int fbo_gptq_w3_unpack_cols(const int32_t* words, int64_t rows, int64_t packed_cols,
                            int qzero_format, uint8_t* zeros) {
  if (packed_cols % 3 || (qzero_format != 1 && qzero_format != 2)) return -1;
  int64_t o = packed_cols / 3 * 32;
  for (int64_t g = 0; g < rows; ++g)
    for (int64_t blk = 0; blk < packed_cols / 3; ++blk) {
      uint32_t w[3];
      uint8_t c[32];
      for (int j = 0; j < 3; ++j) w[j] = (uint32_t)words[g * packed_cols + blk * 3 + j];
      unpack32(w, c);
      for (int i = 0; i < 32; ++i)
        zeros[g * o + blk * 32 + i] = qzero_format == 1 ? (uint8_t)((c[i] + 1) & 7) : c[i];
    }
  return 0;
}

int fbo_gptq_w3_pack_cols(const uint8_t* values, int64_t rows, int64_t cols, int32_t* words) {
  if (cols % 32) return -1;
  int64_t pc = cols / 32 * 3;
  for (int64_t g = 0; g < rows; ++g)
    for (int64_t blk = 0; blk < cols / 32; ++blk) {
      uint32_t w[3];
      pack32(values + g * cols + blk * 32, w);
      for (int j = 0; j < 3; ++j) words[g * pc + blk * 3 + j] = (int32_t)w[j];
    }
  return 0;
}

/* ------------------------------------------------------ W3 planar bit planes */

/* codes [K,O] (original column order) + perm (sorted position -> original column,
 * NULL = identity)  ->  planes uint8 [G,3,O,16].  Byte c of a 16-byte row holds
 * sorted positions g*128 + 8c .. 8c+7, least significant bit first; plane 2 is stored
 * inverted so that q-4 = b0 + 2*b1 - 4*stored_b2.
 * Follows gptq_deployment.py:96-101 (_pack_bytes) and :207-218. */
int fbo_w3_planes_from_codes(const uint8_t* codes, const int16_t* perm, int64_t k, int64_t o,
                             uint8_t* planes) {
  if (k % FBO_GROUP) return -1;
  int64_t groups = k / FBO_GROUP;
  memset(planes, 0, (size_t)(groups * 3 * o * 16));
  for (int64_t sk = 0; sk < k; ++sk) {
    int64_t src = perm ? perm[sk] : sk;
    int64_t g = sk / FBO_GROUP, within = sk % FBO_GROUP;
    int64_t byte = within / 8;
    int bit = (int)(within % 8);
    for (int64_t r = 0; r < o; ++r) {
      uint8_t q = codes[src * o + r];
      uint8_t b[3] = {(uint8_t)(q & 1), (uint8_t)((q >> 1) & 1), (uint8_t)(1 - ((q >> 2) & 1))};
      for (int p = 0; p < 3; ++p)
        planes[((g * 3 + p) * o + r) * 16 + byte] |= (uint8_t)(b[p] << bit);
    }
  }
  return 0;
}

/* planes -> codes [K,O]; original_order != 0 scatters rows back through perm.
 * Follows gptq_deployment.py:104-108 (_unpack_bytes) and :230-244. */
int fbo_w3_codes_from_planes(const uint8_t* planes, const int16_t* perm, int64_t k, int64_t o,
                             int original_order, uint8_t* codes) {
  if (k % FBO_GROUP) return -1;
  for (int64_t sk = 0; sk < k; ++sk) {
    int64_t dst = (original_order && perm) ? perm[sk] : sk;
    int64_t g = sk / FBO_GROUP, within = sk % FBO_GROUP;
    int64_t byte = within / 8;
    int bit = (int)(within % 8);
    for (int64_t r = 0; r < o; ++r) {
      const uint8_t* row = planes + (g * 3 * o + r) * 16 + byte;
      int b0 = (row[0] >> bit) & 1;
      int b1 = (row[o * 16] >> bit) & 1;
      int b2 = 1 - ((row[2 * o * 16] >> bit) & 1);
      codes[dst * o + r] = (uint8_t)(b0 | (b1 << 1) | (b2 << 2));
    }
  }
  return 0;
}

static inline int w3_zero(const uint8_t* zeros, int64_t g, int64_t o, int64_t r) {
  return zeros ? zeros[g * o + r] : 4;
}

/* Dequantise to W [O,K] in the ORIGINAL column order.  The product scale*(q-zero) is
 * formed in the scale's own 16-bit dtype (one rounding), then cast to out_dtype,
 * which is how gptq_deployment.py:247-260 (restore_planar_w3) computes it for bf16
 * scales and zero 4, and how the reference's test expression
 * tests/test_gptq_w3_planar.py:83-90 states the general zero-point form.
 * out: uint16_t bits when out_dtype is FBO_F16/FBO_BF16, float when FBO_F32. */
int fbo_w3_dequant(const uint8_t* planes, const uint16_t* scales, int scale_dtype,
                   const uint8_t* zeros, const int16_t* perm, int64_t k, int64_t o,
                   int out_dtype, void* out) {
  if (k % FBO_GROUP) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r) {
    for (int64_t sk = 0; sk < k; ++sk) {
      int64_t g = sk / FBO_GROUP, within = sk % FBO_GROUP;
      int64_t byte = within / 8;
      int bit = (int)(within % 8);
      const uint8_t* row = planes + (g * 3 * o + r) * 16 + byte;
      int q = ((row[0] >> bit) & 1) | (((row[o * 16] >> bit) & 1) << 1) |
              ((1 - ((row[2 * o * 16] >> bit) & 1)) << 2);
      float s = half_to_f32(scales[g * o + r], scale_dtype);
      float w = round_to(s * (float)(q - w3_zero(zeros, g, o, r)), scale_dtype);
      int64_t col = perm ? perm[sk] : sk;
      if (out_dtype == FBO_F32)
        ((float*)out)[r * k + col] = w;
      else
        ((uint16_t*)out)[r * k + col] = f32_to_half(w, out_dtype);
    }
  }
  return 0;
}

/* y[m,r] = sum_k float(W[r,k]) * float(x[m,k]), fp32 accumulation, W given as fp32.
 * The matmul half of "dequantise then matmul" (tests/test_gptq_w3_planar.py:114-117). */
void fbo_dense_gemv_f32(const float* w, const float* x, int64_t m, int64_t o, int64_t k,
                        float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r)
    for (int64_t i = 0; i < m; ++i) {
      float acc[8] = {0};
      const float* wr = w + r * k;
      const float* xr = x + i * k;
      int64_t j = 0;
      for (; j + 8 <= k; j += 8)
        for (int l = 0; l < 8; ++l) acc[l] += wr[j + l] * xr[j + l];
      float tail = 0.f;
      for (; j < k; ++j) tail += wr[j] * xr[j];
      y[i * o + r] = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7])) + tail;
    }
}

/* Same product with W stored as bf16/f16 bits (what a CPU holding the dequantised
 * 16-bit weight would run; the cast to fp32 happens per element inside the loop). */
void fbo_dense_gemv_half(const uint16_t* w, int w_dtype, const float* x, int64_t m, int64_t o,
                         int64_t k, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r)
    for (int64_t i = 0; i < m; ++i) {
      float acc[8] = {0};
      const uint16_t* wr = w + r * k;
      const float* xr = x + i * k;
      int64_t j = 0;
      for (; j + 8 <= k; j += 8)
        for (int l = 0; l < 8; ++l) acc[l] += half_to_f32(wr[j + l], w_dtype) * xr[j + l];
      float tail = 0.f;
      for (; j < k; ++j) tail += half_to_f32(wr[j], w_dtype) * xr[j];
      y[i * o + r] = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7])) + tail;
    }
}

/* Dequantise-then-matmul in one call: the oracle of record for the W3 GEMV.
 * x: 16-bit activations [M,K]; y: fp32 [M,O]. */
int fbo_w3_gemv_dequant(const uint16_t* x, int act_dtype, int64_t m, const uint8_t* planes,
                        const uint16_t* scales, int scale_dtype, const uint8_t* zeros,
                        const int16_t* perm, int64_t k, int64_t o, float* y) {
  float* w = (float*)malloc(sizeof(float) * (size_t)(o * k));
  float* xf = (float*)malloc(sizeof(float) * (size_t)(m * k));
  if (!w || !xf) { free(w); free(xf); return -3; }
  int rc = fbo_w3_dequant(planes, scales, scale_dtype, zeros, perm, k, o, FBO_F32, w);
  if (rc == 0) {
    fbo_convert_to_f32(x, act_dtype, m * k, xf);
    fbo_dense_gemv_f32(w, xf, m, o, k, y);
  }
  free(w);
  free(xf);
  return rc;
}

/* Structural form: y[r] = sum_g scale[g,r] * sum_{k in g} (q-zero) * x[perm[k]], the
 * inner sum in fp32 over ascending sorted k, then one multiply by the unrounded scale.
 * Follows gptq_deployment.py:263-277 (structural_w3_matvec), with the general
 * zero-point of tests/test_gptq_w3_planar.py:92-103. */
int fbo_w3_gemv_structural(const uint16_t* x, int act_dtype, int64_t m, const uint8_t* planes,
                           const uint16_t* scales, int scale_dtype, const uint8_t* zeros,
                           const int16_t* perm, int64_t k, int64_t o, float* y) {
  if (k % FBO_GROUP) return -1;
  int64_t groups = k / FBO_GROUP;
  float* xs = (float*)malloc(sizeof(float) * (size_t)(m * k));
  if (!xs) return -3;
  for (int64_t i = 0; i < m; ++i)
    for (int64_t sk = 0; sk < k; ++sk)
      xs[i * k + sk] = half_to_f32(x[i * k + (perm ? perm[sk] : sk)], act_dtype);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r)
    for (int64_t i = 0; i < m; ++i) {
      float total = 0.f;
      for (int64_t g = 0; g < groups; ++g) {
        int z = w3_zero(zeros, g, o, r);
        const uint8_t* row = planes + (g * 3 * o + r) * 16;
        float dot = 0.f;
        for (int within = 0; within < FBO_GROUP; ++within) {
          int byte = within / 8, bit = within % 8;
          int q = ((row[byte] >> bit) & 1) | (((row[o * 16 + byte] >> bit) & 1) << 1) |
                  ((1 - ((row[2 * o * 16 + byte] >> bit) & 1)) << 2);
          dot += (float)(q - z) * xs[i * k + g * FBO_GROUP + within];
        }
        total += dot * half_to_f32(scales[g * o + r], scale_dtype);
      }
      y[i * o + r] = total;
    }
  free(xs);
  return 0;
}

/* Emulation of the reference CUDA kernel's arithmetic for zero point 4: 256-entry
 * subset-sum tables built in ascending bit order (csrc/lut8_unsigned.cuh:12-27), three
 * plane accumulators over chunks 0..15, dot = a0 + 2*a1 - 4*a2 (csrc/w3_lut.cu:87-114),
 * one fp32 partial per group summed over ascending groups (csrc/w3_lut.cu:142-150). */
int fbo_w3_gemv_lut_emulation(const uint16_t* x, int act_dtype, const uint8_t* planes,
                              const uint16_t* scales, int scale_dtype, const int16_t* perm,
                              int64_t k, int64_t o, float* y) {
  if (k % FBO_GROUP) return -1;
  int64_t groups = k / FBO_GROUP;
  float* lut = (float*)malloc(sizeof(float) * (size_t)(groups * 16 * 256));
  if (!lut) return -3;
  for (int64_t g = 0; g < groups; ++g)
    for (int c = 0; c < 16; ++c) {
      float v[8];
      for (int j = 0; j < 8; ++j) {
        int64_t sk = g * FBO_GROUP + c * 8 + j;
        v[j] = half_to_f32(x[perm ? perm[sk] : sk], act_dtype);
      }
      float* t = lut + (g * 16 + c) * 256;
      for (int p = 0; p < 256; ++p) {
        float s = 0.f;
        for (int b = 0; b < 8; ++b)
          if ((p >> b) & 1) s += v[b];
        t[p] = s;
      }
    }
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r) {
    float total = 0.f;
    for (int64_t g = 0; g < groups; ++g) {
      const uint8_t* row = planes + (g * 3 * o + r) * 16;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f;
      for (int c = 0; c < 16; ++c) {
        const float* t = lut + (g * 16 + c) * 256;
        a0 += t[row[c]];
        a1 += t[row[o * 16 + c]];
        a2 += t[row[2 * o * 16 + c]];
      }
      float dot = a0 + 2.f * a1 - 4.f * a2;
      total += dot * half_to_f32(scales[g * o + r], scale_dtype);
    }
    y[r] = total;
  }
  free(lut);
  return 0;
}

/* ------------------------------------------------- two-base binary bases */

/* bases int8 [2,O,K] in {-1,+1} -> codes uint8 [O,K/4]; bit 2j = base 0 at position
 * 4i+j, bit 2j+1 = base 1; +1 -> 1, -1 -> 0.  Follows packing.py:14-33. */
int fbo_pack_two_bases(const int8_t* bases, int64_t o, int64_t k, uint8_t* codes) {
  if (k % 4) return -1;
  for (int64_t i = 0; i < 2 * o * k; ++i)
    if (bases[i] != 1 && bases[i] != -1) return -2;
  for (int64_t r = 0; r < o; ++r)
    for (int64_t c = 0; c < k / 4; ++c) {
      uint8_t v = 0;
      for (int j = 0; j < 4; ++j) {
        v |= (uint8_t)((bases[r * k + 4 * c + j] > 0) << (2 * j));
        v |= (uint8_t)((bases[(o + r) * k + 4 * c + j] > 0) << (2 * j + 1));
      }
      codes[r * (k / 4) + c] = v;
    }
  return 0;
}

/* Follows packing.py:36-49. */
void fbo_unpack_two_bases(const uint8_t* codes, int64_t o, int64_t quarter_k, int8_t* bases) {
  int64_t k = quarter_k * 4;
  for (int64_t r = 0; r < o; ++r)
    for (int64_t c = 0; c < quarter_k; ++c)
      for (int j = 0; j < 4; ++j) {
        uint8_t v = codes[r * quarter_k + c];
        bases[r * k + 4 * c + j] = (int8_t)(((v >> (2 * j)) & 1) * 2 - 1);
        bases[(o + r) * k + 4 * c + j] = (int8_t)(((v >> (2 * j + 1)) & 1) * 2 - 1);
      }
}

/* Interleaved pairs of bytes -> two 8-bit planes: [..., 2n] -> [..., 2, n].  Bit j of
 * plane b, byte i is bit 2j+b of the 16-bit word (byte 2i | byte 2i+1 << 8).
 * Follows deployment.py:54-63 (_compact_even, _to_planes). */
void fbo_bb_to_planes(const uint8_t* inter, int64_t rows, int64_t n_pairs, uint8_t* planes) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < n_pairs; ++i) {
      unsigned word = inter[r * 2 * n_pairs + 2 * i] | ((unsigned)inter[r * 2 * n_pairs + 2 * i + 1] << 8);
      uint8_t p0 = 0, p1 = 0;
      for (int j = 0; j < 8; ++j) {
        p0 |= (uint8_t)(((word >> (2 * j)) & 1) << j);
        p1 |= (uint8_t)(((word >> (2 * j + 1)) & 1) << j);
      }
      planes[r * 2 * n_pairs + i] = p0;
      planes[r * 2 * n_pairs + n_pairs + i] = p1;
    }
}

/* Follows deployment.py:66-73 (_from_planes). */
void fbo_bb_from_planes(const uint8_t* planes, int64_t rows, int64_t n_pairs, uint8_t* inter) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < n_pairs; ++i) {
      unsigned p0 = planes[r * 2 * n_pairs + i], p1 = planes[r * 2 * n_pairs + n_pairs + i];
      unsigned word = 0;
      for (int j = 0; j < 8; ++j) word |= (((p0 >> j) & 1) << (2 * j)) | (((p1 >> j) & 1) << (2 * j + 1));
      inter[r * 2 * n_pairs + 2 * i] = (uint8_t)(word & 0xff);
      inter[r * 2 * n_pairs + 2 * i + 1] = (uint8_t)(word >> 8);
    }
}

static inline int sign_of(const uint8_t* codes, int64_t quarter_k, int64_t r, int64_t col, int base) {
  return ((codes[r * quarter_k + col / 4] >> (2 * (col % 4) + base)) & 1) * 2 - 1;
}

/* Dense fp32 weight [O,K] of the seven-field hybrid payload: global two-base term with
 * per-group row scales [2,O,G] and column scales [2,G,128], plus a two-base refinement
 * scatter-added on 8 selected columns per group.  Accumulation order matches
 * evaluation.py:59-95 (base 0 then base 1, each product row*col rounded in fp32) and
 * :98-175 (refinement summed separately, then added). */
int fbo_bb_materialize_hybrid(const uint8_t* codes, const float* rows, const float* cols,
                              const int64_t* indices, const uint8_t* rcodes, const float* rrows,
                              const float* rcols, int64_t o, int64_t g, float* w) {
  int64_t k = g * FBO_GROUP;
  for (int64_t r = 0; r < o; ++r)
    for (int64_t grp = 0; grp < g; ++grp) {
      for (int j = 0; j < FBO_GROUP; ++j) {
        int64_t col = grp * FBO_GROUP + j;
        float acc = 0.f;
        for (int b = 0; b < 2; ++b) {
          float term = (float)sign_of(codes, k / 4, r, col, b);
          term *= rows[(b * o + r) * g + grp];
          term *= cols[(b * g + grp) * FBO_GROUP + j];
          acc += term;
        }
        w[r * k + col] = acc;
      }
      for (int j = 0; j < 8; ++j) {
        int64_t idx = indices[grp * 8 + j];
        if (idx < 0 || idx >= FBO_GROUP) return -2;
        float acc = 0.f;
        for (int b = 0; b < 2; ++b) {
          float term = (float)sign_of(rcodes, g * 2, r, grp * 8 + j, b);
          term *= rrows[(b * o + r) * g + grp];
          term *= rcols[(b * g + grp) * 8 + j];
          acc += term;
        }
        w[r * k + grp * FBO_GROUP + idx] += acc;
      }
    }
  return 0;
}

/* FP64 structural reference on the KERNEL layout (codes [G,O,32] interleaved or
 * [G,O,2,16] planar; rows [G,O,2]; columns [G,128,2]; indices [G,8]; sparse codes
 * [G,O,2] or [G,O,2,1]; sparse rows [G,O,2]; sparse columns [G,8,2]).
 * Follows factored_reference.py:9-42. */
int fbo_bb_structural_f64(const uint16_t* x, int act_dtype, const uint8_t* codes, int planar,
                          const float* rows, const float* cols, const int16_t* indices,
                          const uint8_t* sparse, const float* srows, const float* scols,
                          int64_t o, int64_t g, double* y) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r) {
    double total = 0.0;
    for (int64_t grp = 0; grp < g; ++grp) {
      double w[FBO_GROUP];
      const uint8_t* c = codes + (grp * o + r) * 32;
      for (int j = 0; j < FBO_GROUP; ++j) {
        int s0, s1;
        if (planar) {
          s0 = ((c[j / 8] >> (j % 8)) & 1) * 2 - 1;
          s1 = ((c[16 + j / 8] >> (j % 8)) & 1) * 2 - 1;
        } else {
          unsigned q = c[j / 4] >> (2 * (j % 4));
          s0 = (int)(q & 1) * 2 - 1;
          s1 = (int)((q >> 1) & 1) * 2 - 1;
        }
        w[j] = (double)s0 * rows[(grp * o + r) * 2] * cols[(grp * FBO_GROUP + j) * 2] +
               (double)s1 * rows[(grp * o + r) * 2 + 1] * cols[(grp * FBO_GROUP + j) * 2 + 1];
      }
      const uint8_t* sc = sparse + (grp * o + r) * 2;
      for (int j = 0; j < 8; ++j) {
        int s0, s1;
        if (planar) {
          s0 = ((sc[0] >> j) & 1) * 2 - 1;
          s1 = ((sc[1] >> j) & 1) * 2 - 1;
        } else {
          unsigned q = sc[j / 4] >> (2 * (j % 4));
          s0 = (int)(q & 1) * 2 - 1;
          s1 = (int)((q >> 1) & 1) * 2 - 1;
        }
        w[indices[grp * 8 + j]] +=
            (double)s0 * srows[(grp * o + r) * 2] * scols[(grp * 8 + j) * 2] +
            (double)s1 * srows[(grp * o + r) * 2 + 1] * scols[(grp * 8 + j) * 2 + 1];
      }
      double dot = 0.0;
      for (int j = 0; j < FBO_GROUP; ++j)
        dot += w[j] * (double)half_to_f32(x[grp * FBO_GROUP + j], act_dtype);
      total += dot;
    }
    y[r] = total;
  }
  return 0;
}

/* Global two-base format with matrix-wide scales (no groups): dense
 * W[r,k] = r0[r]*B0[r,k]*c0[k] + r1[r]*B1[r,k]*c1[k], plus dense salient columns
 * W[r, idx[j]] += S[r,j].  sign planes uint8 [2,O,K/8] (bit j of byte i = column
 * 8i+j, 1 = +1); r/c scales fp16 bits; salient bf16 bits [O,n_sal].  The two-base
 * part follows evaluation.py:59-95 with one group spanning all of K.
 * y fp64 [O] = W x in double (the reference's high-precision style,
 * factored_reference.py:9-15). */
int fbo_bb_global_gemv_f64(const uint16_t* x, int act_dtype, const uint8_t* planes,
                           const uint16_t* rscale, const uint16_t* cscale,
                           const int32_t* sal_idx, const uint16_t* sal, int64_t n_sal,
                           int64_t o, int64_t k, double* y) {
  if (k % 8) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r) {
    double total = 0.0;
    for (int b = 0; b < 2; ++b) {
      double acc = 0.0;
      const uint8_t* row = planes + ((int64_t)b * o + r) * (k / 8);
      for (int64_t col = 0; col < k; ++col) {
        int s = ((row[col / 8] >> (col % 8)) & 1) * 2 - 1;
        acc += (double)s * (double)f16_bits_to_f32(cscale[b * k + col]) *
               (double)half_to_f32(x[col], act_dtype);
      }
      total += acc * (double)f16_bits_to_f32(rscale[b * o + r]);
    }
    for (int64_t j = 0; j < n_sal; ++j)
      total += (double)bf16_bits_to_f32(sal[r * n_sal + j]) *
               (double)half_to_f32(x[sal_idx[j]], act_dtype);
    y[r] = total;
  }
  return 0;
}

/* Same format, dense fp32 weight [O,K] (dequantise step of dequantise-then-matmul). */
int fbo_bb_global_materialize(const uint8_t* planes, const uint16_t* rscale,
                              const uint16_t* cscale, const int32_t* sal_idx,
                              const uint16_t* sal, int64_t n_sal, int64_t o, int64_t k, float* w) {
  if (k % 8) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < o; ++r) {
    for (int64_t col = 0; col < k; ++col) {
      float acc = 0.f;
      for (int b = 0; b < 2; ++b) {
        float term = (float)(((planes[((int64_t)b * o + r) * (k / 8) + col / 8] >> (col % 8)) & 1) * 2 - 1);
        term *= f16_bits_to_f32(rscale[b * o + r]);
        term *= f16_bits_to_f32(cscale[b * k + col]);
        acc += term;
      }
      w[r * k + col] = acc;
    }
    for (int64_t j = 0; j < n_sal; ++j) w[r * k + sal_idx[j]] += bf16_bits_to_f32(sal[r * n_sal + j]);
  }
  return 0;
}

/* ------------------------------------------------------- RMSNorm and RoPE */

/* out = weight * dtype( x_f32 * rsqrt(mean(x_f32^2) + eps) ); the cast to the input
 * dtype happens BEFORE the multiply by the weight, and that product is rounded to the
 * dtype again.  Follows fused_modules.py:30-41 (rms_norm_reference). */
void fbo_rmsnorm(const uint16_t* x, const uint16_t* weight, int dtype, int64_t rows, int64_t dim,
                 float eps, uint16_t* out) {
  for (int64_t r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int64_t i = 0; i < dim; ++i) {
      float v = half_to_f32(x[r * dim + i], dtype);
      ss += (double)v * (double)v;
    }
    float var = (float)(ss / (double)dim);
    float inv = 1.0f / sqrtf(var + eps);
    for (int64_t i = 0; i < dim; ++i) {
      float normed = round_to(half_to_f32(x[r * dim + i], dtype) * inv, dtype);
      out[r * dim + i] = f32_to_half(half_to_f32(weight[i], dtype) * normed, dtype);
    }
  }
}

/* Rotary embedding on `heads` vectors of `dim` values sharing one cos/sin row:
 * out = dtype( dtype(v*cos) + rotate_half(v)*sin ), rotate_half(v) = (-v[dim/2:], v[:dim/2]).
 * Follows fused_modules.py:66-85 (q and k concatenated along the head axis, so the
 * same function serves both). */
void fbo_rope(const uint16_t* v, const uint16_t* cosv, const uint16_t* sinv, int dtype,
              int64_t heads, int64_t dim, uint16_t* out) {
  int64_t half = dim / 2;
  for (int64_t h = 0; h < heads; ++h)
    for (int64_t i = 0; i < dim; ++i) {
      float a = half_to_f32(v[h * dim + i], dtype);
      float rot = i < half ? -half_to_f32(v[h * dim + i + half], dtype)
                           : half_to_f32(v[h * dim + i - half], dtype);
      float first = round_to(a * half_to_f32(cosv[i], dtype), dtype);
      float second = rot * half_to_f32(sinv[i], dtype);
      out[h * dim + i] = f32_to_half(first + second, dtype);
    }
}
