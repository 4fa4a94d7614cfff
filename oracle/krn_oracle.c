/* krn_oracle.c — TEST INFRASTRUCTURE, not product code.
 *
 * A CPU restatement, in plain C, of the arithmetic the reference's C backend generates for the tile
 * matrix product and the flash-attention tile pattern. Only tests, the smoke check and the CPU-baseline leg
 * of the benchmark may load this file's library; the product path never does.
 *
 * Parity status:
 *   - tile product (f32 / f16 / bf16 operands): PINNED against the reference's own known-answer tests
 *     (all-ones products 33 / 16 / 256, the forward-error bound 8*2^-24*(k+8)*|A||B| on the seeds and
 *     ragged shapes of tests/compiler/test_tensor_cores.py:314-401,404-508, transposed-rhs product of
 *     tests/frontend/test_tile_ops.py:90-98) — see tests/test_oracle_pins.py.
 *   - flash attention statements: PINNED against the reference's float64 check (atol 2e-3 / 3e-3 on
 *     ragged sequences, examples/04_libraries/08_flash_attention.py:62-86,
 *     tests/frontend/test_tile_ops.py:130-154).
 *   - e4m3fn decode: PINNED against the independent 256-entry table of
 *     tests/compiler/test_tensor_cores.py:200-216.
 *   - e5m2 decode and mixed e4m3 / e5m2 pair products: PINNED against the same tests (seed-81 code draw, all four
 *     pairings, tests/compiler/test_tensor_cores.py:146,219-239).
 *   - block-scaled FP8 product, MXFP8 product, grouped-query / batched attention, paged FP8 decode: PARITY UNPINNED —
 *     the reference has neither an implementation nor a test; the definitions here are ours (the MXFP8 FORMAT is the
 *     reference's, src/krn/data/formats.py:138-144, and its value tables are pinned).
 *
 * Build: see oracle/Makefile (gcc -O2 -march=native -ffp-contract=off -fwrapv -fPIC -shared, the
 * reference's clang flags, src/krn/runtime/cpu.py:48-51, src/krn/runtime/compile_options.py:279-295).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KRN_F32 0
#define KRN_F16 1
#define KRN_BF16 2
#define KRN_E4M3 3
#define KRN_E5M2 4
/* An operand-type argument may name two types: the low byte is A's, bits 8..15 hold B's type + 1 (0 = same as A).
 * The reference multiplies mixed e4m3 / e5m2 pairs (tests/compiler/test_tensor_cores.py:146,219-239). */
#define KRN_A_TYPE(t) ((t) & 0xff)
#define KRN_B_TYPE(t) ((((t) >> 8) & 0xff) ? (((t) >> 8) & 0xff) - 1 : ((t) & 0xff))

/* ---- storage conversions ------------------------------------------------------------------------- */

/* bf16 word -> f32: exact (the C backend's `(float)` cast of a __bf16, src/krn/runtime/cpu.py:96). */
static inline float bf16_to_f32(uint16_t w) {
  uint32_t bits = (uint32_t)w << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* f32 -> bf16 word, round to nearest even, NaN quieted: the emulator's `_bfloat16`
 * (src/krn/emulator/emulate.py:144-150) and what a C cast to __bf16 does. */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  if ((bits & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((bits >> 16) | 0x0040u);
  bits += 0x7FFFu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

static inline float f16_to_f32(uint16_t w) {
  _Float16 h;
  memcpy(&h, &w, 2);
  return (float)h;
}

static inline uint16_t f32_to_f16(float f) {
  _Float16 h = (_Float16)f;
  uint16_t w;
  memcpy(&w, &h, 2);
  return w;
}

/* e4m3fn code -> value: bias 7, no infinities, 0x7F / 0xFF are NaN, subnormals m * 2^-9
 * (src/krn/data/formats.py:59-76,95). */
float krn_oracle_e4m3_decode(uint8_t code) {
  int sign = code >> 7, exponent = (code >> 3) & 15, mantissa = code & 7;
  float value;
  if ((code & 0x7F) == 0x7F) return NAN;
  if (exponent == 0) {
    value = ldexpf((float)mantissa, -9);
  } else {
    value = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
  }
  return sign ? -value : value;
}

/* value -> e4m3fn code: nearest representable, ties to the even code, magnitudes beyond 448 saturate to
 * 448, NaN -> 0x7F (src/krn/compiler/narrow.py:79-105). */
uint8_t krn_oracle_e4m3_encode(float x) {
  if (x != x) return 0x7F;
  uint8_t sign = signbit(x) ? 0x80 : 0;
  float a = fabsf(x);
  if (a >= 448.0f) return sign | 0x7E;
  if (a < 0.015625f) {
    /* below the smallest normal (2^-6): multiples of 2^-9, ties to even (nearbyintf in the default mode);
     * a result of 8 is the code of 2^-6 itself */
    return sign | (uint8_t)nearbyintf(a * 512.0f);
  }
  uint32_t bits;
  memcpy(&bits, &a, 4);
  bits += 0x7FFFFu + ((bits >> 20) & 1u); /* round the 23-bit mantissa to 3 bits, ties to even */
  uint32_t exponent = (bits >> 23) - 127 + 7, mantissa = (bits >> 20) & 7u;
  uint32_t code = (exponent << 3) | mantissa;
  if (code > 0x7E) code = 0x7E; /* rounded past 448 */
  return sign | (uint8_t)code;
}

void krn_oracle_e4m3_encode_array(const float* x, uint8_t* codes, int64_t count) {
  for (int64_t i = 0; i < count; ++i) codes[i] = krn_oracle_e4m3_encode(x[i]);
}

void krn_oracle_e4m3_decode_array(const uint8_t* codes, float* x, int64_t count) {
  for (int64_t i = 0; i < count; ++i) x[i] = krn_oracle_e4m3_decode(codes[i]);
}

void krn_oracle_bf16_round_array(const float* x, uint16_t* words, int64_t count) {
  for (int64_t i = 0; i < count; ++i) words[i] = f32_to_bf16(x[i]);
}

/* e5m2 code -> value: IEEE-style, bias 15, all-ones exponent is inf / NaN (src/krn/data/formats.py:91) — the
 * upper byte of the binary16 word with the same value. */
static inline float e5m2_to_f32(uint8_t code) { return f16_to_f32((uint16_t)((uint16_t)code << 8)); }

static inline float load_as_f32(const void* base, int type, int64_t index) {
  switch (type) {
    case KRN_F32: return ((const float*)base)[index];
    case KRN_F16: return f16_to_f32(((const uint16_t*)base)[index]);
    case KRN_BF16: return bf16_to_f32(((const uint16_t*)base)[index]);
    case KRN_E5M2: return e5m2_to_f32(((const uint8_t*)base)[index]);
    default: return krn_oracle_e4m3_decode(((const uint8_t*)base)[index]);
  }
}

static inline void store_from_f32(void* base, int type, int64_t index, float value) {
  switch (type) {
    case KRN_F32: ((float*)base)[index] = value; break;
    case KRN_F16: ((uint16_t*)base)[index] = f32_to_f16(value); break;
    case KRN_BF16: ((uint16_t*)base)[index] = f32_to_bf16(value); break;
    default: ((uint8_t*)base)[index] = krn_oracle_e4m3_encode(value); break;
  }
}

/* ---- fused epilogue of the library matmul ---------------------------------------------------------------- */

/* The tail of the reference's `matmul_epilogue` kernel (src/krn/lib/lib_kernels.py:40-48) applied to the f32
 * accumulator `acc` (m x n, what the K loop leaves): `acc += bias[cols].to(f32)` when bit 0 of `flags` is set (the bias
 * has the output type, src/krn/lib/lib.py:155-163), then relu / gelu / silu (bits 1-2 = 1 / 2 / 3) with the element
 * functions the C renderer writes for f32 (src/krn/compiler/emit.py:110-114: `x < 0 ? 0 : x`,
 * `0.5f * x * (1 + erff(x * 0.7071067811865476f))`, `x / (1 + expf(-x))`), then `out = acc.to(out type)`. */
void krn_oracle_matmul_epilogue(int c_type, const float* acc, const void* bias, void* out, int64_t m, int64_t n,
                                int flags) {
  const int activation = flags >> 1;
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float x = acc[i * n + j];
      if (flags & 1) x = x + load_as_f32(bias, c_type, j);
      if (activation == 1) x = x < 0 ? 0 : x;
      if (activation == 2) x = 0.5f * x * (1 + erff(x * 0.7071067811865476f));
      if (activation == 3) x = x / (1 + expf(-x));
      store_from_f32(out, c_type, i * n + j, x);
    }
  }
}

/* ---- tile matrix product, faithful loop structure --------------------------------------------------- */

/* The kernel
 *     rows, cols = block.tile(bm, bn); acc = zeros(f32, bm, bn)
 *     for ks in pipelined(K, bk): acc += a[rows, ks] @ b[cols, ks].transpose()   (b_kn == 0)
 *                                 acc += a[rows, ks] @ b[ks, cols]               (b_kn != 0)
 *     c[rows, cols] = acc.to(T)
 * as the reference's C renderer writes it: the whole grid runs in one call, block after block
 * (src/krn/runtime/cpu.py:127-140); each product first stages both operands into f32 buffers with invalid
 * lanes as zero (src/krn/compiler/emit.py:957-974), then for every (i, j)
 *     s = acc[i][j]; for kk in 0..bk: s = fmaf(A[i][kk], B[kk][j], s); acc[i][j] = s
 * (src/krn/compiler/emit.py:791-796); stores are guarded per element (src/krn/compiler/emit.py:763-774).
 * `row_begin/row_end` select a range of block rows so a caller can split the grid over threads (the
 * reference gets concurrency only across streams, src/krn/runtime/runtime.py:949-951); pass 0 and the
 * number of block rows for the whole grid. */
void krn_oracle_gemm_blocks(int ab_type, int c_type, int b_kn, const void* a, const void* b, void* c, int64_t m,
                            int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int bm, int bn, int bk,
                            int64_t row_begin, int64_t row_end) {
  const int a_type = KRN_A_TYPE(ab_type), b_type = KRN_B_TYPE(ab_type);
  float* acc = aligned_alloc(64, ((size_t)bm * bn * 4 + 63) / 64 * 64);
  float* ta = aligned_alloc(64, ((size_t)bm * bk * 4 + 63) / 64 * 64);
  float* tb = aligned_alloc(64, ((size_t)bk * bn * 4 + 63) / 64 * 64);
  int64_t blocks_x = (n + bn - 1) / bn;
  if (blocks_x < 1) blocks_x = 1;
  for (int64_t by = row_begin; by < row_end; ++by) {
    for (int64_t bx = 0; bx < blocks_x; ++bx) {
      int64_t row0 = by * bm, col0 = bx * bn;
      for (int64_t e = 0; e < (int64_t)bm * bn; ++e) acc[e] = (float)0;
      for (int64_t k0 = 0; k0 < k; k0 += bk) {
        for (int i = 0; i < bm; ++i)
          for (int kk = 0; kk < bk; ++kk) {
            int64_t r = row0 + i, kc = k0 + kk;
            ta[i * bk + kk] = (r < m && kc < k) ? load_as_f32(a, a_type, r * lda + kc) : 0.0f;
          }
        for (int kk = 0; kk < bk; ++kk)
          for (int j = 0; j < bn; ++j) {
            int64_t cidx = col0 + j, kc = k0 + kk;
            float v = 0.0f;
            if (cidx < n && kc < k) v = b_kn ? load_as_f32(b, b_type, kc * ldb + cidx) : load_as_f32(b, b_type, cidx * ldb + kc);
            tb[kk * bn + j] = v;
          }
        for (int i = 0; i < bm; ++i)
          for (int j = 0; j < bn; ++j) {
            float s = acc[i * bn + j];
            for (long long kk = 0; kk < bk; ++kk) s = __builtin_fmaf(ta[i * bk + kk], tb[kk * bn + j], s);
            acc[i * bn + j] = s;
          }
      }
      for (int i = 0; i < bm; ++i)
        for (int j = 0; j < bn; ++j) {
          int64_t r = row0 + i, cidx = col0 + j;
          if ((unsigned long long)r < (unsigned long long)m && (unsigned long long)cidx < (unsigned long long)n)
            store_from_f32(c, c_type, r * ldc + cidx, acc[i * bn + j]);
        }
    }
  }
  free(acc);
  free(ta);
  free(tb);
}

/* The same numbers, computed faster: every output element is still the k-ordered single-rounded fma chain
 * starting from +0.0f (the chain does not depend on the tiling because the accumulator is re-read between
 * k tiles), but the j loop is innermost so the compiler can run 16 independent chains per vector. Used by
 * tests that need the oracle at sizes where the faithful loop takes minutes. Rows [row_begin, row_end). */
void krn_oracle_gemm_fast(int ab_type, int c_type, int b_kn, const void* a, const void* b, void* c, int64_t m,
                          int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t row_begin,
                          int64_t row_end) {
  (void)m;
  const int a_type = KRN_A_TYPE(ab_type), b_type = KRN_B_TYPE(ab_type);
  /* B as f32 [k][n] */
  float* bt = aligned_alloc(64, ((size_t)(k > 0 ? k : 1) * n * 4 + 63) / 64 * 64);
  float* row = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j)
      bt[kk * n + j] = b_kn ? load_as_f32(b, b_type, kk * ldb + j) : load_as_f32(b, b_type, j * ldb + kk);
  for (int64_t i = row_begin; i < row_end; ++i) {
    for (int64_t j = 0; j < n; ++j) row[j] = 0.0f;
    for (int64_t kk = 0; kk < k; ++kk) {
      float av = load_as_f32(a, a_type, i * lda + kk);
      const float* brow = bt + kk * n;
      for (int64_t j = 0; j < n; ++j) row[j] = __builtin_fmaf(av, brow[j], row[j]);
    }
    for (int64_t j = 0; j < n; ++j) store_from_f32(c, c_type, i * ldc + j, row[j]);
  }
  free(bt);
  free(row);
}

/* ---- block-scaled FP8 product (our definition; parity unpinned) ---------------------------------------- */

/* C[i,j] = sum over 128-wide K blocks kb of (sa[i,kb] * sb[j/128,kb]) * P_kb[i,j], where P_kb is the fma
 * chain of the decoded e4m3 codes over the block's k range starting from +0.0f, and the outer sum adds the
 * scaled partials in kb order in f32 (multiply and add rounded separately). Codes are exactly representable
 * in f32, so P_kb carries only accumulation rounding. */
void krn_oracle_gemm_fp8_blockscaled(int c_type, const uint8_t* a, const float* sa, const uint8_t* b,
                                     const float* sb, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
                                     int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb, int64_t row_begin,
                                     int64_t row_end) {
  (void)m;
  float table[256];
  for (int i = 0; i < 256; ++i) table[i] = krn_oracle_e4m3_decode((uint8_t)i);
  float* bt = aligned_alloc(64, ((size_t)(k > 0 ? k : 1) * n * 4 + 63) / 64 * 64);
  float* part = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  float* total = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j) bt[kk * n + j] = table[b[j * ldb + kk]];
  for (int64_t i = row_begin; i < row_end; ++i) {
    for (int64_t j = 0; j < n; ++j) total[j] = 0.0f;
    for (int64_t k0 = 0, kb = 0; k0 < k; k0 += 128, ++kb) {
      int64_t k1 = k0 + 128 < k ? k0 + 128 : k;
      for (int64_t j = 0; j < n; ++j) part[j] = 0.0f;
      for (int64_t kk = k0; kk < k1; ++kk) {
        float av = table[a[i * lda + kk]];
        const float* brow = bt + kk * n;
        for (int64_t j = 0; j < n; ++j) part[j] = __builtin_fmaf(av, brow[j], part[j]);
      }
      float sai = sa[i * ldsa + kb];
      for (int64_t j = 0; j < n; ++j) {
        float scale = sai * sb[(j / 128) * ldsb + kb];
        float scaled = scale * part[j];
        total[j] = total[j] + scaled;
      }
    }
    for (int64_t j = 0; j < n; ++j) store_from_f32(c, c_type, i * ldc + j, total[j]);
  }
  free(bt);
  free(part);
  free(total);
}

/* ---- MXFP8 product (the reference's MXFP8 format; its product is declared, not implemented: parity unpinned) ---- */

/* e8m0 scale byte -> value: 2^(code - 127), 0xFF is NaN (src/krn/data/formats.py:98: 8 exponent bits, no mantissa, no
 * sign, bias 127, exponent field 0 is 2^-127 and not zero). */
float krn_oracle_e8m0_decode(uint8_t code) { return code == 0xFF ? NAN : ldexpf(1.0f, (int)code - 127); }

/* C[i,j] = sum over 32-wide K blocks kb of (2^(sa[i,kb]-127) * 2^(sb[j,kb]-127)) * P_kb[i,j], P_kb the fma chain of the
 * decoded e4m3 codes over the block starting from +0.0f; the scaled partials are added in kb order in f32. The product
 * of two powers of two and its multiplication into P_kb are exact (barring overflow), so only the two accumulations
 * round. Rows [row_begin, row_end). */
void krn_oracle_gemm_mxfp8(int c_type, const uint8_t* a, const uint8_t* sa, const uint8_t* b, const uint8_t* sb, void* c,
                           int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa,
                           int64_t ldsb, int64_t row_begin, int64_t row_end) {
  (void)m;
  float table[256];
  for (int i = 0; i < 256; ++i) table[i] = krn_oracle_e4m3_decode((uint8_t)i);
  float* bt = aligned_alloc(64, ((size_t)(k > 0 ? k : 1) * n * 4 + 63) / 64 * 64);
  float* part = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  float* total = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j) bt[kk * n + j] = table[b[j * ldb + kk]];
  for (int64_t i = row_begin; i < row_end; ++i) {
    for (int64_t j = 0; j < n; ++j) total[j] = 0.0f;
    for (int64_t k0 = 0, kb = 0; k0 < k; k0 += 32, ++kb) {
      int64_t k1 = k0 + 32 < k ? k0 + 32 : k;
      for (int64_t j = 0; j < n; ++j) part[j] = 0.0f;
      for (int64_t kk = k0; kk < k1; ++kk) {
        float av = table[a[i * lda + kk]];
        const float* brow = bt + kk * n;
        for (int64_t j = 0; j < n; ++j) part[j] = __builtin_fmaf(av, brow[j], part[j]);
      }
      float sai = krn_oracle_e8m0_decode(sa[i * ldsa + kb]);
      for (int64_t j = 0; j < n; ++j) {
        float scale = sai * krn_oracle_e8m0_decode(sb[j * ldsb + kb]);
        float scaled = scale * part[j];
        total[j] = total[j] + scaled;
      }
    }
    for (int64_t j = 0; j < n; ++j) store_from_f32(c, c_type, i * ldc + j, total[j]);
  }
  free(bt);
  free(part);
  free(total);
}

/* ---- NVFP4 product (the reference's NVFP4 format; its product is declared, not implemented: parity unpinned) ---- */

/* e2m1 code (4 bits: sign, two exponent bits, one mantissa bit; bias 1, subnormal 0.5, every code a number:
 * src/krn/data/formats.py:100,59-76) -> value: 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives. */
float krn_oracle_e2m1_decode(uint8_t code) {
  static const float magnitude[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float v = magnitude[code & 7];
  return (code & 8) ? -v : v;
}

/* C[i,j] = alpha * sum over 16-wide K blocks kb of (sa[i,kb] * sb[j,kb]) * P_kb[i,j]: a, b hold two e2m1 codes per byte,
 * the lower k in the low nibble; sa, sb are e4m3 codes; P_kb is the sum of the block's 16 products (exact in f32, as is
 * the product of the two scales and its multiplication into P_kb); the scaled partials are added in kb order in f32 and
 * the total is multiplied by alpha. Rows [row_begin, row_end). lda / ldb in bytes. */
void krn_oracle_gemm_nvfp4(int c_type, const uint8_t* a, const uint8_t* sa, const uint8_t* b, const uint8_t* sb, float alpha,
                           void* c, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa,
                           int64_t ldsb, int64_t row_begin, int64_t row_end) {
  (void)m;
  float* bt = aligned_alloc(64, ((size_t)(k > 0 ? k : 1) * n * 4 + 63) / 64 * 64);
  float* part = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  float* total = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j) bt[kk * n + j] = krn_oracle_e2m1_decode((uint8_t)((b[j * ldb + kk / 2] >> (4 * (kk & 1))) & 15));
  for (int64_t i = row_begin; i < row_end; ++i) {
    for (int64_t j = 0; j < n; ++j) total[j] = 0.0f;
    for (int64_t k0 = 0, kb = 0; k0 < k; k0 += 16, ++kb) {
      int64_t k1 = k0 + 16 < k ? k0 + 16 : k;
      for (int64_t j = 0; j < n; ++j) part[j] = 0.0f;
      for (int64_t kk = k0; kk < k1; ++kk) {
        float av = krn_oracle_e2m1_decode((uint8_t)((a[i * lda + kk / 2] >> (4 * (kk & 1))) & 15));
        const float* brow = bt + kk * n;
        for (int64_t j = 0; j < n; ++j) part[j] = __builtin_fmaf(av, brow[j], part[j]);
      }
      float sai = krn_oracle_e4m3_decode(sa[i * ldsa + kb]);
      for (int64_t j = 0; j < n; ++j) {
        float scale = sai * krn_oracle_e4m3_decode(sb[j * ldsb + kb]);
        float scaled = scale * part[j];
        total[j] = total[j] + scaled;
      }
    }
    for (int64_t j = 0; j < n; ++j) store_from_f32(c, c_type, i * ldc + j, alpha * total[j]);
  }
  free(bt);
  free(part);
  free(total);
}

/* MXFP4 product (src/krn/data/formats.py:129-135): C[i,j] = sum over 32-wide K blocks kb of (2^(sa[i,kb]-127) *
 * 2^(sb[j,kb]-127)) * P_kb[i,j], a and b as in krn_oracle_gemm_nvfp4 (two e2m1 codes per byte, lower k in the low
 * nibble), the scaled partials added in kb order in f32. Rows [row_begin, row_end). lda / ldb in bytes. */
void krn_oracle_gemm_mxfp4(int c_type, const uint8_t* a, const uint8_t* sa, const uint8_t* b, const uint8_t* sb, void* c,
                           int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa,
                           int64_t ldsb, int64_t row_begin, int64_t row_end) {
  (void)m;
  float* bt = aligned_alloc(64, ((size_t)(k > 0 ? k : 1) * n * 4 + 63) / 64 * 64);
  float* part = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  float* total = aligned_alloc(64, ((size_t)n * 4 + 63) / 64 * 64);
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j) bt[kk * n + j] = krn_oracle_e2m1_decode((uint8_t)((b[j * ldb + kk / 2] >> (4 * (kk & 1))) & 15));
  for (int64_t i = row_begin; i < row_end; ++i) {
    for (int64_t j = 0; j < n; ++j) total[j] = 0.0f;
    for (int64_t k0 = 0, kb = 0; k0 < k; k0 += 32, ++kb) {
      int64_t k1 = k0 + 32 < k ? k0 + 32 : k;
      for (int64_t j = 0; j < n; ++j) part[j] = 0.0f;
      for (int64_t kk = k0; kk < k1; ++kk) {
        float av = krn_oracle_e2m1_decode((uint8_t)((a[i * lda + kk / 2] >> (4 * (kk & 1))) & 15));
        const float* brow = bt + kk * n;
        for (int64_t j = 0; j < n; ++j) part[j] = __builtin_fmaf(av, brow[j], part[j]);
      }
      float sai = krn_oracle_e8m0_decode(sa[i * ldsa + kb]);
      for (int64_t j = 0; j < n; ++j) {
        float scale = sai * krn_oracle_e8m0_decode(sb[j * ldsb + kb]);
        float scaled = scale * part[j];
        total[j] = total[j] + scaled;
      }
    }
    for (int64_t j = 0; j < n; ++j) store_from_f32(c, c_type, i * ldc + j, total[j]);
  }
  free(bt);
  free(part);
  free(total);
}

/* ---- flash attention, statement by statement --------------------------------------------------------- */

static inline float krn_max(float a, float b) { return (a > b || a != a) ? a : b; } /* emit.py:116-120 */

/* One call runs heads [head_begin, head_end) of the flattened (batch * q_heads) axis. Statements and their
 * order follow examples/04_libraries/08_flash_attention.py:44-59 as the C renderer executes them:
 *   m = 0 - 1e30, total = 0, acc = 0
 *   per key tile: s = (q @ k^T) * scale      (fma chains over d from +0, then one multiply)
 *                 causal: s = kpos <= qpos ? s : -1e30
 *                 m_new = maximum(m, rowmax over valid lanes, first valid lane initialises)
 *                 p = exp2(s - m_new); corr = exp2(m - m_new)
 *                 total *= corr; total += rowsum(p) (left to right over valid lanes)
 *                 acc *= corr; acc += p.to(T) @ v   (p rounded to the storage type, fma chain over keys)
 *                 m = m_new
 *   o = (acc / total).to(T)
 * Key lanes past seq_kv are invalid: they enter neither max, sum nor product; query rows past seq_q are
 * not stored (src/krn/compiler/emit.py:997-1034,763-774). Grouped-query attention (kv head = q head /
 * (q_heads / kv_heads)) and the batch axis are extensions the reference does not have.
 * Layouts: q, o [batch, q_heads, seq_q, d]; k, v [batch, kv_heads, seq_kv, d], contiguous. */
void krn_oracle_flash_attention(int type, const void* q, const void* k, const void* v, void* o, int64_t batch,
                                int64_t q_heads, int64_t kv_heads, int64_t seq_q, int64_t seq_kv, int d,
                                float scale, int causal, int bq, int bk, int64_t head_begin, int64_t head_end) {
  (void)batch;
  float* qt = malloc(sizeof(float) * bq * d);
  float* kt = malloc(sizeof(float) * bk * d);
  float* vt = malloc(sizeof(float) * bk * d);
  float* s = malloc(sizeof(float) * bq * bk);
  float* p = malloc(sizeof(float) * bq * bk);
  float* acc = malloc(sizeof(float) * bq * d);
  float* mrow = malloc(sizeof(float) * bq);
  float* total = malloc(sizeof(float) * bq);
  int64_t group = q_heads / kv_heads;
  for (int64_t bh = head_begin; bh < head_end; ++bh) {
    int64_t bidx = bh / q_heads, h = bh % q_heads, hk = h / group;
    int64_t q_base = (bidx * q_heads + h) * seq_q * d;
    int64_t kv_base = (bidx * kv_heads + hk) * seq_kv * d;
    for (int64_t q0 = 0; q0 < seq_q; q0 += bq) {
      for (int i = 0; i < bq; ++i) {
        mrow[i] = 0.0f - 1.0e30f;
        total[i] = 0.0f;
        for (int x = 0; x < d; ++x) {
          acc[i * d + x] = 0.0f;
          qt[i * d + x] = (q0 + i < seq_q) ? load_as_f32(q, type, q_base + (q0 + i) * d + x) : 0.0f;
        }
      }
      for (int64_t c = 0; c < seq_kv; c += bk) {
        int64_t valid = seq_kv - c < bk ? seq_kv - c : bk;
        for (int j = 0; j < bk; ++j)
          for (int x = 0; x < d; ++x) {
            int ok = j < valid;
            kt[j * d + x] = ok ? load_as_f32(k, type, kv_base + (c + j) * d + x) : 0.0f;
            vt[j * d + x] = ok ? load_as_f32(v, type, kv_base + (c + j) * d + x) : 0.0f;
          }
        for (int i = 0; i < bq; ++i) {
          for (int j = 0; j < bk; ++j) {
            float dot = 0.0f;
            for (int x = 0; x < d; ++x) dot = __builtin_fmaf(qt[i * d + x], kt[j * d + x], dot);
            float val = dot * scale;
            if (causal) val = ((c + j) <= (q0 + i)) ? val : -1.0e30f;
            s[i * bk + j] = val;
          }
          float rmax = 0.0f;
          for (int64_t j = 0; j < valid; ++j) {
            float x = s[i * bk + j];
            if (j > 0) rmax = (rmax > x || rmax != rmax) ? rmax : x; else rmax = x;
          }
          float m_new = krn_max(mrow[i], rmax);
          float corr = __builtin_exp2f(mrow[i] - m_new);
          float rsum = 0.0f;
          for (int64_t j = 0; j < valid; ++j) {
            float e = __builtin_exp2f(s[i * bk + j] - m_new);
            p[i * bk + j] = e;
            if (j > 0) rsum = rsum + e; else rsum = e;
          }
          total[i] = total[i] * corr;
          total[i] = total[i] + rsum;
          for (int x = 0; x < d; ++x) {
            float a0 = acc[i * d + x] * corr;
            for (int64_t j = 0; j < valid; ++j) {
              float pj = p[i * bk + j];
              /* p.to(T): one rounding to the storage type before the product */
              float pr = type == KRN_BF16 ? bf16_to_f32(f32_to_bf16(pj)) : type == KRN_F16 ? f16_to_f32(f32_to_f16(pj)) : pj;
              a0 = __builtin_fmaf(pr, vt[j * d + x], a0);
            }
            acc[i * d + x] = a0;
          }
          mrow[i] = m_new;
        }
      }
      for (int i = 0; i < bq; ++i) {
        if (q0 + i >= seq_q) continue;
        for (int x = 0; x < d; ++x) store_from_f32(o, type, q_base + (q0 + i) * d + x, acc[i * d + x] / total[i]);
      }
    }
  }
  free(qt); free(kt); free(vt); free(s); free(p); free(acc); free(mrow); free(total);
}

/* ---- paged FP8 decode attention (our definition; parity unpinned) ------------------------------------- */

/* One query token per sequence. Scores s_j = (q . K_j) * k_scale * scale_log2 with K_j the decoded e4m3
 * codes of token j, softmax in double precision, O = (sum_j p_j V_j) * v_scale, rounded once to bf16.
 * q, o bf16 [batch, q_heads, d]; pages e4m3 [num_pages, page_size, kv_heads, d]; page_table int32
 * [batch, max_pages]; scales f32 [batch, kv_heads]. Sequences [seq_begin, seq_end). */
void krn_oracle_decode_fp8_paged(const uint16_t* q, const uint8_t* k_pages, const uint8_t* v_pages,
                                 const int32_t* page_table, const int32_t* context_len, const float* k_scale,
                                 const float* v_scale, uint16_t* o, int64_t q_heads, int64_t kv_heads, int d,
                                 int page_size, int64_t max_pages, float scale_log2, int64_t seq_begin,
                                 int64_t seq_end) {
  float table[256];
  for (int i = 0; i < 256; ++i) table[i] = krn_oracle_e4m3_decode((uint8_t)i);
  int64_t group = q_heads / kv_heads;
  for (int64_t b = seq_begin; b < seq_end; ++b) {
    int64_t len = context_len[b];
    double* score = malloc(sizeof(double) * (len > 0 ? len : 1));
    for (int64_t h = 0; h < q_heads; ++h) {
      int64_t hk = h / group;
      double ks = (double)k_scale[b * kv_heads + hk] * (double)scale_log2;
      double vs = (double)v_scale[b * kv_heads + hk];
      const uint16_t* qv = q + (b * q_heads + h) * d;
      double best = -INFINITY;
      for (int64_t j = 0; j < len; ++j) {
        int64_t page = page_table[b * max_pages + j / page_size];
        const uint8_t* row = k_pages + ((page * page_size + j % page_size) * kv_heads + hk) * d;
        double dot = 0.0;
        for (int x = 0; x < d; ++x) dot += (double)bf16_to_f32(qv[x]) * (double)table[row[x]];
        score[j] = dot * ks;
        if (score[j] > best) best = score[j];
      }
      double denom = 0.0;
      double out[512];
      for (int x = 0; x < d; ++x) out[x] = 0.0;
      for (int64_t j = 0; j < len; ++j) {
        double pj = exp2(score[j] - best);
        denom += pj;
        int64_t page = page_table[b * max_pages + j / page_size];
        const uint8_t* row = v_pages + ((page * page_size + j % page_size) * kv_heads + hk) * d;
        for (int x = 0; x < d; ++x) out[x] += pj * (double)table[row[x]];
      }
      for (int x = 0; x < d; ++x) o[(b * q_heads + h) * d + x] = f32_to_bf16((float)(out[x] / denom * vs));
    }
    free(score);
  }
}
