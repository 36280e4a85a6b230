/*
 * afir_oracle.c -- CPU restatement of the fused-group semantics of the
 * Ascend-MLIR device-codegen path.  TEST INFRASTRUCTURE ONLY: this file is
 * the checker the CUDA kernels are compared against and the timed host-CPU
 * baseline.  Nothing in the shipped library links, loads or calls it.
 *
 * Each function is the scalar loop nest a stock Linalg->loops->LLVM lowering
 * of the reference's linalg-on-tensors input would execute:
 *   - one rounding to the IR element type after every arith op
 *     (f16/bf16 ops are computed in f32 and rounded back, which is exact
 *     RN behaviour for add/mul because f32 carries >= 2p+2 significand bits);
 *   - no FMA contraction (build with -ffp-contract=off, no fast-math);
 *   - reductions accumulate sequentially in ascending index order;
 *   - arith.maximumf propagates NaN and orders -0 < +0.
 * OpenMP only parallelises the independent leading axis.
 *
 * Parity pin: checked in tests/test_oracle_golden.py against the numpy
 * goldens produced by the reference's own examples/<group>/gen_data.py scripts
 * (committed under tests/golden/ with the script that made them), using
 * the tolerances each reference run.sh states.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define AFO_EXPORT __attribute__((visibility("default")))
#if defined(__x86_64__)
#define AFO_CLONES __attribute__((target_clones("avx2", "default")))
#else
#define AFO_CLONES
#endif

/* ------------------------------------------------------------------ */
/* 16-bit float conversions (round-to-nearest-even, IEEE semantics).   */
/* ------------------------------------------------------------------ */
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    /* subnormal: value = man * 2^-24 */
    float v = (float)man * 5.9604644775390625e-08f;
    return sign ? -v : v;
  }
  if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
  return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

static inline uint16_t f32_to_f16(float f) {
  uint32_t u = f32_bits(f);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);        /* NaN */
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);       /* >= 65520 rounds to inf */
  if (a < 0x33000001u) return sign;                              /* <= 2^-25 rounds to 0 */
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  uint32_t shift;
  uint32_t base;
  if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); base = 0; }  /* subnormal half */
  else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q += 1;
  return (uint16_t)(sign | (base + q));                          /* carry into exponent is correct */
}

/* arith.maximumf: NaN-propagating, -0 < +0. */
static inline float maximumf_ir(float a, float b) {
  if (a != a) return a;
  if (b != b) return b;
  if (a == 0.0f && b == 0.0f) return (f32_bits(a) & 0x80000000u) ? b : a;
  return a > b ? a : b;
}

/* per-op helpers on storage types */
static inline uint16_t h_add(uint16_t a, uint16_t b) { return f32_to_f16(f16_to_f32(a) + f16_to_f32(b)); }
static inline uint16_t h_mul(uint16_t a, uint16_t b) { return f32_to_f16(f16_to_f32(a) * f16_to_f32(b)); }
static inline uint16_t h_max(uint16_t a, uint16_t b) { return f32_to_f16(maximumf_ir(f16_to_f32(a), f16_to_f32(b))); }
static inline uint16_t b_add(uint16_t a, uint16_t b) { return f32_to_bf16(bf16_to_f32(a) + bf16_to_f32(b)); }
static inline uint16_t b_mul(uint16_t a, uint16_t b) { return f32_to_bf16(bf16_to_f32(a) * bf16_to_f32(b)); }

AFO_EXPORT void afo_f32_to_f16(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_f16(src[i]);
}
AFO_EXPORT void afo_f16_to_f32(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f16_to_f32(src[i]);
}
AFO_EXPORT void afo_f32_to_bf16(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}
AFO_EXPORT void afo_bf16_to_f32(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}
AFO_EXPORT void afo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
AFO_EXPORT int afo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------ */
/* Elementwise chains                                                  */
/* ------------------------------------------------------------------ */

/* out = (a + b) * b on f32: afir.add then afir.mul
 * (include/Dialect/AFIR/Ops/Basic/math.td:93,95; sibling lowering
 * lib/Conversion/AFIRToASCIR/Math/Elementwise.cpp:26-57).  Two roundings. */
AFO_EXPORT AFO_CLONES void afo_add_mul_f32(const float *a, const float *b, float *out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float s = a[i] + b[i];
    out[i] = s * b[i];
  }
}

/* x[B,R,2C] f16 split on the last axis into h0 = x[..., :C], h1 = x[..., C:];
 * out[B,R,C] = (max(h0, 0) + bias) * h1, every op rounded to f16.  Body order
 * follows examples/split-relu-brc-add-mul/step0_input.mlir:59-70 (maximumf,
 * addf, mulf); the split is a tensor.extract_slice (ibid. :47-50).  bias_axis
 * 1 indexes bias by the row r (the reference's row map (d0,d1)->(d0)),
 * bias_axis 2 by the column c (numpy trailing-aligned broadcast). */
AFO_EXPORT void afo_split_relu_bias_mul_f16(const uint16_t *x, const uint16_t *bias, uint16_t *out,
                                            int64_t B, int64_t R, int64_t C, int bias_axis) {
#pragma omp parallel for schedule(static)
  for (int64_t br = 0; br < B * R; ++br) {
    const uint16_t *h0 = x + br * 2 * C;
    const uint16_t *h1 = h0 + C;
    uint16_t *o = out + br * C;
    int64_t r = br % R;
    for (int64_t c = 0; c < C; ++c) {
      uint16_t bv = bias[bias_axis == 1 ? r : c];
      uint16_t t = h_max(h0[c], 0);
      t = h_add(t, bv);
      o[c] = h_mul(t, h1[c]);
    }
  }
}

/* The reference's own example shape: a[M,N] split into top/bottom row halves,
 * out_h[m,n] = (max(a_h[m,n],0) + bias_h[m]) * scale_h[n], halves concatenated
 * on axis 0 (examples/split-relu-brc-add-mul/step0_input.mlir:47-90). */
AFO_EXPORT void afo_split_rows_relu_bias_scale_f16(const uint16_t *a, const uint16_t *bias0,
                                                   const uint16_t *bias1, const uint16_t *scale0,
                                                   const uint16_t *scale1, uint16_t *out, int64_t M,
                                                   int64_t N) {
  int64_t HM = M / 2;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < 2 * HM; ++m) {
    const uint16_t *bias = m < HM ? bias0 : bias1;
    const uint16_t *scale = m < HM ? scale0 : scale1;
    int64_t mm = m < HM ? m : m - HM;
    for (int64_t n = 0; n < N; ++n) {
      uint16_t t = h_max(a[m * N + n], 0);
      t = h_add(t, bias[mm]);
      out[m * N + n] = h_mul(t, scale[n]);
    }
  }
}

/* out[2M,N] = concat(a[m] + b[m,n], c[m] * d[m,n]) on axis 0
 * (examples/add-broadcast-concat/step0_input.mlir, two generics + tensor.concat). */
AFO_EXPORT void afo_add_mul_concat_f16(const uint16_t *a, const uint16_t *b, const uint16_t *c,
                                       const uint16_t *d, uint16_t *out, int64_t M, int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      out[m * N + n] = h_add(a[m], b[m * N + n]);
      out[(M + m) * N + n] = h_mul(c[m], d[m * N + n]);
    }
}

/* out[n,m] = max(d0[m,0], 0) + d1[n,m]
 * (examples/relu-broadcast-transpose/step0_input.mlir: relu generic then the
 * generic whose first map is (d0,d1)->(d1,0)). */
AFO_EXPORT void afo_relu_bcast_transpose_add_f16(const uint16_t *d0, const uint16_t *d1, uint16_t *out,
                                                 int64_t M, int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t m = 0; m < M; ++m) out[n * M + m] = h_add(h_max(d0[m], 0), d1[n * M + m]);
}

/* Plain 2-D transpose out[n,m] = in[m,n] for 2- and 4-byte elements
 * (permutation generics, lib/Conversion/LinalgToAscendC/ComputeConversion.cpp:1275-1290). */
AFO_EXPORT void afo_transpose_2d(const void *in, void *out, int64_t M, int64_t N, int elem_bytes) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t m = 0; m < M; ++m)
      memcpy((char *)out + (n * M + m) * elem_bytes, (const char *)in + (m * N + n) * elem_bytes,
             (size_t)elem_bytes);
}

/* ------------------------------------------------------------------ */
/* Broadcast + add + row reduction                                     */
/* ------------------------------------------------------------------ */

/* out[m] = sum_n (a[m] + b[m,n]), f32, zero-initialised accumulator,
 * ascending n (examples/broadcast-add-reduce/step0_input.mlir:47-92).
 * sum64 (optional) receives the same sum accumulated in f64 and
 * abs64 (optional) receives sum_n |a[m] + b[m,n]| for error bounds. */
AFO_EXPORT void afo_bcast_add_rowsum_f32(const float *a, const float *b, float *out, double *sum64,
                                         double *abs64, int64_t M, int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float acc = 0.0f;
    double acc64 = 0.0, accabs = 0.0;
    float am = a[m];
    const float *row = b + m * N;
    for (int64_t n = 0; n < N; ++n) {
      float d = am + row[n];
      acc = acc + d;
      acc64 += (double)d;
      accabs += fabs((double)d);
    }
    out[m] = acc;
    if (sum64) sum64[m] = acc64;
    if (abs64) abs64[m] = accabs;
  }
}

/* Timed variant without the f64 side sums (host-CPU baseline of the same loop). */
AFO_EXPORT AFO_CLONES void afo_bcast_add_rowsum_f32_fast(const float *a, const float *b, float *out,
                                                         int64_t M, int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float acc = 0.0f;
    float am = a[m];
    const float *row = b + m * N;
    for (int64_t n = 0; n < N; ++n) acc = acc + (am + row[n]);
    out[m] = acc;
  }
}

/* f16 form of the reference example: the add rounds to f16 (the IR op type),
 * the reduction runs on f32 casts and the sum is cast back to f16
 * (lib/Target/CannKernel/CannTranslation.cpp:2446-2461). */
AFO_EXPORT void afo_bcast_add_rowsum_f16(const uint16_t *a, const uint16_t *b, uint16_t *out, int64_t M,
                                         int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float acc = 0.0f;
    for (int64_t n = 0; n < N; ++n) acc = acc + f16_to_f32(h_add(a[m], b[m * N + n]));
    out[m] = f32_to_f16(acc);
  }
}

/* ------------------------------------------------------------------ */
/* Gather + elementwise                                                */
/* ------------------------------------------------------------------ */

/* Row gather (the embedding form MarkStructuredOps detects as embedding_dim,
 * lib/Conversion/MarkStructuredOps/MarkStructuredOpsPass.cpp:54-139):
 * out[i,j] = table[idx[i], j] * scale[j] + resid[i,j], bf16, each op rounded.
 * Returns the number of out-of-range indices (those rows are left untouched). */
AFO_EXPORT int64_t afo_gather_rows_scale_resid_bf16(const uint16_t *table, const int32_t *idx,
                                                    const uint16_t *scale, const uint16_t *resid,
                                                    uint16_t *out, int64_t rows, int64_t width,
                                                    int64_t table_rows) {
  int64_t bad = 0;
#pragma omp parallel for schedule(static) reduction(+ : bad)
  for (int64_t i = 0; i < rows; ++i) {
    int64_t r = idx[i];
    if (r < 0 || r >= table_rows) { bad += 1; continue; }
    const uint16_t *src = table + r * width;
    for (int64_t j = 0; j < width; ++j)
      out[i * width + j] = b_add(b_mul(src[j], scale[j]), resid[i * width + j]);
  }
  return bad;
}

/* Column gather with relu pre-op and bias post-op, the form the reference lowers:
 * out[i,j] = max(data[i, idx[j]], 0) + bias[j]
 * (examples/gather-elementwise-fusion/step0_input.mlir:24-76; fusion order
 * pre -> extract -> post, lib/Conversion/FuseGatherElementwise/FuseGatherElementwisePass.cpp:190-274). */
AFO_EXPORT int64_t afo_relu_gather_cols_bias_f16(const uint16_t *data, const int64_t *idx,
                                                 const uint16_t *bias, uint16_t *out, int64_t M,
                                                 int64_t N, int64_t K) {
  int64_t bad = 0;
  for (int64_t j = 0; j < K; ++j)
    if (idx[j] < 0 || idx[j] >= N) bad += 1;
  if (bad) return bad;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < K; ++j)
      out[i * K + j] = h_add(h_max(data[i * N + idx[j]], 0), bias[j]);
  return 0;
}

/* ------------------------------------------------------------------ */
/* Matmul + bias + LeakyReLU                                           */
/* ------------------------------------------------------------------ */

/* acc[n] += a * brow[n]; separate multiply and add roundings, ascending k. */
AFO_CLONES static void axpy_row(float *acc, float a, const float *brow, int64_t N) {
  for (int64_t n = 0; n < N; ++n) {
    float p = a * brow[n];
    acc[n] = acc[n] + p;
  }
}

/* E = max(x, alpha * x), x = A.B + bias[n]; the epilogue is the
 * maximumf(x, mulf(x, alpha)) form the reference matches
 * (lib/Conversion/MarkStructuredOps/AnnotateMixMatmulSemanticsPass.cpp:171-242,
 * examples/matmul-add-leakyrelu/step0_input.mlir:23-52).  A,B,bias,out are
 * bf16 (in_kind 0) or A,B f16 with bias/out f32 (in_kind 1, the reference's
 * example types).  f32 accumulation from zero in ascending k.  Rows
 * [row_begin,row_end) of the output are produced; out points at row 0. */
static void matmul_bias_leakyrelu_impl(const uint16_t *A, const uint16_t *B, const void *bias, void *out,
                                       int64_t M, int64_t N, int64_t K, float alpha, int64_t row_begin,
                                       int64_t row_end, int in_kind) {
  (void)M;
  float *Bf = (float *)malloc((size_t)K * (size_t)N * sizeof(float));
  if (!Bf) return;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < K * N; ++i) Bf[i] = in_kind == 0 ? bf16_to_f32(B[i]) : f16_to_f32(B[i]);
#pragma omp parallel
  {
    float *acc = (float *)malloc((size_t)N * sizeof(float));
#pragma omp for schedule(dynamic, 4)
    for (int64_t m = row_begin; m < row_end; ++m) {
      for (int64_t n = 0; n < N; ++n) acc[n] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        float a = in_kind == 0 ? bf16_to_f32(A[m * K + k]) : f16_to_f32(A[m * K + k]);
        axpy_row(acc, a, Bf + k * N, N);
      }
      for (int64_t n = 0; n < N; ++n) {
        float bv = in_kind == 0 ? bf16_to_f32(((const uint16_t *)bias)[n]) : ((const float *)bias)[n];
        float x = acc[n] + bv;
        float y = maximumf_ir(x, x * alpha);
        if (in_kind == 0) ((uint16_t *)out)[m * N + n] = f32_to_bf16(y);
        else ((float *)out)[m * N + n] = y;
      }
    }
    free(acc);
  }
  free(Bf);
}

AFO_EXPORT void afo_matmul_bias_leakyrelu_bf16(const uint16_t *A, const uint16_t *B, const uint16_t *bias,
                                               uint16_t *out, int64_t M, int64_t N, int64_t K, float alpha,
                                               int64_t row_begin, int64_t row_end) {
  matmul_bias_leakyrelu_impl(A, B, bias, out, M, N, K, alpha, row_begin, row_end, 0);
}

AFO_EXPORT void afo_matmul_bias_leakyrelu_f16_f32(const uint16_t *A, const uint16_t *B, const float *bias,
                                                  float *out, int64_t M, int64_t N, int64_t K, float alpha,
                                                  int64_t row_begin, int64_t row_end) {
  matmul_bias_leakyrelu_impl(A, B, bias, out, M, N, K, alpha, row_begin, row_end, 1);
}

/* One output element with f64 accumulation, for sampled checks of large GEMMs. */
AFO_EXPORT double afo_matmul_bias_leakyrelu_bf16_at(const uint16_t *A, const uint16_t *B,
                                                    const uint16_t *bias, int64_t N, int64_t K, float alpha,
                                                    int64_t m, int64_t n) {
  double acc = 0.0;
  for (int64_t k = 0; k < K; ++k) acc += (double)bf16_to_f32(A[m * K + k]) * (double)bf16_to_f32(B[k * N + n]);
  double x = acc + (double)bf16_to_f32(bias[n]);
  double y = x * (double)alpha;
  return x > y ? x : y;
}

/* ------------------------------------------------------------------ */
/* Output comparator                                                   */
/* ------------------------------------------------------------------ */

/* The reference's validation rule: an element fails when
 * |actual - expected| > atol + rtol * |expected|
 * (lib/Runtime/Execution/OutputComparator.cpp:75-140).  Returns the number of
 * failing elements; max/mean absolute difference are reported. */
AFO_EXPORT int64_t afo_compare_f32(const float *actual, const float *expected, int64_t n, double atol,
                                   double rtol, double *max_abs, double *mean_abs) {
  int64_t fails = 0;
  double mx = 0.0, sum = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    double a = actual[i], e = expected[i];
    double d = fabs(a - e);
    if (!(d <= atol + rtol * fabs(e))) fails += 1;
    if (d > mx) mx = d;
    sum += d;
  }
  if (max_abs) *max_abs = mx;
  if (mean_abs) *mean_abs = n ? sum / (double)n : 0.0;
  return fails;
}
