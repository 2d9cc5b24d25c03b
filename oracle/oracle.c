/*
 * oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C CPU restatement of the arithmetic the reference holds its device path to
 * (its CPU comparison backend burn-flex, pinned `=0.21.0` in Cargo.toml:46, is not in
 * the reference tree, so parity against burn-flex's own bits is UNPINNED; what is
 * pinned are the closed-form known-answer cases of the reference's tests, see
 * tests/test_oracle_kats.py).  Only tests, the smoke check and the benchmark's CPU
 * baseline leg may load this file's library; the engine never does.
 *
 * IEEE-754 binary32, round to nearest even, denormals kept.  Built with
 * -O2 -fno-fast-math -ffp-contract=off so no product-sum is fused.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* BF16 narrowing: crates/tt-tests/tests/step270_native_bf16.rs:244-255 (ties to even, NaN
 * quieted keeping sign and high payload, BF16 subnormals to signed zero). */
uint16_t orc_bf16_round(uint32_t x) {
  uint32_t r;
  if ((x & 0x7fffffffu) > 0x7f800000u) r = x | 0x00400000u;
  else r = x + 0x7fffu + ((x >> 16) & 1u);
  r &= 0xffff0000u;
  if ((r & 0x7fffffffu) < 0x00800000u) r &= 0x80000000u;
  return (uint16_t)(r >> 16);
}
void orc_bf16_round_n(const uint32_t* in, uint16_t* out, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) out[i] = orc_bf16_round(in[i]);
}

/* C = op(A) op(B) in F32: each output element is a sum over k ascending, one rounding a
 * multiply and one an add (what a plain CPU loop gives; crates/tt-tests/tests/step11_burn.rs:
 * 15-32 names burn-flex's product as the comparison).  Row-major stored matrices; *_t says
 * the stored matrix is the transpose of the logical operand.  OpenMP over row blocks. */
void orc_gemm_f32(const float* a, int a_t, const float* b, int b_t, float* c, uint64_t m, uint64_t k, uint64_t n) {
  const uint64_t lda = a_t ? m : k, ldb = b_t ? k : n;
  /* pack B as [k][n] once if transposed, so the inner loop streams */
  float* bp = NULL;
  if (b_t) {
    bp = (float*)malloc(sizeof(float) * k * n);
    for (uint64_t j = 0; j < n; ++j)
      for (uint64_t p = 0; p < k; ++p) bp[p * n + j] = b[j * ldb + p];
    b = bp;
  }
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t i = 0; i < (int64_t)m; ++i) {
    float* ci = c + (uint64_t)i * n;
    for (uint64_t j = 0; j < n; ++j) ci[j] = 0.0f;
    for (uint64_t p = 0; p < k; ++p) {
      const float av = a_t ? a[p * lda + i] : a[(uint64_t)i * lda + p];
      const float* bj = b + p * n;
      for (uint64_t j = 0; j < n; ++j) ci[j] = ci[j] + av * bj[j];
    }
  }
  free(bp);
}

/* The truth a product is compared against: F64 accumulation of the exact inputs, and
 * S_ij = sum_k |a_ik| |b_kj|, the reference's normaliser (step11_burn.rs:15-17,101-111). */
void orc_gemm_truth(const float* a, int a_t, const float* b, int b_t, double* c, double* s, uint64_t m, uint64_t k,
                    uint64_t n) {
  const uint64_t lda = a_t ? m : k, ldb = b_t ? k : n;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t i = 0; i < (int64_t)m; ++i) {
    double* ci = c + (uint64_t)i * n;
    double* si = s ? s + (uint64_t)i * n : NULL;
    for (uint64_t j = 0; j < n; ++j) { ci[j] = 0.0; if (si) si[j] = 0.0; }
    for (uint64_t p = 0; p < k; ++p) {
      const double av = a_t ? a[p * lda + i] : a[(uint64_t)i * lda + p];
      for (uint64_t j = 0; j < n; ++j) {
        const double bv = b_t ? b[j * ldb + p] : b[p * ldb + j];
        ci[j] += av * bv;
        if (si) si[j] += fabs(av) * fabs(bv);
      }
    }
  }
}

/* Sum over rows, [rows, cols] -> [cols]: a left fold from +0.0, rows in order
 * (crates/tt-kernels/src/sfpu/reduce.rs:31-38, test at :1162-1193). */
void orc_sum_rows_in_order(const float* a, uint64_t rows, uint64_t cols, float* out) {
  for (uint64_t c = 0; c < cols; ++c) out[c] = 0.0f;
  for (uint64_t r = 0; r < rows; ++r)
    for (uint64_t c = 0; c < cols; ++c) out[c] = out[c] + a[r * cols + c];
}

/* Full sum in the reference's order (crates/burn-tt/src/ops.rs:3329-3397): the stored
 * matrix in column chunks of 512; each chunk summed over columns, then over rows; the
 * chunk partials added in ascending order.  Within a chunk the reference's column sum is
 * a tree whose exact shape is Tensix-specific; a left fold stands in, and comparisons
 * use the bound 2 gamma_{n-1} sum|x| (crates/tt-tests/tests/step63_burn_full_reduce.rs:104-122). */
float orc_full_sum(const float* a, uint64_t rows, uint64_t cols) {
  float total = 0.0f;
  for (uint64_t c0 = 0; c0 < cols; c0 += 512) {
    const uint64_t c1 = c0 + 512 < cols ? c0 + 512 : cols;
    float chunk = 0.0f;
    for (uint64_t r = 0; r < rows; ++r) {
      float rs = 0.0f;
      for (uint64_t c = c0; c < c1; ++c) rs = rs + a[r * cols + c];
      chunk = chunk + rs;
    }
    total = total + chunk;
  }
  return total;
}
double orc_full_sum_f64(const float* a, uint64_t n, double* abs_sum) {
  double s = 0.0, t = 0.0;
  for (uint64_t i = 0; i < n; ++i) { s += a[i]; t += fabs((double)a[i]); }
  if (abs_sum) *abs_sum = t;
  return s;
}

/* Row softmax of scale*x with an optional Bool mask (crates/tt-kernels/src/sfpu/softmax.rs:
 * 1-45): max clamped to >= -FLT_MAX, sum clamped to >= FLT_MIN, so a fully masked row is
 * zeros.  exp in F64, rounded once: the bound of the comparison covers a device expf. */
void orc_softmax_rows(const float* x, const uint32_t* mask, uint64_t mask_rows, float scale, int log_form, float* out,
                      uint64_t rows, uint64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const float* xr = x + (uint64_t)r * cols;
    const uint32_t* mr = mask ? mask + ((uint64_t)r % mask_rows) * cols : NULL;
    float* o = out + (uint64_t)r * cols;
    float m = -INFINITY;
    int has_nan = 0;
    for (uint64_t c = 0; c < cols; ++c) {
      float s = scale != 1.0f ? xr[c] * scale : xr[c];
      if (mr && mr[c]) s = -INFINITY;
      o[c] = s;
      if (s != s) has_nan = 1;
      if (s > m) m = s;
    }
    if (has_nan) m = NAN;
    if (m < -3.402823466e38f) m = -3.402823466e38f;
    float sum = 0.0f;
    for (uint64_t c = 0; c < cols; ++c) {
      const float d = o[c] - m;
      const float e = (float)exp((double)d);
      if (log_form) o[c] = d; else o[c] = e;
      sum = sum + e;
    }
    if (log_form) {
      const float l = (float)log((double)sum);
      for (uint64_t c = 0; c < cols; ++c) o[c] = o[c] - l;
    } else {
      if (sum < 1.17549435e-38f) sum = 1.17549435e-38f;
      for (uint64_t c = 0; c < cols; ++c) o[c] = o[c] / sum;
    }
  }
}

/* First maximum; any NaN beats every number and the first NaN wins; -0 == +0
 * (crates/tt-tests/tests/step211_argmax_row.rs:8-10). */
int32_t orc_argmax(const float* v, uint64_t n) {
  uint64_t best = 0;
  for (uint64_t i = 0; i < n; ++i) {
    if (v[i] != v[i]) return (int32_t)i;
  }
  for (uint64_t i = 1; i < n; ++i)
    if (v[i] > v[best]) best = i;
  return (int32_t)best;
}

/* sqrt(mean(x x) + eps) per row: MUL, sum over columns, MUL_SCALAR(1/n), ADD_SCALAR(eps),
 * SQRT (crates/tt-kernels/src/sfpu/norm.rs:1-25). The sum's order is free (bounded). */
void orc_rms(const float* a, uint64_t rows, uint64_t cols, float eps, float* out) {
  const float inv = 1.0f / (float)cols;
  for (uint64_t r = 0; r < rows; ++r) {
    float ss = 0.0f;
    for (uint64_t c = 0; c < cols; ++c) ss = ss + a[r * cols + c] * a[r * cols + c];
    out[r] = sqrtf(ss * inv + eps);
  }
}

/* Simple unary / binary maps used by the CPU baseline timing (the memory-bound suite). */
void orc_map_unary(int which, const float* a, float* out, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    const float x = a[i];
    float y;
    switch (which) {
      case 0: y = expf(x); break;
      case 1: y = logf(x); break;
      case 2: y = 1.0f / x; break;
      case 3: y = sqrtf(x); break;
      case 4: y = x > 0.0f ? x : 0.0f; break;
      case 5: y = (0.5f * x) * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * (x * x * x)))); break;
      case 6: { const float e = expf(-fabsf(x)); const float d = 1.0f + e; y = x * (x >= 0.0f ? 1.0f / d : e / d); break; }
      default: y = x;
    }
    out[i] = y;
  }
}
