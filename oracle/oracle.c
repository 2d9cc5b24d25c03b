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
 * -O3 -fno-fast-math -ffp-contract=off so no product-sum is fused and no sum is reassociated.
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
/* The F32 product: every element is the left fold over k ascending of separately rounded products and
 * sums (no fused multiply-add), which is what a plain scalar loop gives.  The loops are blocked for the
 * caches and four rows share each load of B, but an element's own sequence of additions is untouched,
 * so the bits are those of the scalar loop whatever the vector width (the clones differ in nothing else). */
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define ORC_CLONES __attribute__((target_clones("avx512f", "avx2", "default")))
#else
#define ORC_CLONES
#endif
enum { ORC_JB = 512, ORC_KB = 256, ORC_IB = 4 };

ORC_CLONES
static void orc_gemm_rows(const float* a, uint64_t lda, int a_t, const float* b, uint64_t n, float* c, uint64_t i0,
                          uint64_t rows, uint64_t k) {
  for (uint64_t r = 0; r < rows; ++r)
    for (uint64_t j = 0; j < n; ++j) c[(i0 + r) * n + j] = 0.0f;
  for (uint64_t j0 = 0; j0 < n; j0 += ORC_JB) {
    const uint64_t jn = (j0 + ORC_JB <= n ? ORC_JB : n - j0);
    for (uint64_t p0 = 0; p0 < k; p0 += ORC_KB) {
      const uint64_t pn = (p0 + ORC_KB <= k ? p0 + ORC_KB : k);
      if (rows == ORC_IB) {
        float* c0 = c + (i0 + 0) * n + j0;
        float* c1 = c + (i0 + 1) * n + j0;
        float* c2 = c + (i0 + 2) * n + j0;
        float* c3 = c + (i0 + 3) * n + j0;
        for (uint64_t p = p0; p < pn; ++p) {
          const float a0 = a_t ? a[p * lda + i0 + 0] : a[(i0 + 0) * lda + p];
          const float a1 = a_t ? a[p * lda + i0 + 1] : a[(i0 + 1) * lda + p];
          const float a2 = a_t ? a[p * lda + i0 + 2] : a[(i0 + 2) * lda + p];
          const float a3 = a_t ? a[p * lda + i0 + 3] : a[(i0 + 3) * lda + p];
          const float* bj = b + p * n + j0;
          for (uint64_t j = 0; j < jn; ++j) {
            const float bv = bj[j];
            c0[j] = c0[j] + a0 * bv;
            c1[j] = c1[j] + a1 * bv;
            c2[j] = c2[j] + a2 * bv;
            c3[j] = c3[j] + a3 * bv;
          }
        }
      } else {
        for (uint64_t r = 0; r < rows; ++r) {
          float* cr = c + (i0 + r) * n + j0;
          for (uint64_t p = p0; p < pn; ++p) {
            const float av = a_t ? a[p * lda + i0 + r] : a[(i0 + r) * lda + p];
            const float* bj = b + p * n + j0;
            for (uint64_t j = 0; j < jn; ++j) cr[j] = cr[j] + av * bj[j];
          }
        }
      }
    }
  }
}

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
  const int64_t blocks = (int64_t)((m + ORC_IB - 1) / ORC_IB);
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t ib = 0; ib < blocks; ++ib) {
    const uint64_t i0 = (uint64_t)ib * ORC_IB;
    orc_gemm_rows(a, lda, a_t, b, n, c, i0, (i0 + ORC_IB <= m ? ORC_IB : m - i0), k);
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

/* The seeded uniform draw of oracle.py (`uniform`): splitmix64 from seed ^ tag, the top 24 bits as
 * k 2^-24, then lo + (hi - lo) k with separate F32 roundings.  The same numbers as the NumPy form,
 * for the tensors of tens of millions of elements the full-size parity tests draw. */
void orc_uniform(uint64_t seed, uint64_t tag, uint64_t n, float lo, float hi, float* out) {
  const uint64_t s0 = seed ^ tag;
  const float span = hi - lo;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    uint64_t z = s0 + 0x9E3779B97F4A7C15ull * (uint64_t)(i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    const float u = (float)(z >> 40) / 16777216.0f;
    const float t = span * u;
    out[i] = lo + t;
  }
}

/* oracle.py `ulp_error`: the largest |got - want| in units of 2^-24 max(|want|, 2^-125); words that are
 * equal, and two NaNs, count as no error; anything else not finite counts as infinite. */
double orc_ulp_error(const uint32_t* got, const uint32_t* want, uint64_t n) {
  double worst = 0.0;
#pragma omp parallel for schedule(static) reduction(max : worst)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    if (got[i] == want[i]) continue;
    float gf, wf;
    memcpy(&gf, &got[i], 4);
    memcpy(&wf, &want[i], 4);
    const double g = gf, w = wf;
    if (isnan(g) && isnan(w)) continue;
    double scale = fabs(w);
    if (!(scale > 0x1p-125)) scale = 0x1p-125;     /* also when want is a NaN */
    double e = fabs(g - w) / (scale * 0x1p-24);
    if (!isfinite(e)) e = INFINITY;
    if (e > worst) worst = e;
  }
  return worst;
}

/* The seeded normal draw of oracle.py (`normal`) for large tensors: Box-Muller on draws i and n + i of the
 * splitmix64 stream, in F64, rounded once to F32.  libm's log and cos may differ from NumPy's in the last
 * place of an F64, so a value can differ from the NumPy form's by one F32 step; a draw is reproducible
 * within this form, and nothing compares the two. */
void orc_normal(uint64_t seed, uint64_t tag, uint64_t n, double sigma, float* out) {
  const uint64_t s0 = seed ^ tag;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    uint64_t z[2];
    for (int h = 0; h < 2; ++h) {
      uint64_t v = s0 + 0x9E3779B97F4A7C15ull * (uint64_t)(i + 1 + (h ? (int64_t)n : 0));
      v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
      v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
      z[h] = v ^ (v >> 31);
    }
    const double u1 = ((double)(z[0] >> 40) + 1.0) / 16777216.0;
    const double u2 = (double)(z[1] >> 40) / 16777216.0;
    const double g = sqrt(-2.0 * log(u1)) * cos(2.0 * 3.14159265358979323846 * u2);
    out[i] = (float)(g * sigma);
  }
}
