/*
 * CPU oracle for the seven kernel.h kernel templates.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA kernels are
 * compared against; nothing on the product path may call it. Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * Every routine restates, in plain C, an fp64 CPU reference or an input
 * generator that the reference project keeps inside its end-to-end tests
 * (paths below are relative to the reference project root). The restatement
 * is pinned two ways: against the reference's own routines compiled from
 * their sources (oracle/ref_bridge, outputs under oracle/_ref) and against the
 * committed fixtures in tests/golden that were generated from that build.
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -shared).
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* Host thread count actually used by the parallel routines.                 */
/* ------------------------------------------------------------------------ */
int kho_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void kho_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------ */
/* Reference-exact input generators                                          */
/* ------------------------------------------------------------------------ */

/* test/unit/e2e_vecadd_test.cpp:40-46 : a[i] = (i % 257) * 0.5,
 * b[i] = (i % 331) * 0.25 + 0.5 (every value exact in fp32, b never 0). */
void kho_fill_vecadd_pattern(float *a, float *b, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    a[i] = (float)(i % 257) * 0.5f;
    b[i] = (float)(i % 331) * 0.25f + 0.5f;
  }
}

/* test/unit/e2e_gemm_test.cpp:70-75 : small exact integers in [0, 64). */
void kho_fill_gemm_pattern(float *a, float *b, int64_t m, int64_t n, int64_t k) {
  for (int64_t i = 0; i < m; ++i)
    for (int64_t kk = 0; kk < k; ++kk)
      a[i * k + kk] = (float)((i * 131 + kk * 17 + 7) & 63);
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j)
      b[kk * n + j] = (float)((kk * 97 + j * 41 + 3) & 63);
}

/* The 32-bit LCG shared by the softmax, layernorm, fused_gelu and attention
 * tests (e.g. test/unit/e2e_softmax_test.cpp:67-74): values on a 2^16-point
 * grid in [-1, 1). The seed is advanced in place so one stream can feed
 * several tensors in turn, as the layernorm test does
 * (test/unit/e2e_layernorm_test.cpp:122-125). The attention test passes its
 * seed by value (test/unit/e2e_attention_test.cpp:72): callers simply discard
 * the updated seed there. */
void kho_fill_lcg(float *v, int64_t n, uint32_t *seed) {
  uint32_t s = *seed;
  for (int64_t i = 0; i < n; ++i) {
    s = s * 1664525u + 1013904223u;
    v[i] = (float)((int32_t)(s >> 8) & 0xffff) / 32768.0f - 1.0f;
  }
  *seed = s;
}

/* 32-bit Mersenne Twister (MT19937, Matsumoto & Nishimura 1998), the engine
 * behind std::mt19937 that the scan test draws from
 * (test/unit/e2e_scan_test.cpp:63-68): x = (float)rng() * 2^-32. */
typedef struct {
  uint32_t mt[624];
  int idx;
} kho_mt19937;

static void mt_seed(kho_mt19937 *g, uint32_t seed) {
  g->mt[0] = seed;
  for (int i = 1; i < 624; ++i)
    g->mt[i] = 1812433253u * (g->mt[i - 1] ^ (g->mt[i - 1] >> 30)) + (uint32_t)i;
  g->idx = 624;
}

static uint32_t mt_next(kho_mt19937 *g) {
  if (g->idx >= 624) {
    for (int i = 0; i < 624; ++i) {
      uint32_t y = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % 624] & 0x7fffffffu);
      uint32_t v = g->mt[(i + 397) % 624] ^ (y >> 1);
      if (y & 1u) v ^= 0x9908b0dfu;
      g->mt[i] = v;
    }
    g->idx = 0;
  }
  uint32_t y = g->mt[g->idx++];
  y ^= y >> 11;
  y ^= (y << 7) & 0x9d2c5680u;
  y ^= (y << 15) & 0xefc60000u;
  y ^= y >> 18;
  return y;
}

void kho_fill_mt19937_unit(float *v, int64_t n, uint32_t seed) {
  kho_mt19937 g;
  mt_seed(&g, seed);
  for (int64_t i = 0; i < n; ++i)
    v[i] = (float)mt_next(&g) * (1.0f / 4294967296.0f);
}

/* ------------------------------------------------------------------------ */
/* Synthetic generators for the benchmark configurations                     */
/*                                                                            */
/* The benchmark configurations name distributions (U[-1,1), U[0,1), N(0,1),  */
/* ...) that the reference's own tests do not use. These generators define    */
/* them exactly: xoshiro256** seeded through splitmix64, uniforms from the    */
/* top 53 bits, normals by Box-Muller on two such uniforms. Values are        */
/* produced in double and rounded once to fp32.                               */
/* ------------------------------------------------------------------------ */
typedef struct {
  uint64_t s[4];
} kho_xoshiro;

static uint64_t splitmix64(uint64_t *x) {
  uint64_t z = (*x += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

static void xo_seed(kho_xoshiro *g, uint64_t seed) {
  for (int i = 0; i < 4; ++i) g->s[i] = splitmix64(&seed);
}

static inline uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

static uint64_t xo_next(kho_xoshiro *g) {
  const uint64_t result = rotl64(g->s[1] * 5, 7) * 9;
  const uint64_t t = g->s[1] << 17;
  g->s[2] ^= g->s[0];
  g->s[3] ^= g->s[1];
  g->s[1] ^= g->s[2];
  g->s[0] ^= g->s[3];
  g->s[2] ^= t;
  g->s[3] = rotl64(g->s[3], 45);
  return result;
}

static inline double xo_unit(kho_xoshiro *g) {
  return (double)(xo_next(g) >> 11) * (1.0 / 9007199254740992.0);
}

void kho_fill_uniform(float *v, int64_t n, uint64_t seed, double lo, double hi) {
  kho_xoshiro g;
  xo_seed(&g, seed);
  for (int64_t i = 0; i < n; ++i) v[i] = (float)(lo + (hi - lo) * xo_unit(&g));
}

void kho_fill_normal(float *v, int64_t n, uint64_t seed, double mean, double sigma) {
  kho_xoshiro g;
  xo_seed(&g, seed);
  const double two_pi = 6.283185307179586476925286766559;
  for (int64_t i = 0; i < n; i += 2) {
    double u1 = xo_unit(&g);
    const double u2 = xo_unit(&g);
    if (u1 < 1e-300) u1 = 1e-300;
    const double r = sqrt(-2.0 * log(u1));
    v[i] = (float)(mean + sigma * r * cos(two_pi * u2));
    if (i + 1 < n) v[i + 1] = (float)(mean + sigma * r * sin(two_pi * u2));
  }
}

/* ------------------------------------------------------------------------ */
/* fp64 references                                                            */
/* ------------------------------------------------------------------------ */

/* test/unit/e2e_vecadd_test.cpp:104-114 : the sum formed in double, rounded
 * once to fp32. `subtract` selects the negative control a-b (219-235). */
void kho_vecadd_ref(const float *a, const float *b, float *out, int64_t n, int subtract) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const double s = subtract ? (double)a[i] - (double)b[i] : (double)a[i] + (double)b[i];
    out[i] = (float)s;
  }
}

/* test/unit/e2e_gemm_test.cpp:92-108 : C = A.B with row-major A (m x k),
 * B (k x n); each output row is accumulated in double as k rank-1 updates in
 * increasing k, then rounded once to fp32. Rows [row_begin, row_end) only, so
 * a bounded sample of a large product can be formed; `out` holds
 * (row_end-row_begin) x n values. `b_transposed` selects the negative control
 * A.B^T (352-374; needs k == n). */
void kho_gemm_ref_rows(const float *a, const float *b, float *out, int64_t m, int64_t n,
                       int64_t k, int64_t row_begin, int64_t row_end, int b_transposed) {
  (void)m;
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)n);
#pragma omp for schedule(dynamic, 1)
    for (int64_t i = row_begin; i < row_end; ++i) {
      for (int64_t j = 0; j < n; ++j) acc[j] = 0.0;
      if (!b_transposed) {
        for (int64_t kk = 0; kk < k; ++kk) {
          const double av = (double)a[i * k + kk];
          const float *brow = b + kk * n;
          for (int64_t j = 0; j < n; ++j) acc[j] += av * (double)brow[j];
        }
      } else {
        for (int64_t j = 0; j < n; ++j) {
          double s = 0.0;
          for (int64_t kk = 0; kk < k; ++kk) s += (double)a[i * k + kk] * (double)b[j * k + kk];
          acc[j] = s;
        }
      }
      float *orow = out + (i - row_begin) * n;
      for (int64_t j = 0; j < n; ++j) orow[j] = (float)acc[j];
    }
    free(acc);
  }
}

void kho_gemm_ref(const float *a, const float *b, float *out, int64_t m, int64_t n, int64_t k) {
  kho_gemm_ref_rows(a, b, out, m, n, k, 0, m, 0);
}

/* Selected rows of C (for a random-row sample of a large product). */
void kho_gemm_ref_pick_rows(const float *a, const float *b, float *out, int64_t n, int64_t k,
                            const int64_t *rows, int64_t nrows) {
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)n);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r = 0; r < nrows; ++r) {
      const int64_t i = rows[r];
      for (int64_t j = 0; j < n; ++j) acc[j] = 0.0;
      for (int64_t kk = 0; kk < k; ++kk) {
        const double av = (double)a[i * k + kk];
        const float *brow = b + kk * n;
        for (int64_t j = 0; j < n; ++j) acc[j] += av * (double)brow[j];
      }
      for (int64_t j = 0; j < n; ++j) out[r * n + j] = (float)acc[j];
    }
    free(acc);
  }
}

/* test/unit/e2e_softmax_test.cpp:78-91 : true row maximum, then
 * exp(x-max)/sum, all in double. `uniform_control` gives the negative
 * control 1/cols (323 onward). */
void kho_softmax_ref(const float *x, double *out, int64_t rows, int64_t cols, int uniform_control) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    double *orow = out + r * cols;
    if (uniform_control) {
      for (int64_t c = 0; c < cols; ++c) orow[c] = 1.0 / (double)cols;
      continue;
    }
    double m = (double)xr[0];
    for (int64_t c = 1; c < cols; ++c)
      if ((double)xr[c] > m) m = (double)xr[c];
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += exp((double)xr[c] - m);
    for (int64_t c = 0; c < cols; ++c) orow[c] = exp((double)xr[c] - m) / s;
  }
}

/* test/unit/e2e_layernorm_test.cpp:68-91 : mean, biased variance (divide by
 * cols) and 1/sqrt(var+eps) in double; eps is a parameter because the
 * negative control uses eps = 0 (336-425). */
void kho_layernorm_ref(const float *x, const float *gamma, const float *beta, double *out,
                       int64_t rows, int64_t cols, double eps) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    double *orow = out + r * cols;
    double mean = 0.0;
    for (int64_t c = 0; c < cols; ++c) mean += (double)xr[c];
    mean /= (double)cols;
    double var = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      const double d = (double)xr[c] - mean;
      var += d * d;
    }
    var /= (double)cols;
    const double inv = 1.0 / sqrt(var + eps);
    for (int64_t c = 0; c < cols; ++c)
      orow[c] = ((double)xr[c] - mean) * inv * (double)gamma[c] + (double)beta[c];
  }
}

/* test/unit/e2e_scan_test.cpp:159-172 : running double sum, each prefix
 * rounded to fp32. `exclusive` selects the negative control (260-285). */
void kho_scan_ref(const float *x, float *out, int64_t n, int exclusive) {
  double acc = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    const double xv = (double)x[i];
    const double pref = exclusive ? acc : acc + xv;
    acc += xv;
    out[i] = (float)pref;
  }
}

/* test/unit/e2e_fused_gelu_test.cpp:59-70 : t = alpha*x + beta (the
 * reference fixes alpha = 1.5, beta = 0.5), tanh-form GELU of t in double.
 * `no_tanh_control` replaces tanh(z) by z (the negative control, 72-76). */
static inline double gelu_tanh_f64(double t, int no_tanh) {
  const double c = 0.7978845608;
  const double d = 0.044715;
  const double z = c * (t + d * t * t * t);
  return 0.5 * t * (1.0 + (no_tanh ? z : tanh(z)));
}

void kho_fused_gelu_ref(const float *x, double *out, int64_t n, double alpha, double beta,
                        int no_tanh_control) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    out[i] = gelu_tanh_f64(alpha * (double)x[i] + beta, no_tanh_control);
}

/* The benchmark's bias form: y = GELU_tanh(x + bias), same tanh-form GELU. */
void kho_bias_gelu_ref(const float *x, const float *bias, double *out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = gelu_tanh_f64((double)x[i] + (double)bias[i], 0);
}

/* test/unit/e2e_attention_test.cpp:87-122 : per query row, scores (times
 * 1/sqrt(head_dim) when `scaled`), max, exp, sum, then sum_t p/l * V, all in
 * double. Tensors are [batch, heads, seq, head_dim] contiguous. The range
 * [bh_begin, bh_end) of flattened (batch, head) problems is computed; `out`
 * is indexed like the full tensor. */
void kho_attention_ref(const float *q, const float *k, const float *v, double *out, int64_t batch,
                       int64_t heads, int64_t seq, int64_t head_dim, int scaled, int64_t bh_begin,
                       int64_t bh_end) {
  (void)batch;
  (void)heads;
  const double scale = scaled ? 1.0 / sqrt((double)head_dim) : 1.0;
  const int64_t per = seq * head_dim;
#pragma omp parallel
  {
    double *s = (double *)malloc(sizeof(double) * (size_t)seq);
#pragma omp for schedule(dynamic, 8) collapse(2)
    for (int64_t bh = bh_begin; bh < bh_end; ++bh) {
      for (int64_t i = 0; i < seq; ++i) {
        const float *qrow = q + bh * per + i * head_dim;
        const float *kmat = k + bh * per;
        const float *vmat = v + bh * per;
        double m = -INFINITY;
        for (int64_t t = 0; t < seq; ++t) {
          double dot = 0.0;
          for (int64_t d = 0; d < head_dim; ++d)
            dot += (double)qrow[d] * (double)kmat[t * head_dim + d];
          s[t] = dot * scale;
          if (s[t] > m) m = s[t];
        }
        double l = 0.0;
        for (int64_t t = 0; t < seq; ++t) {
          s[t] = exp(s[t] - m);
          l += s[t];
        }
        double *orow = out + bh * per + i * head_dim;
        for (int64_t j = 0; j < head_dim; ++j) {
          double acc = 0.0;
          for (int64_t t = 0; t < seq; ++t) acc += s[t] / l * (double)vmat[t * head_dim + j];
          orow[j] = acc;
        }
      }
    }
    free(s);
  }
}

/* ------------------------------------------------------------------------ */
/* Comparison metrics                                                         */
/* ------------------------------------------------------------------------ */

/* got (fp32) against a double reference. Fills:
 *   max_abs          max |got - ref|
 *   max_rel          max |got - ref| / max(|ref|, rms(ref)): the relative error
 *                    the parity bounds are stated on. fp32 arithmetic cannot
 *                    promise a small per-element relative error where a sum
 *                    cancels to (nearly) zero, so elements smaller than the
 *                    tensor's rms are measured against the rms instead.
 *   max_rel_floored  the same with the floor at 1e-3 * rms(ref) (reported only)
 *   rel_frobenius    sqrt(sum (got-ref)^2 / sum ref^2)
 *                    (test/unit/e2e_gemm_test.cpp:111-122)
 *   max_violation    max (|got - ref| - rtol * |ref|), the attention test's
 *                    acceptance quantity (test/unit/e2e_attention_test.cpp:299-306)
 *   non_finite       count of NaN/Inf in `got`
 * A NaN in either operand makes max_abs NaN so that a comparison "<= tol"
 * fails, as it does in the reference's tests. */
void kho_compare_f32_f64(const float *got, const double *ref, int64_t n, double rtol,
                         kho_compare_result *res) {
  double sum_sq = 0.0;
  for (int64_t i = 0; i < n; ++i) sum_sq += ref[i] * ref[i];
  const double rms = n > 0 ? sqrt(sum_sq / (double)n) : 0.0;
  const double floor_v = 1e-3 * rms;
  double max_abs = 0.0, max_rel = 0.0, max_rel_rms = 0.0, diff_sq = 0.0, max_viol = -INFINITY;
  int64_t non_finite = 0;
  int saw_nan = 0;
  for (int64_t i = 0; i < n; ++i) {
    const double g = (double)got[i];
    if (!isfinite(g)) ++non_finite;
    const double d = fabs(g - ref[i]);
    if (isnan(d)) {
      saw_nan = 1;
      continue;
    }
    if (d > max_abs) max_abs = d;
    const double den = fabs(ref[i]) > floor_v ? fabs(ref[i]) : floor_v;
    if (den > 0.0 && d / den > max_rel) max_rel = d / den;
    const double den2 = fabs(ref[i]) > rms ? fabs(ref[i]) : rms;
    if (den2 > 0.0 && d / den2 > max_rel_rms) max_rel_rms = d / den2;
    else if (den2 == 0.0 && d > 0.0) max_rel_rms = INFINITY;
    diff_sq += d * d;
    const double viol = d - rtol * fabs(ref[i]);
    if (viol > max_viol) max_viol = viol;
  }
  res->max_abs = saw_nan ? NAN : max_abs;
  res->max_rel_floored = saw_nan ? NAN : max_rel;
  res->max_rel = saw_nan ? NAN : max_rel_rms;
  res->rel_frobenius = saw_nan ? NAN : (sum_sq > 0.0 ? sqrt(diff_sq / sum_sq) : sqrt(diff_sq));
  res->max_violation = saw_nan ? NAN : max_viol;
  res->non_finite = non_finite;
  res->ref_rms = rms;
}

void kho_compare_f32_f32(const float *got, const float *ref, int64_t n, double rtol,
                         kho_compare_result *res) {
  double *tmp = (double *)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
  for (int64_t i = 0; i < n; ++i) tmp[i] = (double)ref[i];
  kho_compare_f32_f64(got, tmp, n, rtol, res);
  free(tmp);
}

/* Number of positions whose 32-bit patterns differ (vecadd's bit-exact bar). */
int64_t kho_count_bit_mismatch(const float *got, const float *ref, int64_t n) {
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i) {
    uint32_t a, b;
    memcpy(&a, got + i, 4);
    memcpy(&b, ref + i, 4);
    if (a != b) ++bad;
  }
  return bad;
}

/* 64-bit FNV-1a over raw bytes: the fixture files store this instead of whole
 * tensors. */
uint64_t kho_fnv1a(const void *data, int64_t bytes) {
  const unsigned char *p = (const unsigned char *)data;
  uint64_t h = 0xcbf29ce484222325ull;
  for (int64_t i = 0; i < bytes; ++i) {
    h ^= p[i];
    h *= 0x100000001b3ull;
  }
  return h;
}
