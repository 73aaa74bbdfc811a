/*
 * CPU oracle (test infrastructure, never on the product path): declarations.
 * See oracle.c for what each routine restates and where it comes from.
 */
#ifndef KERNELH_B200_ORACLE_H
#define KERNELH_B200_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  double max_abs;
  double max_rel_floored;
  double max_rel;
  double rel_frobenius;
  double max_violation;
  double ref_rms;
  int64_t non_finite;
} kho_compare_result;

int kho_num_threads(void);
void kho_set_num_threads(int n);

/* reference-exact generators */
void kho_fill_vecadd_pattern(float *a, float *b, int64_t n);
void kho_fill_gemm_pattern(float *a, float *b, int64_t m, int64_t n, int64_t k);
void kho_fill_lcg(float *v, int64_t n, uint32_t *seed);
void kho_fill_mt19937_unit(float *v, int64_t n, uint32_t seed);

/* synthetic generators for the benchmark configurations */
void kho_fill_uniform(float *v, int64_t n, uint64_t seed, double lo, double hi);
void kho_fill_normal(float *v, int64_t n, uint64_t seed, double mean, double sigma);

/* fp64 references */
void kho_vecadd_ref(const float *a, const float *b, float *out, int64_t n, int subtract);
void kho_gemm_ref(const float *a, const float *b, float *out, int64_t m, int64_t n, int64_t k);
void kho_gemm_ref_rows(const float *a, const float *b, float *out, int64_t m, int64_t n,
                       int64_t k, int64_t row_begin, int64_t row_end, int b_transposed);
void kho_gemm_ref_pick_rows(const float *a, const float *b, float *out, int64_t n, int64_t k,
                            const int64_t *rows, int64_t nrows);
void kho_softmax_ref(const float *x, double *out, int64_t rows, int64_t cols, int uniform_control);
void kho_layernorm_ref(const float *x, const float *gamma, const float *beta, double *out,
                       int64_t rows, int64_t cols, double eps);
void kho_scan_ref(const float *x, float *out, int64_t n, int exclusive);
void kho_fused_gelu_ref(const float *x, double *out, int64_t n, double alpha, double beta,
                        int no_tanh_control);
void kho_bias_gelu_ref(const float *x, const float *bias, double *out, int64_t n);
void kho_attention_ref(const float *q, const float *k, const float *v, double *out, int64_t batch,
                       int64_t heads, int64_t seq, int64_t head_dim, int scaled, int64_t bh_begin,
                       int64_t bh_end);

/* comparison metrics */
void kho_compare_f32_f64(const float *got, const double *ref, int64_t n, double rtol,
                         kho_compare_result *res);
void kho_compare_f32_f32(const float *got, const float *ref, int64_t n, double rtol,
                         kho_compare_result *res);
int64_t kho_count_bit_mismatch(const float *got, const float *ref, int64_t n);
uint64_t kho_fnv1a(const void *data, int64_t bytes);

#ifdef __cplusplus
}
#endif

#endif
