/*
 * CPU restatement of primitiv's matmul_fw / matmul_bw.  TEST INFRASTRUCTURE ONLY:
 * see matmul_oracle.h for who may call this and for the parity pins.
 *
 * Build: gcc -O3 -ffp-contract=off -fopenmp -fPIC -shared (see Makefile).
 * -ffp-contract=off matters: the *_naive_f32 functions promise the reference
 * Naive device's exact fp32 rounding sequence, which has no fused multiply-add.
 */
#include "matmul_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

static inline uint32_t umin(uint32_t a, uint32_t b) { return a < b ? a : b; }

/*
 * One {di,dj}.{dj,dk} product.  The reference (naive/ops/matmul.cc:26-45) walks
 * 8x8x8 blocks; what that fixes numerically is, for every output element, the
 * order of additions: the contraction index is cut into runs of 8, each run is
 * summed from zero in fp32, and the run totals are added to the output in order.
 * Output elements are independent, so they are simply visited column by column.
 */
static void product_naive_order(
    const float *a, const float *b, float *y,
    uint32_t di, uint32_t dj, uint32_t dk) {
  for (uint32_t col = 0; col < dk; ++col) {
    const float *bcol = b + (size_t)col * dj;
    float *ycol = y + (size_t)col * di;
    for (uint32_t row = 0; row < di; ++row) {
      float acc = 0.0f;
      for (uint32_t j0 = 0; j0 < dj; j0 += 8) {
        const uint32_t j1 = umin(j0 + 8, dj);
        float run = 0.0f;
        for (uint32_t j = j0; j < j1; ++j) {
          run += a[row + (size_t)j * di] * bcol[j];
        }
        acc += run;
      }
      ycol[row] = acc;
    }
  }
}

void oracle_matmul_fw_naive_f32(
    const float *a, const float *b, float *y,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb) {
  const uint32_t bs = ba > bb ? ba : bb;
  const size_t sa = ba > 1 ? (size_t)di * dj : 0;
  const size_t sb = bb > 1 ? (size_t)dj * dk : 0;
  const size_t sy = (size_t)di * dk;
#pragma omp parallel for schedule(dynamic, 1)
  for (uint32_t n = 0; n < bs; ++n) {
    product_naive_order(a + n * sa, b + n * sb, y + n * sy, di, dj, dk);
  }
}

/* {r,c} x bs column-major -> {c,r} x bs (naive/ops/transpose.cc:9-28). */
static float *transposed_copy(const float *x, uint32_t r, uint32_t c, uint32_t bs) {
  float *t = (float *)malloc(sizeof(float) * (size_t)r * c * bs);
  for (uint32_t n = 0; n < bs; ++n) {
    const float *src = x + (size_t)n * r * c;
    float *dst = t + (size_t)n * r * c;
    for (uint32_t j = 0; j < c; ++j)
      for (uint32_t i = 0; i < r; ++i)
        dst[j + (size_t)i * c] = src[i + (size_t)j * r];
  }
  return t;
}

/* dest[n or 0] += src[n], batch order (naive/ops/inplace_add.cc:9-25). */
static void accumulate_batches(
    const float *src, float *dest, size_t vol, uint32_t bs_src, uint32_t bs_dest) {
  const uint32_t bs = bs_src > bs_dest ? bs_src : bs_dest;
  for (uint32_t n = 0; n < bs; ++n) {
    const float *s = src + (bs_src > 1 ? n * vol : 0);
    float *d = dest + (bs_dest > 1 ? n * vol : 0);
    for (size_t i = 0; i < vol; ++i) d[i] += s[i];
  }
}

void oracle_matmul_bw_naive_f32(
    const float *a, const float *b, const float *gy, float *ga, float *gb,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb) {
  const uint32_t bs = ba > bb ? ba : bb;
  /* ga += matmul_fw(gy, transpose(b)) : {di,dk}xbs . {dk,dj}xbb -> {di,dj}xbs */
  {
    float *bt = transposed_copy(b, dj, dk, bb);
    float *tmp = (float *)malloc(sizeof(float) * (size_t)di * dj * bs);
    oracle_matmul_fw_naive_f32(gy, bt, tmp, di, dk, dj, bs, bb);
    accumulate_batches(tmp, ga, (size_t)di * dj, bs, ba);
    free(tmp);
    free(bt);
  }
  /* gb += matmul_fw(transpose(a), gy) : {dj,di}xba . {di,dk}xbs -> {dj,dk}xbs */
  {
    float *at = transposed_copy(a, di, dj, ba);
    float *tmp = (float *)malloc(sizeof(float) * (size_t)dj * dk * bs);
    oracle_matmul_fw_naive_f32(at, gy, tmp, dj, di, dk, ba, bs);
    accumulate_batches(tmp, gb, (size_t)dj * dk, bs, bb);
    free(tmp);
    free(at);
  }
}

/* ---- fp64 arbiter, Eigen-device call structure (eigen/ops/matmul.cc) ---- */

/* c (m x n, ld m) = or += a (m x k, col-major) . b (k x n, col-major). */
static void gemm_nn_f64(const float *a, const float *b, double *c,
                        size_t m, size_t n, size_t k, int accumulate) {
#pragma omp parallel for schedule(static)
  for (size_t col = 0; col < n; ++col) {
    double *cc = c + col * m;
    if (!accumulate) memset(cc, 0, sizeof(double) * m);
    for (size_t p = 0; p < k; ++p) {
      const double bv = (double)b[p + col * k];
      const float *ac = a + p * m;
      for (size_t row = 0; row < m; ++row) cc[row] += (double)ac[row] * bv;
    }
  }
}

/* c (m x n) += a (m x k, col-major) . b^T, b is (n x k, col-major). */
static void gemm_nt_f64(const float *a, const float *b, double *c,
                        size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
  for (size_t col = 0; col < n; ++col) {
    double *cc = c + col * m;
    for (size_t p = 0; p < k; ++p) {
      const double bv = (double)b[col + p * n];
      const float *ac = a + p * m;
      for (size_t row = 0; row < m; ++row) cc[row] += (double)ac[row] * bv;
    }
  }
}

/* c (m x n) += a^T . b, a is (k x m, col-major), b is (k x n, col-major). */
static void gemm_tn_f64(const float *a, const float *b, double *c,
                        size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
  for (size_t col = 0; col < n; ++col) {
    const float *bc = b + col * k;
    for (size_t row = 0; row < m; ++row) {
      const float *ac = a + row * k;
      double s = 0.0;
      for (size_t p = 0; p < k; ++p) s += (double)ac[p] * (double)bc[p];
      c[row + col * m] += s;
    }
  }
}

void oracle_matmul_fw_f64(
    const float *a, const float *b, double *y64,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb) {
  if (ba > 1) {  /* eigen/ops/matmul.cc:18-29 */
    const size_t a_skip = (size_t)di * dj;
    const size_t b_skip = bb > 1 ? (size_t)dj * dk : 0;
    const size_t y_skip = (size_t)di * dk;
    for (uint32_t n = 0; n < ba; ++n)
      gemm_nn_f64(a + n * a_skip, b + n * b_skip, y64 + n * y_skip, di, dk, dj, 0);
  } else {       /* eigen/ops/matmul.cc:30-37: one product over dk*bb columns */
    gemm_nn_f64(a, b, y64, di, (size_t)dk * bb, dj, 0);
  }
}

void oracle_matmul_bw_f64(
    const float *a, const float *b, const float *gy, double *ga64, double *gb64,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb) {
  if (ba > 1) {  /* eigen/ops/matmul.cc:53-67 */
    const size_t a_skip = (size_t)di * dj;
    const size_t b_skip = bb > 1 ? (size_t)dj * dk : 0;
    const size_t y_skip = (size_t)di * dk;
    for (uint32_t n = 0; n < ba; ++n) {
      gemm_nt_f64(gy + n * y_skip, b + n * b_skip, ga64 + n * a_skip, di, dj, dk);
      gemm_tn_f64(a + n * a_skip, gy + n * y_skip, gb64 + n * b_skip, dj, dk, di);
    }
  } else {       /* eigen/ops/matmul.cc:68-78 */
    const size_t dkb = (size_t)dk * bb;
    gemm_nt_f64(gy, b, ga64, di, dj, dkb);
    gemm_tn_f64(a, gy, gb64, dj, dkb, di);
  }
}

double oracle_normwise_rel_err_f32(const float *x, const double *ref, uint64_t n) {
  double num = 0.0, den = 0.0;
#pragma omp parallel for reduction(+ : num, den)
  for (uint64_t i = 0; i < n; ++i) {
    const double d = (double)x[i] - ref[i];
    num += d * d;
    den += ref[i] * ref[i];
  }
  if (den == 0.0) return num == 0.0 ? 0.0 : INFINITY;
  return sqrt(num / den);
}

static float half_round_trip(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint32_t sign = u & 0x80000000u;
  uint32_t mag = u & 0x7fffffffu;
  float out;
  if (mag >= 0x7f800000u) {            /* inf / nan stay */
    out = f;
    return out;
  }
  if (mag >= 0x477ff000u) {            /* rounds to >= 65520 -> inf */
    mag = 0x7f800000u;
  } else if (mag < 0x38800000u) {      /* below the smallest normal half 2^-14 */
    /* subnormal half: quantum 2^-24; round to nearest even through fp32 add */
    float a;
    memcpy(&a, &mag, 4);
    const float magic = 0.5f;          /* ulp(0.5f) = 2^-24 */
    a = (a + magic) - magic;
    memcpy(&mag, &a, 4);
  } else {                             /* normal: keep 10 mantissa bits, RNE */
    const uint32_t lsb = (mag >> 13) & 1u;
    mag += 0x0fffu + lsb;
    mag &= ~0x1fffu;
  }
  u = sign | mag;
  memcpy(&out, &u, 4);
  return out;
}

void oracle_round_to_half(const float *x, float *y, uint64_t n) {
#pragma omp parallel for
  for (uint64_t i = 0; i < n; ++i) y[i] = half_round_trip(x[i]);
}
