/*
 * CPU restatement of primitiv's minibatch-broadcasting matrix product.
 *
 * TEST INFRASTRUCTURE ONLY.  The shipped library never links, loads or calls
 * anything in this directory; only the test-suite, the smoke check and the
 * bench's CPU-baseline leg do, and only as the checker.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks every function below
 * against (1) the known-answer vectors of the reference's own matmul tests
 * (test/tensor_forward_test.cc:1798-1905, test/tensor_backward_test.cc:1599-1668,
 * test/operator_impl_test.cc:1132-1144, kept as tests/golden/matmul_known_answers.json)
 * and (2) outputs of the reference's own Naive device compiled from its sources
 * (oracle/_ref/libprimitiv_c.so) on seeded random inputs.
 *
 * Layout (primitiv/core/device.h:298-299): every tensor is column-major and
 * densely packed, the minibatch is the outermost stride, so element (i, j, n)
 * of a Shape({r, c}, batch) tensor is at  i + j*r + n*r*c.
 * An operand with batch == 1 is broadcast over the other operand's batch.
 */
#ifndef PRIMITIV_B200_ORACLE_MATMUL_H_
#define PRIMITIV_B200_ORACLE_MATMUL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * y[n] = a[n or 0] . b[n or 0], overwrite.
 * Same loop nest, blocking (8x8x8) and fp32 summation order as
 * primitiv/devices/naive/ops/matmul.cc:9-50, so the result is bit-identical
 * to the reference Naive device.
 * a: {di, dj} x ba, b: {dj, dk} x bb, y: {di, dk} x max(ba, bb).
 */
void oracle_matmul_fw_naive_f32(
    const float *a, const float *b, float *y,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb);

/*
 * ga[n or 0] += gy[n] . b[n or 0]^T ;  gb[n or 0] += a[n or 0]^T . gy[n].
 * Follows primitiv/devices/naive/ops/matmul.cc:52-58: transpose the operand,
 * run the forward product above into a {.,.} x batch temporary, then
 * inplace_add it (summing over the batch for a broadcast destination, in
 * batch order, as primitiv/devices/naive/ops/inplace_add.cc does).
 * Bit-identical to the reference Naive device.
 */
void oracle_matmul_bw_naive_f32(
    const float *a, const float *b, const float *gy, float *ga, float *gb,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb);

/*
 * The same two contractions with the call structure of
 * primitiv/devices/eigen/ops/matmul.cc:9-79 (per-batch products when `a` has a
 * batch, else one product over the combined {dj, dk*bb} matrix), evaluated in
 * fp64 from fp32 inputs.  This is the arbiter for normwise error.
 * y64 is overwritten; ga64 / gb64 must hold the pre-fill on entry (+=).
 * Multi-threaded with OpenMP over output columns.
 */
void oracle_matmul_fw_f64(
    const float *a, const float *b, double *y64,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb);

void oracle_matmul_bw_f64(
    const float *a, const float *b, const float *gy, double *ga64, double *gb64,
    uint32_t di, uint32_t dj, uint32_t dk, uint32_t ba, uint32_t bb);

/* sqrt(sum (x - ref)^2) / sqrt(sum ref^2) over n elements (0 if both are 0). */
double oracle_normwise_rel_err_f32(const float *x, const double *ref, uint64_t n);

/* Round fp32 -> IEEE half (nearest even) -> fp32, as the CUDA16 device stores. */
void oracle_round_to_half(const float *x, float *y, uint64_t n);

#ifdef __cplusplus
}
#endif

#endif  /* PRIMITIV_B200_ORACLE_MATMUL_H_ */
