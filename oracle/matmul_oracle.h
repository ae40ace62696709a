/* TEST INFRASTRUCTURE — the CPU oracle.  Never linked into, imported by or
 * executed from the product path; only tests, the smoke check and the
 * benchmark's CPU-baseline leg may use it.
 *
 * A plain-C restatement of the reference engine's CPU arithmetic for its matrix
 * product hot path, each function citing the reference file:line it follows
 * (paths relative to the reference project root).  Parity status: PINNED —
 * checked bit-for-bit against the unmodified reference compiled from its own
 * sources (oracle/_ref, see the Makefile) and against the reference's own
 * known-answer and PyTorch golden vectors (tests/golden/).
 */
#ifndef B200_MATMUL_ORACLE_H
#define B200_MATMUL_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* C = A x B, batched.  Restates Tensor::matmul's CPU loop, src/tensor_ops.cpp:543-562:
 * C zero-filled, then for every output row: for k ascending: a = A[row,k];
 * if (a == 0) continue; for j: C[row,j] += a * B[k,j]   (fp32 multiply, then fp32 add —
 * no fused multiply-add, as in the reference's Release build).
 * a_batched / b_batched == 0 means the operand is one matrix shared by every
 * batch element (stride 0, src/tensor_ops.cpp:514-515).
 * Rows are independent, so any thread count gives bit-identical output
 * (tests/test_tensor.cpp:456-476); threads <= 0 uses every core. */
void oracle_matmul_f32(const float* a, const float* b, float* c, size_t batch, size_t M, size_t K,
                       size_t N, int a_batched, int b_batched, int threads);

/* dst[b][j][i] = src[b][i][j] — the materialised transpose the reference's backward
 * pass and attention/conv call sites build before a plain product
 * (Tensor::transpose, src/tensor_ops.cpp:335-370). */
void oracle_transpose_f32(const float* src, float* dst, size_t batch, size_t rows, size_t cols);

/* The transposed forms, computed exactly as the reference computes them: materialise
 * the transpose, then the plain product above.
 *   NT: C = A x B^T, B stored (batch?, N, K)   — dA = dC x B^T, Q x K^T, cols x W^T
 *   TN: C = A^T x B, A stored (batch?, K, M)   — dB = A^T x dC */
void oracle_matmul_nt_f32(const float* a, const float* b, float* c, size_t batch, size_t M,
                          size_t K, size_t N, int a_batched, int b_batched, int threads);
void oracle_matmul_tn_f32(const float* a, const float* b, float* c, size_t batch, size_t M,
                          size_t K, size_t N, int a_batched, int b_batched, int threads);

/* Backward of C = A x B for a given dC (matmul's backward lambda,
 * src/tensor_ops.cpp:570-585): dA = dC x B^T, dB = A^T x dC; the gradient of an
 * operand shared across the batch is the sum of the per-batch contributions in
 * ascending batch order (fold_leading, src/tensor_detail.hpp:182-206).
 * grad_a / grad_b have the shapes of a / b. */
void oracle_matmul_backward_f32(const float* a, const float* b, const float* grad_c, float* grad_a,
                                float* grad_b, size_t batch, size_t M, size_t K, size_t N,
                                int a_batched, int b_batched, int threads);

/* out = op(A) x op(B) with fp64 accumulation of the fp32 inputs (not in the reference):
 * separates the fp32 oracle's own rounding drift from a kernel's error.
 * op(A) is M x K: element (i,k) at a[i*lda + k] (trans_a == 0) or a[k*lda + i]. */
void oracle_matmul_f64(const float* a, const float* b, double* c, size_t M, size_t K, size_t N,
                       int trans_a, int trans_b, size_t lda, size_t ldb, int threads);

/* Tensor::softmax over the last axis and its backward (src/tensor_ops.cpp:621-668), in the
 * reference's operation order. */
void oracle_softmax_rows_f32(const float* x, float* y, size_t rows, size_t cols);
void oracle_softmax_backward_f32(const float* y, const float* g, float* dx, size_t rows, size_t cols);

/* The reference's random streams: one global std::mt19937 (src/tensor.cpp:24-31) drawn
 * through std::uniform_real_distribution<float> (Tensor::rand, src/tensor.cpp:117-125) and
 * std::normal_distribution<float> (Tensor::randn, src/tensor.cpp:127-135), restated for
 * libstdc++'s algorithms so the same seed gives the same bytes. */
typedef struct oracle_rng {
    uint32_t mt[624];
    int idx;
} oracle_rng;

void oracle_seed(oracle_rng* g, uint64_t seed);
void oracle_rand(oracle_rng* g, float* out, size_t n, float lo, float hi);
void oracle_randn(oracle_rng* g, float* out, size_t n, float mean, float stddev);

#ifdef __cplusplus
}
#endif
#endif
