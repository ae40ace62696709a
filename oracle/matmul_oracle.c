/* TEST INFRASTRUCTURE — the CPU oracle (see matmul_oracle.h).  Plain C11; built with
 * -ffp-contract=off so every product is rounded to fp32 before it is added, which is
 * what the reference's Release build (no -march, no -mfma) does. */
#include "matmul_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <stdatomic.h>
#include <unistd.h>

/* A minimal row-parallel loop: workers grab chunks of rows from a shared counter.  Which
 * thread computes a row never changes what is computed for it. */
typedef void (*row_fn)(long row, void* ctx);
typedef struct {
    row_fn fn;
    void* ctx;
    long rows, chunk;
    atomic_long next;
} row_job;

static void* row_worker(void* arg) {
    row_job* job = (row_job*)arg;
    for (;;) {
        const long from = atomic_fetch_add(&job->next, job->chunk);
        if (from >= job->rows) break;
        const long to = from + job->chunk < job->rows ? from + job->chunk : job->rows;
        for (long r = from; r < to; ++r) job->fn(r, job->ctx);
    }
    return NULL;
}

static void parallel_rows(long rows, int threads, row_fn fn, void* ctx) {
    int nt = threads > 0 ? threads : (int)sysconf(_SC_NPROCESSORS_ONLN);
    if (nt < 1) nt = 1;
    if (nt > 256) nt = 256;
    if ((long)nt > rows) nt = rows > 0 ? (int)rows : 1;
    row_job job;
    job.fn = fn;
    job.ctx = ctx;
    job.rows = rows;
    job.chunk = rows / (8L * nt) > 0 ? rows / (8L * nt) : 1;
    atomic_init(&job.next, 0);
    if (nt == 1) {
        row_worker(&job);
        return;
    }
    pthread_t tid[256];
    int started = 0;
    for (int t = 0; t < nt - 1; ++t) {
        if (pthread_create(&tid[started], NULL, row_worker, &job) == 0) ++started;
    }
    row_worker(&job);
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}

typedef struct {
    const float* a;
    const float* b;
    float* c;
    size_t M, K, N, a_stride, b_stride;
} mm_ctx;

/* One output row: src/tensor_ops.cpp:545-560 */
static void mm_row(long row, void* vctx) {
    const mm_ctx* x = (const mm_ctx*)vctx;
    const size_t bi = (size_t)row / x->M;
    const size_t i = (size_t)row % x->M;
    const float* restrict a_row = x->a + bi * x->a_stride + i * x->K;
    const float* restrict bm = x->b + bi * x->b_stride;
    float* restrict c_row = x->c + bi * x->M * x->N + i * x->N;
    const size_t K = x->K, N = x->N;
    for (size_t k = 0; k < K; ++k) {
        const float a_ik = a_row[k];
        if (a_ik == 0.0f) continue; /* the zero-skip, :555 */
        const float* restrict b_row = bm + k * N;
        for (size_t j = 0; j < N; ++j) c_row[j] += a_ik * b_row[j];
    }
}

/* src/tensor_ops.cpp:543-562 */
void oracle_matmul_f32(const float* a, const float* b, float* c, size_t batch, size_t M, size_t K,
                       size_t N, int a_batched, int b_batched, int threads) {
    const size_t a_stride = a_batched ? M * K : 0; /* src/tensor_ops.cpp:514-515 */
    const size_t b_stride = b_batched ? K * N : 0;
    memset(c, 0, sizeof(float) * batch * M * N); /* Tensor C(out_shape, 0.0f): :511 */
    mm_ctx ctx = {a, b, c, M, K, N, a_stride, b_stride};
    parallel_rows((long)(batch * M), threads, mm_row, &ctx);
}

/* src/tensor_ops.cpp:335-370 (values only; the blocking of the reference's loop does not
 * change what is written where) */
void oracle_transpose_f32(const float* src, float* dst, size_t batch, size_t rows, size_t cols) {
    for (size_t b = 0; b < batch; ++b) {
        const float* s = src + b * rows * cols;
        float* d = dst + b * rows * cols;
        for (size_t i = 0; i < rows; ++i)
            for (size_t j = 0; j < cols; ++j) d[j * rows + i] = s[i * cols + j];
    }
}

void oracle_matmul_nt_f32(const float* a, const float* b, float* c, size_t batch, size_t M,
                          size_t K, size_t N, int a_batched, int b_batched, int threads) {
    const size_t nb = b_batched ? batch : 1;
    float* bt = (float*)malloc(sizeof(float) * nb * K * N);
    oracle_transpose_f32(b, bt, nb, N, K); /* (N,K) -> (K,N) */
    oracle_matmul_f32(a, bt, c, batch, M, K, N, a_batched, b_batched, threads);
    free(bt);
}

void oracle_matmul_tn_f32(const float* a, const float* b, float* c, size_t batch, size_t M,
                          size_t K, size_t N, int a_batched, int b_batched, int threads) {
    const size_t na = a_batched ? batch : 1;
    float* at = (float*)malloc(sizeof(float) * na * K * M);
    oracle_transpose_f32(a, at, na, K, M); /* (K,M) -> (M,K) */
    oracle_matmul_f32(at, b, c, batch, M, K, N, a_batched, b_batched, threads);
    free(at);
}

/* fold_leading, src/tensor_detail.hpp:182-206: zero, then add block r = 0, 1, ... */
static void fold_leading(const float* full, float* folded, size_t repeat, size_t inner) {
    memset(folded, 0, sizeof(float) * inner);
    for (size_t r = 0; r < repeat; ++r)
        for (size_t j = 0; j < inner; ++j) folded[j] += full[r * inner + j];
}

/* add_grad's first write, src/tensor.cpp:168-203: the gradient buffer starts at zero and
 * the incoming value is added to it. */
static void first_grad(const float* g, float* grad, size_t n) {
    for (size_t i = 0; i < n; ++i) grad[i] = 0.0f + g[i];
}

/* src/tensor_ops.cpp:570-585 */
void oracle_matmul_backward_f32(const float* a, const float* b, const float* grad_c, float* grad_a,
                                float* grad_b, size_t batch, size_t M, size_t K, size_t N,
                                int a_batched, int b_batched, int threads) {
    /* dA = grad_out.matmul(B.transpose()) : (batch, M, N) x (batch?, N, K) */
    {
        const int g_batched = (a_batched || b_batched) ? 1 : 0;
        float* dA = (float*)malloc(sizeof(float) * batch * M * K);
        /* B stored (K,N); B.transpose() is (N,K) stored row-major; the product then reads it as
         * its K x N operand with inner dimension N. */
        const size_t nb = b_batched ? batch : 1;
        float* bt = (float*)malloc(sizeof(float) * nb * K * N);
        oracle_transpose_f32(b, bt, nb, K, N);
        oracle_matmul_f32(grad_c, bt, dA, batch, M, N, K, g_batched, b_batched, threads);
        if (a_batched || batch == 1) {
            first_grad(dA, grad_a, batch * M * K);
        } else {
            float* folded = (float*)malloc(sizeof(float) * M * K);
            fold_leading(dA, folded, batch, M * K);
            first_grad(folded, grad_a, M * K);
            free(folded);
        }
        free(bt);
        free(dA);
    }
    /* dB = A.transpose().matmul(grad_out) : (batch?, K, M) x (batch, M, N) */
    {
        const int g_batched = (a_batched || b_batched) ? 1 : 0;
        float* dB = (float*)malloc(sizeof(float) * batch * K * N);
        const size_t na = a_batched ? batch : 1;
        float* at = (float*)malloc(sizeof(float) * na * M * K);
        oracle_transpose_f32(a, at, na, M, K);
        oracle_matmul_f32(at, grad_c, dB, batch, K, M, N, a_batched, g_batched, threads);
        if (b_batched || batch == 1) {
            first_grad(dB, grad_b, batch * K * N);
        } else {
            float* folded = (float*)malloc(sizeof(float) * K * N);
            fold_leading(dB, folded, batch, K * N);
            first_grad(folded, grad_b, K * N);
            free(folded);
        }
        free(at);
        free(dB);
    }
}

typedef struct {
    const float* a;
    const float* b;
    double* c;
    size_t K, N, lda, ldb;
    int trans_a, trans_b;
} f64_ctx;

static void f64_row(long row, void* vctx) {
    const f64_ctx* x = (const f64_ctx*)vctx;
    const size_t i = (size_t)row, K = x->K, N = x->N;
    double* c_row = x->c + i * N;
    for (size_t j = 0; j < N; ++j) c_row[j] = 0.0;
    for (size_t k = 0; k < K; ++k) {
        const double a_ik = x->trans_a ? (double)x->a[k * x->lda + i] : (double)x->a[i * x->lda + k];
        if (!x->trans_b) {
            const float* b_row = x->b + k * x->ldb;
            for (size_t j = 0; j < N; ++j) c_row[j] += a_ik * (double)b_row[j];
        } else {
            for (size_t j = 0; j < N; ++j) c_row[j] += a_ik * (double)x->b[j * x->ldb + k];
        }
    }
}

void oracle_matmul_f64(const float* a, const float* b, double* c, size_t M, size_t K, size_t N,
                       int trans_a, int trans_b, size_t lda, size_t ldb, int threads) {
    f64_ctx ctx = {a, b, c, K, N, lda, ldb, trans_a, trans_b};
    parallel_rows((long)M, threads, f64_row, &ctx);
}

/* ------------------------------------------------------------------------------------------
 * Random streams.  std::mt19937 is the standard 32-bit Mersenne twister (the C++ standard
 * fixes its output); the two distributions follow libstdc++'s published algorithms:
 *   generate_canonical<float, 24>: one 32-bit draw, converted to float, divided by 2^32;
 *     a result that rounds up to 1 is replaced by the largest float below 1;
 *   uniform_real_distribution<float>(lo, hi): canonical * (hi - lo) + lo;
 *   normal_distribution<float>: Marsaglia's polar method, producing values in pairs and
 *     keeping the second of each pair for the next call; Tensor::randn builds a fresh
 *     distribution per tensor, so a kept value never crosses tensors.
 * ------------------------------------------------------------------------------------------ */
void oracle_seed(oracle_rng* g, uint64_t seed) {
    g->mt[0] = (uint32_t)seed; /* static_cast<std::mt19937::result_type>(seed), src/tensor.cpp:30 */
    for (int i = 1; i < 624; ++i)
        g->mt[i] = 1812433253u * (g->mt[i - 1] ^ (g->mt[i - 1] >> 30)) + (uint32_t)i;
    g->idx = 624;
}

static uint32_t mt_next(oracle_rng* g) {
    if (g->idx >= 624) {
        for (int i = 0; i < 624; ++i) {
            const uint32_t y = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % 624] & 0x7fffffffu);
            g->mt[i] = g->mt[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
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

static float canonical(oracle_rng* g) {
    const float sum = (float)mt_next(g);
    float ret = sum / 4294967296.0f;
    if (ret >= 1.0f) ret = nextafterf(1.0f, 0.0f);
    return ret;
}

void oracle_rand(oracle_rng* g, float* out, size_t n, float lo, float hi) {
    const float span = hi - lo;
    for (size_t i = 0; i < n; ++i) out[i] = canonical(g) * span + lo;
}

void oracle_randn(oracle_rng* g, float* out, size_t n, float mean, float stddev) {
    int saved_available = 0;
    float saved = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float ret;
        if (saved_available) {
            saved_available = 0;
            ret = saved;
        } else {
            float x, y, r2;
            do {
                x = (float)((double)(2.0f * canonical(g)) - 1.0);
                y = (float)((double)(2.0f * canonical(g)) - 1.0);
                r2 = x * x + y * y;
            } while (r2 > 1.0f || r2 == 0.0f);
            const float mult = sqrtf(-2.0f * logf(r2) / r2);
            saved = x * mult;
            saved_available = 1;
            ret = y * mult;
        }
        out[i] = ret * stddev + mean;
    }
}

/* Tensor::softmax over the last axis (src/tensor_ops.cpp:621-647): row maximum, expf of the
 * difference, fp32 sum in ascending column order, division. */
void oracle_softmax_rows_f32(const float* x, float* y, size_t rows, size_t cols) {
    for (size_t i = 0; i < rows; ++i) {
        const float* row = x + i * cols;
        float* out = y + i * cols;
        float max_v = row[0];
        for (size_t j = 1; j < cols; ++j)
            if (max_v < row[j]) max_v = row[j];
        float denom = 0.0f;
        for (size_t j = 0; j < cols; ++j) {
            const float e = expf(row[j] - max_v);
            out[j] = e;
            denom += e;
        }
        for (size_t j = 0; j < cols; ++j) out[j] /= denom;
    }
}

/* Its backward (src/tensor_ops.cpp:649-668): dX_ij = y_ij * (g_ij - sum_k g_ik * y_ik), the dot
 * in fp32, ascending k, product rounded before it is added. */
void oracle_softmax_backward_f32(const float* y, const float* g, float* dx, size_t rows, size_t cols) {
    for (size_t i = 0; i < rows; ++i) {
        const float* yr = y + i * cols;
        const float* gr = g + i * cols;
        float dot = 0.0f;
        for (size_t j = 0; j < cols; ++j) dot += gr[j] * yr[j];
        for (size_t j = 0; j < cols; ++j) dx[i * cols + j] = yr[j] * (gr[j] - dot);
    }
}
