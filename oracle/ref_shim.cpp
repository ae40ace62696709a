// TEST INFRASTRUCTURE — not part of the product path.
//
// A thin extern "C" face over the UNMODIFIED reference engine (cpp-ai-engine,
// CPU build, no ENGINE_CUDA), so that Python tests and the benchmark's CPU arm
// can drive the reference's own code: its global RNG (src/tensor.cpp:24-31,
// 117-135), its Tensor::matmul with the CPU i-k-j loop (src/tensor_ops.cpp:475-588)
// and the autograd backward of that node (src/tensor_ops.cpp:570-585,
// src/autograd.cpp:104-156).
//
// This file contains no reference source; it only includes the reference's
// public headers and is linked against objects compiled from the reference
// tree where it lies (see the Makefile beside this file).  Outputs go to
// oracle/_ref/ and stay out of version control.
#include "engine/autograd.hpp"
#include "engine/conv.hpp"
#include "engine/nn.hpp"
#include "engine/parallel.hpp"
#include "engine/tensor.hpp"
#include "engine/transformer.hpp"

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <exception>
#include <vector>

using engine::Tensor;

namespace {

thread_local char g_error[512] = {0};

void set_error(const char* what) {
    std::strncpy(g_error, what, sizeof(g_error) - 1);
    g_error[sizeof(g_error) - 1] = 0;
}

std::vector<size_t> mat_shape(size_t batch, int batched, size_t rows, size_t cols) {
    if (batched) return {batch, rows, cols};
    return {rows, cols};
}

Tensor from_buffer(const float* src, const std::vector<size_t>& shape, bool requires_grad) {
    Tensor t(shape, 0.0f, requires_grad);
    std::copy_n(src, t.size(), t.data());
    return t;
}

}  // namespace

extern "C" {

const char* ref_last_error(void) { return g_error; }

int ref_num_threads(void) { return static_cast<int>(engine::parallel::num_threads()); }
void ref_set_num_threads(int n) { engine::parallel::set_num_threads(static_cast<size_t>(n)); }

void ref_manual_seed(uint64_t seed) { engine::manual_seed(seed); }

// Tensor::rand({n}, lo, hi) / Tensor::randn({n}, mean, stddev) from the engine's global generator.
void ref_rand(float* out, size_t n, float lo, float hi) {
    Tensor t = Tensor::rand({n}, lo, hi);
    std::copy_n(t.data(), n, out);
}
void ref_randn(float* out, size_t n, float mean, float stddev) {
    Tensor t = Tensor::randn({n}, mean, stddev);
    std::copy_n(t.data(), n, out);
}

// C = A.matmul(B).  A is (batch, M, K) when a_batched else (M, K); B likewise (K, N).
// Returns 0, or 1 with ref_last_error() set when the engine throws.
int ref_matmul(const float* a, const float* b, float* c, size_t batch, size_t M, size_t K,
               size_t N, int a_batched, int b_batched) {
    try {
        Tensor A = from_buffer(a, mat_shape(batch, a_batched, M, K), false);
        Tensor B = from_buffer(b, mat_shape(batch, b_batched, K, N), false);
        Tensor C = A.matmul(B);
        std::copy_n(C.data(), C.size(), c);
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}

// Same product, timed: only A.matmul(B) sits between the two clock reads (operands are
// built before, the result is not copied out).  Returns seconds of the best of `repeats`.
double ref_matmul_time(const float* a, const float* b, size_t batch, size_t M, size_t K, size_t N,
                       int a_batched, int b_batched, int repeats) {
    try {
        Tensor A = from_buffer(a, mat_shape(batch, a_batched, M, K), false);
        Tensor B = from_buffer(b, mat_shape(batch, b_batched, K, N), false);
        double best = 1e300;
        for (int r = 0; r < repeats; ++r) {
            auto t0 = std::chrono::steady_clock::now();
            Tensor C = A.matmul(B);
            auto t1 = std::chrono::steady_clock::now();
            volatile float sink = C.data()[0];
            (void)sink;
            best = std::min(best, std::chrono::duration<double>(t1 - t0).count());
        }
        return best;
    } catch (const std::exception& e) {
        set_error(e.what());
        return -1.0;
    }
}

// Forward and backward through the engine's autograd with an explicit grad_output.
// grad_a / grad_b have the shapes of a / b (a shared operand's gradient is folded
// over the batch by the engine itself).
int ref_matmul_backward(const float* a, const float* b, const float* grad_out, float* out,
                        float* grad_a, float* grad_b, size_t batch, size_t M, size_t K, size_t N,
                        int a_batched, int b_batched) {
    try {
        Tensor A = from_buffer(a, mat_shape(batch, a_batched, M, K), true);
        Tensor B = from_buffer(b, mat_shape(batch, b_batched, K, N), true);
        Tensor C = A.matmul(B);
        Tensor G = from_buffer(grad_out, C.shape(), false);
        C.backward(G);
        if (out) std::copy_n(C.data(), C.size(), out);
        Tensor gA = A.grad();
        Tensor gB = B.grad();
        std::copy_n(gA.data(), gA.size(), grad_a);
        std::copy_n(gB.data(), gB.size(), grad_b);
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}

// The two transposed forms exactly as the reference writes them:
//   NT: A.matmul(B.transpose())     with B stored (batch?, N, K)
//   TN: A.transpose().matmul(B)     with A stored (batch?, K, M)
int ref_matmul_nt(const float* a, const float* b, float* c, size_t batch, size_t M, size_t K,
                  size_t N, int a_batched, int b_batched) {
    try {
        Tensor A = from_buffer(a, mat_shape(batch, a_batched, M, K), false);
        Tensor B = from_buffer(b, mat_shape(batch, b_batched, N, K), false);
        Tensor C = A.matmul(B.transpose());
        std::copy_n(C.data(), C.size(), c);
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}
int ref_matmul_tn(const float* a, const float* b, float* c, size_t batch, size_t M, size_t K,
                  size_t N, int a_batched, int b_batched) {
    try {
        Tensor A = from_buffer(a, mat_shape(batch, a_batched, K, M), false);
        Tensor B = from_buffer(b, mat_shape(batch, b_batched, K, N), false);
        Tensor C = A.transpose().matmul(B);
        std::copy_n(C.data(), C.size(), c);
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}

// im2col as the reference's Conv2d builds its GEMM operand: (N*oH*oW, C*kH*kW).
int ref_im2col(const float* x, float* cols, size_t n, size_t c, size_t h, size_t w, size_t kh,
               size_t kw, size_t stride, size_t pad) {
    try {
        Tensor X = from_buffer(x, {n, c, h, w}, false);
        engine::nn::Window2d win(kh, kw, stride, pad);
        Tensor Cm = engine::nn::im2col(X, win);
        std::copy_n(Cm.data(), Cm.size(), cols);
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}

// Conv2d forward and backward through the engine's own layer and autograd
// (src/conv.cpp:280-338): y and the three gradients for an explicit grad_output.
int ref_conv2d_backward(const float* x, const float* weight, const float* bias, const float* grad_out,
                        float* y, float* grad_x, float* grad_w, float* grad_b, size_t n, size_t c, size_t h,
                        size_t w, size_t out_c, size_t kh, size_t kw, size_t stride, size_t pad) {
    try {
        engine::nn::Conv2d conv(c, out_c, engine::nn::Window2d(kh, kw, stride, pad), bias != nullptr);
        std::copy_n(weight, conv.weight().size(), conv.weight().data());
        conv.weight().set_requires_grad(true);
        conv.weight().zero_grad();
        if (bias != nullptr) {
            std::copy_n(bias, out_c, conv.bias().data());
            conv.bias().set_requires_grad(true);
            conv.bias().zero_grad();
        }
        Tensor X = from_buffer(x, {n, c, h, w}, true);
        Tensor Y = conv(X);
        Tensor G = from_buffer(grad_out, Y.shape(), false);
        Y.backward(G);
        if (y) std::copy_n(Y.data(), Y.size(), y);
        Tensor gx = X.grad();
        Tensor gw = conv.weight().grad();
        if (grad_x) std::copy_n(gx.data(), gx.size(), grad_x);
        if (grad_w) std::copy_n(gw.data(), gw.size(), grad_w);
        if (grad_b && bias != nullptr) {
            Tensor gb = conv.bias().grad();
            std::copy_n(gb.data(), gb.size(), grad_b);
        }
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}

// scaled_dot_product_attention forward and backward through the engine's own autograd
// (src/transformer.cpp:279-304): output, attention weights and the gradients of q, k, v for an
// explicit grad_output.  lead = number of (batch, head) matrices; mask may be null.
int ref_attention_backward(const float* q, const float* k, const float* v, const float* mask,
                           const float* grad_out, float* out, float* weights, float* grad_q, float* grad_k,
                           float* grad_v, size_t lead, size_t s_q, size_t s_k, size_t d_k, size_t d_v) {
    try {
        Tensor Q = from_buffer(q, {lead, s_q, d_k}, true);
        Tensor K = from_buffer(k, {lead, s_k, d_k}, true);
        Tensor V = from_buffer(v, {lead, s_k, d_v}, true);
        Tensor M;
        if (mask != nullptr) M = from_buffer(mask, {s_q, s_k}, false);
        Tensor W;
        Tensor O = engine::nn::scaled_dot_product_attention(Q, K, V, mask != nullptr ? &M : nullptr, &W);
        Tensor G = from_buffer(grad_out, O.shape(), false);
        O.backward(G);
        if (out) std::copy_n(O.data(), O.size(), out);
        if (weights) std::copy_n(W.data(), W.size(), weights);
        Tensor gq = Q.grad(), gk = K.grad(), gv = V.grad();
        std::copy_n(gq.data(), gq.size(), grad_q);
        std::copy_n(gk.data(), gk.size(), grad_k);
        std::copy_n(gv.data(), gv.size(), grad_v);
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return 1;
    }
}

}  // extern "C"
