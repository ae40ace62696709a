// Tests of the C++17 host side (cpp-ai-engine_b200/host) on a B200, written to read like
// the reference's own tests of its matrix product:
//   known answers, shapes and throws          tests/test_tensor.cpp:47-65, 182-202
//   PyTorch golden vectors with gradients     tests/test_reference.cpp:99-114 (abs tol 1e-4)
//   numerical gradients                       tests/test_tensor.cpp:245-258, tests/test_support.hpp:78-121
//   CPU/GPU parity shape list, "a kernel must have run", residency / transfer counts
//                                             tests/test_cuda_parity.cpp:62-137, 192-247, 790-818
//   layers: Conv2d with gradients, attention, MultiHeadAttention
//                                             tests/test_reference.cpp:216-251, 296-349 (abs tol 1e-4)
// The CPU side of the parity checks is the oracle library (test infrastructure).
#include "engine_b200.hpp"

#include "../../oracle/matmul_oracle.h"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <functional>
#include <iostream>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

using engine::Tensor;

namespace {

int g_checks = 0;
int g_failures = 0;

void section(const std::string& name) { std::cout << "\n== " << name << " ==\n"; }

void check(bool ok, const std::string& what) {
    ++g_checks;
    if (!ok) ++g_failures;
    std::cout << (ok ? "  [ ok ] " : "  [FAIL] ") << what << "\n";
}

void check_close(float got, float want, const std::string& what, float tol = 1e-5f) {
    check(std::fabs(got - want) <= tol, what + " (got " + std::to_string(got) + ")");
}

template <class F>
void check_throws(F&& f, const std::string& what) {
    bool threw = false;
    try {
        f();
    } catch (const std::invalid_argument&) {
        threw = true;
    }
    check(threw, what);
}

// max |got - want| / max(1, |want|): the reference's parity metric (tests/test_cuda_parity.cpp:100-102)
double scaled_error(const std::vector<float>& got, const std::vector<float>& want) {
    if (got.size() != want.size()) return 1e30;
    double worst = 0.0;
    for (size_t i = 0; i < got.size(); ++i) {
        const double w = want[i];
        worst = std::max(worst, std::fabs(got[i] - w) / std::max(1.0, std::fabs(w)));
    }
    return worst;
}

double tolerance(size_t K) { return std::max(1e-5, 2.0 * static_cast<double>(K) / 16777216.0); }

size_t count(const std::vector<size_t>& s) {
    size_t n = 1;
    for (size_t d : s) n *= d;
    return n;
}

std::vector<float> oracle_matmul(const Tensor& a, const Tensor& b) {
    const auto& sa = a.shape();
    const auto& sb = b.shape();
    const bool ab = sa.size() > 2, bb = sb.size() > 2;
    const std::vector<size_t> dims = ab ? std::vector<size_t>(sa.begin(), sa.end() - 2)
                                        : std::vector<size_t>(sb.begin(), sb.end() - 2);
    const size_t batch = count(dims);
    const size_t M = sa[sa.size() - 2], K = sa[sa.size() - 1], N = sb[sb.size() - 1];
    std::vector<float> va = a.to_vector(), vb = b.to_vector(), c(batch * M * N);
    oracle_matmul_f32(va.data(), vb.data(), c.data(), batch, M, K, N, ab, bb, 0);
    return c;
}

void test_matmul_known_answers() {
    section("Tensor: matrix multiplication");
    Tensor M1({2, 3}, {1, 2, 3, 4, 5, 6});
    Tensor M2({3, 2}, {7, 8, 9, 1, 2, 3});
    const size_t before = engine::cuda::kernels_launched();
    Tensor R = M1.matmul(M2);
    check(engine::cuda::kernels_launched() > before, "a device kernel was launched");
    check(R.shape() == std::vector<size_t>({2, 2}), "(2,3) x (3,2) gives (2,2)");
    check_close(R(0, 0), 31.0f, "R[0,0] == 31");
    check_close(R(0, 1), 19.0f, "R[0,1] == 19");
    check_close(R(1, 0), 85.0f, "R[1,0] == 85");
    check_close(R(1, 1), 55.0f, "R[1,1] == 55");
    check_throws([&] { (void)M1.matmul(M1); }, "incompatible inner dimensions throw");
    Tensor T = M1.transpose();
    check(T.shape() == std::vector<size_t>({3, 2}), "transpose flips the shape");
    check_close(T(2, 1), 6.0f, "transpose swaps the indices");
    check(T.is_transposed_view(), "transpose is a view: no data moved");

    Tensor A({2, 2, 3}, {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12});
    Tensor B({2, 3, 2}, {1, 0, 0, 1, 1, 1, 2, 0, 0, 2, 1, 1});
    Tensor C = A.matmul(B);
    check(C.shape() == std::vector<size_t>({2, 2, 2}), "batched matmul gives (B, M, N)");
    check_close(C.at(0), 4.0f, "batch 0: 1*1 + 2*0 + 3*1 == 4");
    check_close(C.at(1), 5.0f, "batch 0: 1*0 + 2*1 + 3*1 == 5");
    check_close(C.at(4), 23.0f, "batch 1: 7*2 + 8*0 + 9*1 == 23");
    Tensor shared({3, 2}, {1, 0, 0, 1, 1, 1});
    Tensor Cs = A.matmul(shared);
    check(Cs.shape() == std::vector<size_t>({2, 2, 2}), "matmul with a shared 2D matrix gives (B, M, N)");
    check_close(Cs.at(0), 4.0f, "the shared matrix applies to the first batch");
    check_close(Cs.at(4), 16.0f, "and the same matrix to the second (7 + 9)");
    check_throws([&] { (void)Tensor({2, 2, 3}, 1.0f).matmul(Tensor({3, 3, 2}, 1.0f)); },
                 "matmul with mismatched batches throws");
    check_throws([&] { (void)Tensor({4}, 1.0f).matmul(Tensor({4}, 1.0f)); }, "matmul of 1D vectors throws");
}

void test_golden_vectors(const std::string& golden_dir) {
    section("PyTorch: matrix multiplication (golden vectors)");
    std::map<std::string, Tensor> f;
    for (auto& kv : engine::load_tensors(golden_dir + "/pytorch_matmul.bin")) f.emplace(kv.first, kv.second);
    auto largest_dev = [](const Tensor& got, const Tensor& want) {
        std::vector<float> g = got.to_vector(), w = want.to_vector();
        float m = got.shape() == want.shape() ? 0.0f : 1e30f;
        for (size_t i = 0; i < g.size() && i < w.size(); ++i) m = std::max(m, std::fabs(g[i] - w[i]));
        return m;
    };
    for (const std::string name : {"matmul", "matmul_batched", "matmul_shared"}) {
        Tensor a = f.at(name + "/a").detach();
        Tensor b = f.at(name + "/b").detach();
        a.set_requires_grad(true);
        b.set_requires_grad(true);
        Tensor out = a.matmul(b);
        check(largest_dev(out, f.at(name + "/output")) <= 1e-4f, name + ": output");
        out.backward(f.at(name + "/grad_output"));
        check(largest_dev(a.grad(), f.at(name + "/grad.a")) <= 1e-4f, name + ": gradient of A");
        check(largest_dev(b.grad(), f.at(name + "/grad.b")) <= 1e-4f, name + ": gradient of B");
    }
}

// Central differences of loss = sum(w * f(x)) against the analytical gradient (h = 1e-3, tol 2e-2).
void check_gradient(const std::function<Tensor(const Tensor&)>& f, const Tensor& x0, const std::string& what) {
    Tensor x = x0.detach();
    x.set_requires_grad(true);
    Tensor y = f(x);
    engine::manual_seed(123);
    Tensor w = Tensor::rand(y.shape(), -1.0f, 1.0f);
    y.backward(w);
    std::vector<float> analytic = x.grad().to_vector();
    std::vector<float> wv = w.to_vector(), base = x0.to_vector();
    auto loss = [&](const std::vector<float>& v) {
        Tensor yy = f(Tensor(x0.shape(), v));
        std::vector<float> out = yy.to_vector();
        double s = 0.0;
        for (size_t i = 0; i < out.size(); ++i) s += static_cast<double>(wv[i]) * out[i];
        return s;
    };
    const float h = 1e-3f;
    double worst = 0.0;
    for (size_t i = 0; i < base.size(); i += std::max<size_t>(1, base.size() / 12)) {
        std::vector<float> p = base, m = base;
        p[i] += h;
        m[i] -= h;
        const double numeric = (loss(p) - loss(m)) / (2.0 * h);
        worst = std::max(worst, std::fabs(numeric - analytic[i]) / std::max(1.0, std::fabs(numeric)));
    }
    check(worst <= 2e-2, what + " (largest deviation " + std::to_string(worst) + ")");
}

void test_numerical_gradients() {
    section("Autograd: numerical gradients of matmul");
    engine::manual_seed(5);
    Tensor A = Tensor::randn({2, 3, 4});
    Tensor B = Tensor::randn({2, 4, 5});
    Tensor S = Tensor::randn({4, 2});
    check_gradient([&](const Tensor& x) { return x.matmul(B); }, A, "batched matmul, gradient of A");
    check_gradient([&](const Tensor& x) { return A.matmul(x); }, B, "batched matmul, gradient of B");
    check_gradient([&](const Tensor& x) { return A.matmul(x); }, S, "gradient of a matrix shared by the batch");
    check_gradient([&](const Tensor& x) { return x.matmul(S); }, A, "batched operand against a shared matrix");
    Tensor Q = Tensor::randn({3, 5, 4});
    Tensor Kt = Tensor::randn({3, 6, 4});
    check_gradient([&](const Tensor& x) { return Q.matmul(x.transpose()); }, Kt,
                   "Q x K^T through a transposed view, gradient of K");
    check_gradient([&](const Tensor& x) { return x.transpose().matmul(Q); }, Tensor::randn({3, 5, 2}),
                   "A^T x B through a transposed view, gradient of A");
}

void test_parity_shapes() {
    section("CPU/GPU parity (reference shape list)");
    struct Case {
        std::vector<size_t> a, b;
    };
    const std::vector<Case> cases = {
        {{1, 1}, {1, 1}},         {{17, 23}, {23, 31}},           {{32, 32}, {32, 32}},
        {{33, 129}, {129, 65}},   {{127, 129}, {129, 128}},       {{128, 128}, {128, 128}},
        {{129, 257}, {257, 256}}, {{256, 256}, {256, 260}},       {{4, 3, 17, 23}, {4, 3, 23, 11}},
        {{8, 12, 40}, {40, 20}},  {{131, 135}, {135, 133}},       {{9, 6272}, {6272, 16}},
        {{144, 1568}, {1568, 32}}, {{7, 5000}, {5000, 5}},        {{2048, 96}, {96, 121}},
    };
    engine::manual_seed(42);
    for (const Case& c : cases) {
        Tensor a = Tensor::randn(c.a), b = Tensor::randn(c.b);
        const size_t before = engine::cuda::kernels_launched();
        Tensor got = a.matmul(b);
        const bool launched = engine::cuda::kernels_launched() > before;
        const double err = scaled_error(got.to_vector(), oracle_matmul(a, b));
        check(launched && err <= tolerance(c.a.back()),
              "matmul " + a.shape_str() + " x " + b.shape_str() + " (error " + std::to_string(err) + ")");
    }
    // transposed views against materialised transposes
    Tensor a = Tensor::randn({130, 45}), bt = Tensor::randn({121, 45});
    Tensor got = a.matmul(bt.transpose());
    Tensor b_mat({45, 121}, bt.transpose().to_vector());
    check(scaled_error(got.to_vector(), oracle_matmul(a, b_mat)) <= 1e-5, "A x B^T with B^T as a view");
    Tensor at = Tensor::randn({45, 130});
    Tensor got2 = at.transpose().matmul(b_mat);
    Tensor a_mat({130, 45}, at.transpose().to_vector());
    check(scaled_error(got2.to_vector(), oracle_matmul(a_mat, b_mat)) <= 1e-5, "A^T x B with A^T as a view");
    // exact on small integers
    std::vector<float> ia(131 * 135), ib(135 * 133);
    for (size_t i = 0; i < ia.size(); ++i) ia[i] = static_cast<float>(static_cast<int>(i * 7 % 9) - 4);
    for (size_t i = 0; i < ib.size(); ++i) ib[i] = static_cast<float>(static_cast<int>(i * 5 % 7) - 3);
    Tensor A({131, 135}, ia), B({135, 133}, ib);
    check(A.matmul(B).to_vector() == oracle_matmul(A, B), "integer inputs give the exact product");
}

void test_residency_and_seam() {
    section("Residency: results stay on the device, operands are uploaded once");
    engine::manual_seed(9);
    Tensor x = Tensor::randn({64, 96}), w1 = Tensor::randn({96, 96}), w2 = Tensor::randn({96, 32});
    engine::cuda::reset_transfer_stats();
    Tensor h = x.matmul(w1);
    Tensor y = h.matmul(w2);
    Tensor y2 = h.matmul(w2);
    auto st = engine::cuda::transfer_stats();
    check(st.to_device_count == 3, "three operands, three uploads (" + std::to_string(st.to_device_count) + ")");
    check(st.to_host_count == 0, "nothing came back to the host");
    check(h.resident_on_device() && y.resident_on_device(), "intermediate and result live on the device");
    std::vector<float> v = y.to_vector();
    st = engine::cuda::transfer_stats();
    check(st.to_host_count == 1 && st.to_host_bytes == 64 * 32 * sizeof(float), "reading the result downloads it once");
    check(v == y2.to_vector(), "the same product twice gives the same bits");

    // the seam itself, with beta onto a non-zero destination (tests/test_cuda_parity.cpp:263-290)
    engine::Storage a(std::vector<float>(65 * 70, 0.5f)), b(std::vector<float>(70 * 36, 0.25f));
    engine::Storage out(std::vector<float>(65 * 36, 3.0f));
    check(engine::cuda::ops::matmul(a, b, out, 1, 65, 70, 36, false, false, 1.0f), "ops::matmul reports the device did it");
    check_close(out.host()[100], 3.0f + 70 * 0.125f, "out = a x b + 1 * out", 1e-4f);
    bool threw = false;
    try {
        engine::Storage wrong(10, 0.0f);
        engine::cuda::ops::matmul(a, b, wrong, 1, 65, 70, 36, false, false);
    } catch (const std::runtime_error&) {
        threw = true;
    }
    check(threw, "a mis-sized output is an error, not a silent CPU fallback");
}

void test_reduced_precision_is_opt_in() {
    section("TF32 is opt-in and less precise (tests/test_cuda_parity.cpp:392-419, 480-505)");
    engine::manual_seed(17);
    Tensor a = Tensor::randn({256, 256}), b = Tensor::randn({256, 256});
    std::vector<float> va = a.to_vector(), vb = b.to_vector();
    std::vector<double> ref(256 * 256);
    oracle_matmul_f64(va.data(), vb.data(), ref.data(), 256, 256, 256, 0, 0, 256, 256, 0);
    auto err = [&](const std::vector<float>& got) {
        double worst = 0;
        for (size_t i = 0; i < got.size(); ++i)
            worst = std::max(worst, std::fabs(got[i] - ref[i]) / std::max(1.0, std::fabs(ref[i])));
        return worst;
    };
    check(engine::cuda::matmul_kernel() == engine::cuda::MatmulKernel::Auto, "the default is the fp32-accurate kernel");
    const double e3 = err(a.matmul(b).to_vector());
    engine::cuda::set_matmul_kernel(engine::cuda::MatmulKernel::TensorCore);
    const double e1 = err(a.matmul(b).to_vector());
    engine::cuda::set_matmul_kernel(engine::cuda::MatmulKernel::Auto);
    check(e3 <= 1e-5, "default error " + std::to_string(e3) + " <= 1e-5");
    check(e1 <= 4.0 * std::sqrt(256.0) / 2048.0, "tf32 error " + std::to_string(e1) + " within 4*sqrt(K)*2^-11");
    check(e1 > 10.0 * e3, "tf32 is more than 10x less precise");
}


double max_abs_diff(const std::vector<float>& got, const std::vector<float>& want) {
    if (got.size() != want.size()) return 1e30;
    double worst = 0.0;
    for (size_t i = 0; i < got.size(); ++i) worst = std::max(worst, std::fabs(double(got[i]) - double(want[i])));
    return worst;
}

// The layer bodies as single kernels, against the reference's PyTorch vectors
// (tests/test_reference.cpp:216-251 Conv2d with gradients, :296-349 attention and
// MultiHeadAttention; abs tol 1e-4 as there) and against the oracle product for Linear.
void test_layers(const std::string& golden_dir) {
    section("Layers as single kernels (golden vectors)");
    std::map<std::string, Tensor> f;
    for (auto& kv : engine::load_tensors(golden_dir + "/pytorch_layers.bin")) f.emplace(kv.first, kv.second);
    namespace nn = engine::nn;

    struct ConvCase {
        std::string name;
        size_t stride, pad;
    };
    for (const ConvCase& cc : {ConvCase{"conv2d_pad1", 1, 1}, ConvCase{"conv2d_stride2", 2, 0}}) {
        Tensor x = f.at(cc.name + "/input").detach();
        Tensor w = f.at(cc.name + "/weight").detach();
        Tensor b = f.at(cc.name + "/bias").detach();
        x.set_requires_grad(true);
        w.set_requires_grad(true);
        b.set_requires_grad(true);
        const size_t before = engine::cuda::kernels_launched();
        Tensor y = nn::conv2d(x, w, &b, nn::Window2d(3, 3, cc.stride, cc.pad));
        check(engine::cuda::kernels_launched() == before + 1, cc.name + ": the forward is one kernel");
        check(max_abs_diff(y.to_vector(), f.at(cc.name + "/output").to_vector()) <= 1e-4, cc.name + ": output");
        y.backward(f.at(cc.name + "/grad_output"));
        check(max_abs_diff(x.grad().to_vector(), f.at(cc.name + "/grad.input").to_vector()) <= 1e-4,
              cc.name + ": gradient of the input");
        check(max_abs_diff(w.grad().to_vector(), f.at(cc.name + "/grad.weight").to_vector()) <= 1e-4,
              cc.name + ": gradient of the kernel");
        check(max_abs_diff(b.grad().to_vector(), f.at(cc.name + "/grad.bias").to_vector()) <= 1e-4,
              cc.name + ": gradient of the bias");
        // a second backward accumulates (Tensor::add_grad)
        const std::vector<float> once = w.grad().to_vector();
        Tensor y2 = nn::conv2d(x, w, &b, nn::Window2d(3, 3, cc.stride, cc.pad));
        y2.backward(f.at(cc.name + "/grad_output"));
        std::vector<float> twice = w.grad().to_vector(), want2(once.size());
        for (size_t i = 0; i < once.size(); ++i) want2[i] = 2.0f * once[i];
        check(max_abs_diff(twice, want2) <= 1e-4, cc.name + ": a second backward adds to the stored gradient");
    }
    check_throws([&] { nn::conv2d(Tensor({2, 3, 8}), Tensor({4, 3, 3, 3}), nullptr, nn::Window2d(3)); },
                 "conv2d of a 3-D input throws");
    check_throws([&] { nn::conv2d(Tensor({2, 2, 8, 8}), Tensor({4, 3, 3, 3}), nullptr, nn::Window2d(3)); },
                 "conv2d with mismatched channels throws");

    for (const std::string name : {"attention", "attention_causal"}) {
        const bool has_mask = f.count(name + "/mask") != 0;
        Tensor mask = has_mask ? f.at(name + "/mask") : Tensor();
        Tensor weights;
        const size_t before = engine::cuda::kernels_launched();
        Tensor out = nn::scaled_dot_product_attention(f.at(name + "/q"), f.at(name + "/k"), f.at(name + "/v"),
                                                      has_mask ? &mask : nullptr, &weights);
        check(engine::cuda::kernels_launched() == before + 1, name + ": one kernel");
        check(max_abs_diff(out.to_vector(), f.at(name + "/output").to_vector()) <= 1e-4, name + ": output");
        const std::vector<float> wv = weights.to_vector();
        const size_t s_k = weights.shape().back();
        double worst = 0.0;
        for (size_t r = 0; r < wv.size() / s_k; ++r) {
            double sum = 0.0;
            for (size_t j = 0; j < s_k; ++j) sum += wv[r * s_k + j];
            worst = std::max(worst, std::fabs(sum - 1.0));
        }
        check(worst <= 1e-5, name + ": attention weights sum to one per row");
    }
    for (const std::string name : {"attention", "attention_causal"}) {
        const bool has_mask = f.count(name + "/mask") != 0;
        Tensor mask = has_mask ? f.at(name + "/mask") : Tensor();
        Tensor q = f.at(name + "/q").detach(), k = f.at(name + "/k").detach(), v = f.at(name + "/v").detach();
        q.set_requires_grad(true);
        k.set_requires_grad(true);
        v.set_requires_grad(true);
        Tensor out = nn::scaled_dot_product_attention(q, k, v, has_mask ? &mask : nullptr);
        const size_t before = engine::cuda::kernels_launched();
        out.backward(f.at(name + "/grad_output"));
        check(engine::cuda::kernels_launched() == before + 1, name + ": the backward is one kernel");
        check(max_abs_diff(q.grad().to_vector(), f.at(name + "/grad.q").to_vector()) <= 1e-4, name + ": gradient of Q");
        check(max_abs_diff(k.grad().to_vector(), f.at(name + "/grad.k").to_vector()) <= 1e-4, name + ": gradient of K");
        check(max_abs_diff(v.grad().to_vector(), f.at(name + "/grad.v").to_vector()) <= 1e-4, name + ": gradient of V");
    }

    // MultiHeadAttention(8, 2): four Linear layers around the strided attention core
    {
        Tensor x = f.at("multihead/input");
        std::map<std::string, Tensor> proj;
        for (const std::string tag : {"query", "key", "value"}) {
            Tensor bias = f.at("multihead/w." + tag + ".bias");
            proj.emplace(tag, nn::linear(x, f.at("multihead/w." + tag + ".weight"), &bias));
        }
        const size_t before = engine::cuda::kernels_launched();
        Tensor merged = nn::multi_head_attention_core(proj.at("query"), proj.at("key"), proj.at("value"), 2);
        check(engine::cuda::kernels_launched() == before + 1, "multihead: split, attention and merge are one kernel");
        Tensor out_bias = f.at("multihead/w.out.bias");
        Tensor out = nn::linear(merged, f.at("multihead/w.out.weight"), &out_bias);
        check(max_abs_diff(out.to_vector(), f.at("multihead/output").to_vector()) <= 1e-4, "multihead: output");
    }

    // A head beyond the fused kernels' tiles (S = 200, d = 80): the layer runs it composed on the device
    // and must agree with the reference's sequence of steps (src/transformer.cpp:279-304 and the backward
    // lambdas of its nodes) evaluated by the CPU oracle.
    {
        engine::manual_seed(33);
        const size_t B = 3, S = 200, D = 80;
        Tensor q = Tensor::randn({B, S, D}, 0.0f, 1.0f, true), k = Tensor::randn({B, S, D}, 0.0f, 1.0f, true);
        Tensor v = Tensor::randn({B, S, D}, 0.0f, 1.0f, true), g = Tensor::randn({B, S, D});
        const float scale = 1.0f / std::sqrt(static_cast<float>(D));
        Tensor out = nn::scaled_dot_product_attention(q, k, v);
        out.backward(g);
        const std::vector<float> vq = q.to_vector(), vk = k.to_vector(), vv = v.to_vector(), vg = g.to_vector();
        std::vector<float> sc(B * S * S), w(B * S * S), want(B * S * D), dw(B * S * S), ds(B * S * S);
        std::vector<float> dq(B * S * D), dk(B * S * D), dv(B * S * D);
        oracle_matmul_nt_f32(vq.data(), vk.data(), sc.data(), B, S, D, S, 1, 1, 0);
        for (float& x : sc) x *= scale;
        oracle_softmax_rows_f32(sc.data(), w.data(), B * S, S);
        oracle_matmul_f32(w.data(), vv.data(), want.data(), B, S, S, D, 1, 1, 0);
        oracle_matmul_nt_f32(vg.data(), vv.data(), dw.data(), B, S, D, S, 1, 1, 0);       // dW = g x v^T
        oracle_matmul_tn_f32(w.data(), vg.data(), dv.data(), B, S, S, D, 1, 1, 0);        // dv = W^T x g
        oracle_softmax_backward_f32(w.data(), dw.data(), ds.data(), B * S, S);
        for (float& x : ds) x *= scale;
        oracle_matmul_f32(ds.data(), vk.data(), dq.data(), B, S, S, D, 1, 1, 0);          // dq = dS x k
        oracle_matmul_tn_f32(ds.data(), vq.data(), dk.data(), B, S, S, D, 1, 1, 0);       // dk = dS^T x q
        check(scaled_error(out.to_vector(), want) <= 2e-5, "attention S=200 d=80 (composed on the device): output");
        check(scaled_error(q.grad().to_vector(), dq) <= 4e-5, "attention S=200 d=80: gradient of Q");
        check(scaled_error(k.grad().to_vector(), dk) <= 4e-5, "attention S=200 d=80: gradient of K");
        check(scaled_error(v.grad().to_vector(), dv) <= 4e-5, "attention S=200 d=80: gradient of V");
    }

    section("Linear: fused bias / ReLU and gradients");
    engine::manual_seed(21);
    Tensor x = Tensor::randn({4, 33, 96}, 0.0f, 1.0f, true);
    Tensor w = Tensor::rand({96, 121}, -0.17f, 0.17f, true);
    Tensor b = Tensor::randn({121}, 0.0f, 1.0f, true);
    {
        const size_t before = engine::cuda::kernels_launched();
        Tensor y = nn::linear(x, w, &b);
        check(engine::cuda::kernels_launched() == before + 1, "linear: product and bias are one kernel");
        std::vector<float> want = oracle_matmul(x.reshape({4 * 33, 96}), w), bv = b.to_vector();
        for (size_t i = 0; i < want.size(); ++i) want[i] += bv[i % 121];
        check(y.shape() == std::vector<size_t>({4, 33, 121}), "linear: the leading axes are restored");
        check(scaled_error(y.to_vector(), want) <= tolerance(96), "linear: output against the CPU loop + bias");
        std::vector<float> relu_want = want;
        for (float& v : relu_want) v = std::max(v, 0.0f);
        check(scaled_error(nn::linear(x, w, &b, true).to_vector(), relu_want) <= tolerance(96),
              "linear: fused ReLU");
        Tensor g = Tensor::randn({4, 33, 121});
        y.backward(g);
        // the same gradients through the plain product
        Tensor x2 = x.detach().reshape({4 * 33, 96}), w2 = w.detach();
        x2.set_requires_grad(true);
        w2.set_requires_grad(true);
        Tensor y2 = x2.matmul(w2);
        y2.backward(g.reshape({4 * 33, 121}));
        check(scaled_error(x.grad().to_vector(), x2.grad().to_vector()) <= 1e-5, "linear: gradient of the input");
        check(scaled_error(w.grad().to_vector(), w2.grad().to_vector()) <= 1e-5, "linear: gradient of the weight");
        std::vector<float> gv = g.to_vector(), db(121, 0.0f);
        for (size_t r = 0; r < 4 * 33; ++r)
            for (size_t c = 0; c < 121; ++c) db[c] += gv[r * 121 + c];
        check(scaled_error(b.grad().to_vector(), db) <= tolerance(4 * 33), "linear: gradient of the bias");
    }
    check_throws([&] { nn::linear(Tensor({4, 95}), w); }, "linear with a wrong input width throws");
}

// Informational: what one engine-sized product costs a C++ caller, back to back (no result is
// read in between, so launches queue up behind each other like in a training step).
void report_call_cost() {
    section("Cost per call from C++ (informational)");
    engine::manual_seed(31);
    Tensor x = Tensor::randn({2048, 96}), w = Tensor::rand({96, 384}, -0.1f, 0.1f);
    Tensor b = Tensor::randn({384});
    for (int i = 0; i < 20; ++i) x.matmul(w);
    engine::cuda::synchronize();
    const int reps = 500;
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < reps; ++i) x.matmul(w);
    auto t1 = std::chrono::steady_clock::now();
    engine::cuda::synchronize();
    auto t2 = std::chrono::steady_clock::now();
    const double issue_us = std::chrono::duration<double, std::micro>(t1 - t0).count() / reps;
    const double total_us = std::chrono::duration<double, std::micro>(t2 - t0).count() / reps;
    std::cout << "  Tensor::matmul (2048 x 96) x (96 x 384): " << issue_us << " us of host time per call, " << total_us
              << " us per call until the device is idle\n";
    for (int i = 0; i < 20; ++i) engine::nn::linear(x, w, &b, true);
    engine::cuda::synchronize();
    t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < reps; ++i) engine::nn::linear(x, w, &b, true);
    t1 = std::chrono::steady_clock::now();
    engine::cuda::synchronize();
    t2 = std::chrono::steady_clock::now();
    std::cout << "  nn::linear with bias and ReLU, same shape: "
              << std::chrono::duration<double, std::micro>(t1 - t0).count() / reps << " us of host time per call, "
              << std::chrono::duration<double, std::micro>(t2 - t0).count() / reps << " us per call until the device is idle\n";
}

}  // namespace

int main(int argc, char** argv) {
    const std::string golden_dir = argc > 1 ? argv[1] : "tests/golden";
    if (!engine::cuda::available()) {
        std::cout << "no CUDA device: the host side has no CPU path to test\n";
        return 2;
    }
    try {
        test_matmul_known_answers();
        test_golden_vectors(golden_dir);
        test_numerical_gradients();
        test_parity_shapes();
        test_residency_and_seam();
        test_reduced_precision_is_opt_in();
        test_layers(golden_dir);
        report_call_cost();
        engine::cuda::check_device_status();
    } catch (const std::exception& e) {
        std::cout << "EXCEPTION: " << e.what() << "\n";
        return 1;
    }
    std::cout << "\n" << (g_failures ? "FAILURES: " + std::to_string(g_failures) : std::string("ALL TESTS PASSED"))
              << " (" << g_checks << " checks)\n";
    return g_failures ? 1 : 0;
}
