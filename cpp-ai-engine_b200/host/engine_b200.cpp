// Implementation of the C++17 host side (see engine_b200.hpp).  Device memory comes from the
// CUDA stream-ordered pool, as in the reference (src/cuda/runtime.cu:352-362); every product
// goes through the C ABI of libb200gemm.so.
#include "engine_b200.hpp"

#include "b200_gemm.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <numeric>
#include <random>
#include <stdexcept>
#include <unordered_set>

namespace engine {

namespace {

void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
}

void check_b200(int rc, const char* what) {
    if (rc != 0) throw std::runtime_error(std::string(what) + ": " + b200_gemm_strerror(rc));
}

std::mt19937& global_rng() {
    static std::mt19937 gen(std::random_device{}());
    return gen;
}

cuda::TransferStats g_transfers;
cuda::MatmulKernel g_kernel = cuda::MatmulKernel::Auto;

float* device_alloc(size_t count) {
    static bool pool_ready = false;
    if (!pool_ready) {
        // Keep freed blocks in the pool instead of returning them to the driver.
        cudaMemPool_t pool;
        int dev = 0;
        check(cudaGetDevice(&dev), "cudaGetDevice");
        check(cudaDeviceGetDefaultMemPool(&pool, dev), "cudaDeviceGetDefaultMemPool");
        uint64_t threshold = UINT64_MAX;
        check(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold),
              "cudaMemPoolSetAttribute");
        pool_ready = true;
    }
    void* p = nullptr;
    check(cudaMallocAsync(&p, std::max<size_t>(count, 1) * sizeof(float), nullptr), "cudaMallocAsync");
    return static_cast<float*>(p);
}

void device_free(float* p) noexcept {
    if (p) cudaFreeAsync(p, nullptr);
}

size_t product(const std::vector<size_t>& v, size_t from = 0, size_t to = SIZE_MAX) {
    size_t n = 1;
    for (size_t i = from; i < std::min(to, v.size()); ++i) n *= v[i];
    return n;
}

// Grow-only scratch for the split-K path, one per process (single device, single stream,
// like the reference's scratch_buffer, src/cuda/kernels.cu:593-604).
struct Scratch {
    void* ptr = nullptr;
    size_t bytes = 0;
    void* get(size_t need) {
        if (need > bytes) {
            if (ptr) cudaFree(ptr);
            ptr = nullptr;
            bytes = 0;
            check(cudaMalloc(&ptr, need), "cudaMalloc(scratch)");
            bytes = need;
        }
        return ptr;
    }
} g_scratch;

}  // namespace

void manual_seed(uint64_t seed) {
    global_rng().seed(static_cast<std::mt19937::result_type>(seed));
}

// ------------------------------------------------------------------------------- Storage
Storage::Buffer::~Buffer() { device_free(device); }

Storage::Storage() : buf_(std::make_shared<Buffer>()) {}

Storage::Storage(size_t count, float fill) : buf_(std::make_shared<Buffer>()) {
    buf_->count = count;
    buf_->fill = fill;  // the host vector is allocated on first host access
}

Storage::Storage(std::vector<float> values) : buf_(std::make_shared<Buffer>()) {
    buf_->count = values.size();
    buf_->host = std::move(values);
}

void Storage::materialise() const {
    if (buf_->host.size() != buf_->count) buf_->host.assign(buf_->count, buf_->fill);
}

void Storage::ensure_device_buffer() const {
    if (!buf_->device) buf_->device = device_alloc(buf_->count);
}

const std::vector<float>& Storage::host() const {
    if (!buf_->host_valid) {
        buf_->host.resize(buf_->count);
        if (buf_->count) {
            check(cudaMemcpy(buf_->host.data(), buf_->device, buf_->count * sizeof(float),
                             cudaMemcpyDeviceToHost),
                  "cudaMemcpy(D2H)");
            g_transfers.to_host_bytes += buf_->count * sizeof(float);
            g_transfers.to_host_count += 1;
        }
        buf_->host_valid = true;
    } else {
        materialise();
    }
    return buf_->host;
}

std::vector<float>& Storage::host_mut() {
    host();
    buf_->device_valid = false;
    return buf_->host;
}

const float* Storage::device() const {
    ensure_device_buffer();
    if (!buf_->device_valid) {
        materialise();
        if (buf_->count) {
            check(cudaMemcpy(buf_->device, buf_->host.data(), buf_->count * sizeof(float),
                             cudaMemcpyHostToDevice),
                  "cudaMemcpy(H2D)");
            g_transfers.to_device_bytes += buf_->count * sizeof(float);
            g_transfers.to_device_count += 1;
        }
        buf_->device_valid = true;
    }
    return buf_->device;
}

float* Storage::device_mut() {
    device();
    buf_->host_valid = false;
    return buf_->device;
}

float* Storage::device_write() {
    ensure_device_buffer();
    buf_->reverted_host_valid = buf_->host_valid;
    buf_->device_valid = true;
    buf_->host_valid = false;
    return buf_->device;
}

void Storage::revert_device_write() {
    buf_->device_valid = false;
    buf_->host_valid = true;  // the constructor's fill (or the previous host values) stand
}

Storage Storage::clone() const {
    Storage out(buf_->count, buf_->fill);
    if (buf_->device_valid && !buf_->host_valid) {
        float* dst = out.device_write();
        if (buf_->count) {
            check(cudaMemcpyAsync(dst, buf_->device, buf_->count * sizeof(float),
                                  cudaMemcpyDeviceToDevice, nullptr),
                  "cudaMemcpyAsync(D2D)");
        }
    } else {
        out.buf_->host = host();
    }
    return out;
}

Storage Storage::share() const {
    Storage out;
    out.buf_ = buf_;
    return out;
}

// ------------------------------------------------------------------------------- cuda::
namespace cuda {

bool available() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return n > 0;
}

void synchronize() { check(cudaDeviceSynchronize(), "cudaDeviceSynchronize"); }

TransferStats transfer_stats() { return g_transfers; }
void reset_transfer_stats() { g_transfers = TransferStats{}; }
size_t kernels_launched() { return static_cast<size_t>(b200_gemm_launch_count()); }

void set_matmul_kernel(MatmulKernel kernel) { g_kernel = kernel; }
MatmulKernel matmul_kernel() { return g_kernel; }

void check_device_status() { check_b200(b200_gemm_status(), "device status"); }

namespace ops {

bool matmul_ex(const Storage& a, const Storage& b, Storage& out, size_t batch, size_t rows,
               size_t inner_dim, size_t cols, bool a_batched, bool b_batched, bool a_transposed,
               bool b_transposed, float beta) {
    const size_t a_need = (a_batched ? batch : 1) * rows * inner_dim;
    const size_t b_need = (b_batched ? batch : 1) * inner_dim * cols;
    if (a.size() != a_need || b.size() != b_need || out.size() != batch * rows * cols) {
        throw std::runtime_error("cuda::ops::matmul: buffer sizes do not match the shapes");
    }
    if (out.size() == 0) return true;
    const float* pa = a.device();
    const float* pb = b.device();
    // beta == 0: the output is written in full, never uploaded; otherwise it is read first.
    float* pc = (beta == 0.0f) ? out.device_write() : out.device_mut();
    const int64_t M = static_cast<int64_t>(rows), K = static_cast<int64_t>(inner_dim),
                  N = static_cast<int64_t>(cols), nb = static_cast<int64_t>(batch);
    const size_t ws_bytes = b200_gemm_f32_workspace(nb, M, N, K);
    void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
    const int precision =
        g_kernel == MatmulKernel::TensorCore ? B200_PRECISION_TF32 : B200_PRECISION_3XTF32;
    const int rc = b200_gemm_f32(pa, pb, pc, nb, M, N, K, a_transposed ? 1 : 0, b_transposed ? 1 : 0,
                                 a_transposed ? M : K, b_transposed ? K : N, N,
                                 a_batched ? M * K : 0, b_batched ? K * N : 0, M * N, 1.0f, beta,
                                 precision, ws, ws_bytes, nullptr);
    if (rc != 0) {
        if (beta == 0.0f) out.revert_device_write();
        throw std::runtime_error(std::string("cuda::ops::matmul: ") + b200_gemm_strerror(rc));
    }
    return true;
}

bool matmul(const Storage& a, const Storage& b, Storage& out, size_t batch, size_t rows,
            size_t inner_dim, size_t cols, bool a_batched, bool b_batched, float beta) {
    return matmul_ex(a, b, out, batch, rows, inner_dim, cols, a_batched, b_batched, false, false,
                     beta);
}

}  // namespace ops
}  // namespace cuda

// ------------------------------------------------------------------------------- Tensor
struct TensorImpl {
    std::vector<size_t> shape;  // logical shape
    Storage storage;            // stored row-major; last two axes swapped when `transposed`
    bool transposed = false;
    bool requires_grad = false;
    std::shared_ptr<TensorImpl> grad;  // same layout as this tensor's storage
    std::vector<std::shared_ptr<TensorImpl>> parents;
    std::function<void(const Tensor&)> backward_fn;

    static Tensor wrap(std::shared_ptr<TensorImpl> p) { return Tensor(std::move(p)); }
    static const std::shared_ptr<TensorImpl>& of(const Tensor& t) { return t.impl_; }
};

namespace {

thread_local bool g_grad_enabled = true;
struct NoGradGuard {
    bool saved;
    NoGradGuard() : saved(g_grad_enabled) { g_grad_enabled = false; }
    ~NoGradGuard() { g_grad_enabled = saved; }
};

std::string shape_to_string(const std::vector<size_t>& s) {
    std::string out = "(";
    for (size_t i = 0; i < s.size(); ++i) {
        if (i) out += ", ";
        out += std::to_string(s[i]);
    }
    return out + ")";
}

std::shared_ptr<TensorImpl> make_impl(const std::vector<size_t>& shape, Storage storage,
                                      bool requires_grad) {
    auto p = std::make_shared<TensorImpl>();
    p->shape = shape;
    p->storage = std::move(storage);
    p->requires_grad = requires_grad;
    return p;
}

}  // namespace

Tensor::Tensor() : impl_(make_impl({}, Storage(), false)) {}
Tensor::Tensor(std::shared_ptr<TensorImpl> impl) : impl_(std::move(impl)) {}

Tensor::Tensor(const std::vector<size_t>& shape, float fill_value, bool requires_grad)
    : impl_(make_impl(shape, Storage(product(shape), fill_value), requires_grad)) {}

Tensor::Tensor(const std::vector<size_t>& shape, const std::vector<float>& data, bool requires_grad) {
    if (data.size() != product(shape)) {
        throw std::invalid_argument("Tensor: " + std::to_string(data.size()) +
                                    " values do not fill shape " + shape_to_string(shape) + ".");
    }
    impl_ = make_impl(shape, Storage(data), requires_grad);
}

Tensor Tensor::zeros(const std::vector<size_t>& shape, bool requires_grad) {
    return Tensor(shape, 0.0f, requires_grad);
}
Tensor Tensor::ones(const std::vector<size_t>& shape, bool requires_grad) {
    return Tensor(shape, 1.0f, requires_grad);
}

Tensor Tensor::rand(const std::vector<size_t>& shape, float min_val, float max_val,
                    bool requires_grad) {
    std::vector<float> v(product(shape));
    std::uniform_real_distribution<float> dis(min_val, max_val);
    for (float& x : v) x = dis(global_rng());
    return Tensor(shape, v, requires_grad);
}

Tensor Tensor::randn(const std::vector<size_t>& shape, float mean, float stddev, bool requires_grad) {
    std::vector<float> v(product(shape));
    std::normal_distribution<float> dis(mean, stddev);
    for (float& x : v) x = dis(global_rng());
    return Tensor(shape, v, requires_grad);
}

bool Tensor::requires_grad() const { return impl_->requires_grad; }
void Tensor::set_requires_grad(bool r) { impl_->requires_grad = r; }
bool Tensor::has_grad() const { return impl_->grad != nullptr; }
void Tensor::zero_grad() { impl_->grad.reset(); }

Tensor Tensor::grad() const {
    if (!impl_->grad) throw std::runtime_error("This tensor has no gradient.");
    return Tensor(impl_->grad);
}

const std::vector<size_t>& Tensor::shape() const { return impl_->shape; }
size_t Tensor::ndim() const { return impl_->shape.size(); }
size_t Tensor::size() const { return product(impl_->shape); }
std::string Tensor::shape_str() const { return shape_to_string(impl_->shape); }
bool Tensor::resident_on_device() const { return impl_->storage.resident_on_device(); }
bool Tensor::is_transposed_view() const { return impl_->transposed; }

std::vector<float> Tensor::to_vector() const {
    const std::vector<float>& stored = impl_->storage.host();
    if (!impl_->transposed) return stored;
    const size_t nd = impl_->shape.size();
    const size_t rows = impl_->shape[nd - 2], cols = impl_->shape[nd - 1];
    const size_t batch = product(impl_->shape, 0, nd - 2);
    std::vector<float> out(stored.size());
    for (size_t b = 0; b < batch; ++b)
        for (size_t i = 0; i < rows; ++i)
            for (size_t j = 0; j < cols; ++j)
                out[(b * rows + i) * cols + j] = stored[(b * cols + j) * rows + i];
    return out;
}

float Tensor::at(size_t flat_index) const {
    if (flat_index >= size()) throw std::out_of_range("Tensor::at: index out of range.");
    return to_vector()[flat_index];
}

float Tensor::operator()(size_t row, size_t col) const {
    if (ndim() != 2 || row >= impl_->shape[0] || col >= impl_->shape[1]) {
        throw std::out_of_range("Tensor(row, col): needs a 2-D tensor and indices in range.");
    }
    const std::vector<float>& stored = impl_->storage.host();
    return impl_->transposed ? stored[col * impl_->shape[0] + row] : stored[row * impl_->shape[1] + col];
}

Tensor Tensor::detach() const {
    auto p = make_impl(impl_->shape, impl_->storage.share(), false);
    p->transposed = impl_->transposed;
    return Tensor(p);
}

Tensor Tensor::transpose() const {
    if (ndim() < 2) throw std::invalid_argument("transpose requires at least 2 dimensions.");
    std::vector<size_t> shape = impl_->shape;
    std::swap(shape[shape.size() - 1], shape[shape.size() - 2]);
    const bool track = g_grad_enabled && impl_->requires_grad;
    auto p = make_impl(shape, impl_->storage.share(), track);
    p->transposed = !impl_->transposed;
    if (track) {
        p->parents = {impl_};
        Tensor self = *this;
        // The gradient of a view arrives in the view's layout: the same bytes are the base's
        // gradient in the base's layout.
        p->backward_fn = [self](const Tensor& g) mutable { self.add_grad(g.transpose()); };
    }
    return Tensor(p);
}

Tensor Tensor::reshape(const std::vector<size_t>& new_shape) const {
    if (product(new_shape) != size()) {
        throw std::invalid_argument("reshape: cannot view " + shape_str() + " as " +
                                    shape_to_string(new_shape) + ".");
    }
    const bool track = g_grad_enabled && impl_->requires_grad;
    Storage st = impl_->transposed ? Storage(to_vector()) : impl_->storage.share();
    auto p = make_impl(new_shape, std::move(st), track);
    if (track) {
        p->parents = {impl_};
        Tensor self = *this;
        std::vector<size_t> old_shape = impl_->shape;
        p->backward_fn = [self, old_shape](const Tensor& g) mutable {
            self.add_grad(g.reshape(old_shape));
        };
    }
    return Tensor(p);
}

// First write shares the incoming buffer, later writes accumulate (src/tensor.cpp:168-203).
// The products of the backward pass accumulate on the device through beta = 1 and never come
// here twice; this host-side sum serves the view nodes (transpose / reshape of a tensor that
// is used more than once).
void Tensor::add_grad(const Tensor& g) {
    if (!requires_grad()) return;
    if (g.shape() != shape()) {
        throw std::invalid_argument("Gradient shape " + g.shape_str() +
                                    " incompatible with the tensor's " + shape_str() + ".");
    }
    const bool same_layout = g.impl_->transposed == impl_->transposed;
    if (!impl_->grad) {
        Storage st = same_layout ? g.impl_->storage.clone() : Storage(g.to_vector());
        if (!same_layout && impl_->transposed) {
            // store in this tensor's (transposed) layout
            Tensor tmp(g.shape(), g.to_vector());
            st = Storage(tmp.transpose().to_vector());
        }
        auto p = make_impl(impl_->shape, std::move(st), false);
        p->transposed = impl_->transposed;
        impl_->grad = p;
        return;
    }
    std::vector<float> add = same_layout ? g.impl_->storage.host() : g.to_vector();
    if (!same_layout && impl_->transposed) {
        Tensor tmp(g.shape(), g.to_vector());
        add = tmp.transpose().to_vector();
    }
    std::vector<float>& dst = impl_->grad->storage.host_mut();
    for (size_t i = 0; i < dst.size(); ++i) dst[i] += add[i];
}

namespace {

struct Operand {
    std::shared_ptr<TensorImpl> impl;
    bool batched;
};

// One product on raw device pointers (row-major, contiguous matrices).
void raw_gemm(const float* a, const float* b, float* c, size_t batch, size_t M, size_t K, size_t N,
              bool a_t, bool b_t, size_t stride_a, size_t stride_b, float beta) {
    const int64_t m = static_cast<int64_t>(M), k = static_cast<int64_t>(K), n = static_cast<int64_t>(N),
                  nb = static_cast<int64_t>(batch);
    const size_t ws_bytes = b200_gemm_f32_workspace(nb, m, n, k);
    void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
    const int precision =
        g_kernel == cuda::MatmulKernel::TensorCore ? B200_PRECISION_TF32 : B200_PRECISION_3XTF32;
    check_b200(b200_gemm_f32(a, b, c, nb, m, n, k, a_t ? 1 : 0, b_t ? 1 : 0, a_t ? m : k, b_t ? k : n, n,
                             static_cast<int64_t>(stride_a), static_cast<int64_t>(stride_b), m * n, 1.0f,
                             beta, precision, ws, ws_bytes, nullptr),
               "matmul backward");
}

// Gradient of one operand of C = A x B, computed straight into (or accumulated onto) the
// operand's own storage layout with one transposed-form product — no transpose is built.
// `first` selects A (dA = g x B^T) or B (dB = A^T x g).
void operand_gradient(bool first, const Operand& A, const Operand& B, const Tensor& g, size_t batch,
                      size_t M, size_t K, size_t N) {
    const Operand& X = first ? A : B;
    TensorImpl& x = *X.impl;
    const bool a_t = A.impl->transposed, b_t = B.impl->transposed;
    const float beta = x.grad ? 1.0f : 0.0f;
    if (!x.grad) {
        auto p = make_impl(x.shape, Storage(product(x.shape), 0.0f), false);
        p->transposed = x.transposed;
        x.grad = p;
    }
    const float* pg = TensorImpl::of(g)->storage.device();
    const float* pa = A.impl->storage.device();
    const float* pb = B.impl->storage.device();
    float* out = (beta == 0.0f) ? x.grad->storage.device_write() : x.grad->storage.device_mut();
    const size_t sg = M * N, sa = A.batched ? M * K : 0, sb = B.batched ? K * N : 0;

    // The four layouts of one gradient product over `nb` batch elements starting at element b0.
    auto run = [&](size_t b0, size_t nb, float bt) {
        const float* g0 = pg + b0 * sg;
        const float* a0 = pa + b0 * sa;
        const float* b0p = pb + b0 * sb;
        float* o0 = out + (X.batched ? b0 * (first ? M * K : K * N) : 0);
        if (first && !a_t) {  // dA (M x K) = g (M x N) x B^T
            raw_gemm(g0, b0p, o0, nb, M, N, K, false, !b_t, sg, sb, bt);
        } else if (first) {  // A = S^T: dS (K x M) = B (K x N) x g^T (N x M)
            raw_gemm(b0p, g0, o0, nb, K, N, M, b_t, true, sb, sg, bt);
        } else if (!b_t) {  // dB (K x N) = A^T (K x M) x g (M x N)
            raw_gemm(a0, g0, o0, nb, K, M, N, !a_t, false, sa, sg, bt);
        } else {  // B = S^T: dS (N x K) = g^T (N x M) x A (M x K)
            raw_gemm(g0, a0, o0, nb, N, M, K, true, a_t, sg, sa, bt);
        }
    };

    if (X.batched || batch == 1) {
        run(0, batch, beta);
        return;
    }
    // The operand is one matrix shared by the whole batch: its gradient is the sum of the
    // per-element contributions (src/tensor_ops.cpp:577-583).
    if (!first && !b_t && !a_t) {
        // A is (batch*M) x K and g is (batch*M) x N, both contiguous: one product over batch*M.
        raw_gemm(pa, pg, out, 1, K, batch * M, N, true, false, 0, 0, beta);
        return;
    }
    // Otherwise accumulate element by element, in ascending batch order like fold_leading.
    for (size_t bi = 0; bi < batch; ++bi) run(bi, 1, bi == 0 ? beta : 1.0f);
}

}  // namespace

Tensor Tensor::matmul(const Tensor& B) const {
    if (ndim() < 2 || B.ndim() < 2) {
        throw std::invalid_argument("MatMul requires at least 2 dimensions in both operands.");
    }
    const size_t nd_a = ndim(), nd_b = B.ndim();
    const std::vector<size_t> batch_a(shape().begin(), shape().end() - 2);
    const std::vector<size_t> batch_b(B.shape().begin(), B.shape().end() - 2);
    const bool a_batched = !batch_a.empty();
    const bool b_batched = !batch_b.empty();
    if (a_batched && b_batched && batch_a != batch_b) {
        throw std::invalid_argument("Batched MatMul needs identical batch axes: " + shape_str() +
                                    " and " + B.shape_str() + ".");
    }
    const std::vector<size_t>& batch_dims = a_batched ? batch_a : batch_b;
    const size_t M = shape()[nd_a - 2], K = shape()[nd_a - 1];
    const size_t K2 = B.shape()[nd_b - 2], N = B.shape()[nd_b - 1];
    if (K != K2) {
        throw std::invalid_argument("Incompatible dimensions for MatMul: " + shape_str() + " and " +
                                    B.shape_str() + ".");
    }
    const size_t batch = product(batch_dims);
    std::vector<size_t> out_shape = batch_dims;
    out_shape.push_back(M);
    out_shape.push_back(N);
    const bool req_g = g_grad_enabled && (requires_grad() || B.requires_grad());
    Tensor C(out_shape, 0.0f, req_g);

    cuda::ops::matmul_ex(impl_->storage, B.impl_->storage, C.impl_->storage, batch, M, K, N, a_batched,
                         b_batched, impl_->transposed, B.impl_->transposed, 0.0f);

    if (req_g) {
        C.impl_->parents = {impl_, B.impl_};
        const Operand opA{impl_, a_batched}, opB{B.impl_, b_batched};
        C.impl_->backward_fn = [opA, opB, batch, M, K, N](const Tensor& grad_out) {
            Tensor g = grad_out.is_transposed_view() ? Tensor(grad_out.shape(), grad_out.to_vector())
                                                     : grad_out;
            if (opA.impl->requires_grad) operand_gradient(true, opA, opB, g, batch, M, K, N);
            if (opB.impl->requires_grad) operand_gradient(false, opA, opB, g, batch, M, K, N);
        };
    }
    return C;
}

void Tensor::backward() {
    if (size() != 1) throw std::runtime_error("backward() without an argument needs a scalar.");
    backward(Tensor(shape(), 1.0f));
}

// Iterative topological sort, then a reverse sweep (src/autograd.cpp:23-83, 104-156); the sweep
// builds no graph of its own.
void Tensor::backward(const Tensor& grad_output) {
    if (grad_output.shape() != shape()) {
        throw std::invalid_argument("Gradient shape " + grad_output.shape_str() +
                                    " incompatible with the tensor's " + shape_str() + ".");
    }
    std::vector<TensorImpl*> order;
    std::unordered_set<TensorImpl*> seen;
    std::vector<std::pair<TensorImpl*, bool>> stack{{impl_.get(), false}};
    while (!stack.empty()) {
        auto [node, expanded] = stack.back();
        stack.pop_back();
        if (expanded) {
            order.push_back(node);
            continue;
        }
        if (!seen.insert(node).second) continue;
        stack.push_back({node, true});
        for (const auto& parent : node->parents) stack.push_back({parent.get(), false});
    }
    NoGradGuard guard;
    const bool was_tracked = impl_->requires_grad;
    impl_->requires_grad = true;
    impl_->grad.reset();
    add_grad(grad_output);
    impl_->requires_grad = was_tracked;
    for (auto it = order.rbegin(); it != order.rend(); ++it) {
        TensorImpl* node = *it;
        if (node->backward_fn && node->grad) node->backward_fn(Tensor(node->grad));
    }
}

// ------------------------------------------------------------------------------- nn
namespace nn {

namespace {

int current_precision() {
    return g_kernel == cuda::MatmulKernel::TensorCore ? B200_PRECISION_TF32 : B200_PRECISION_3XTF32;
}

const std::shared_ptr<TensorImpl>& impl_of(const Tensor& t) { return TensorImpl::of(t); }

// Row-major values of a tensor on the device (a transposed view is first copied into logical order).
Tensor contiguous(const Tensor& t) {
    if (!t.is_transposed_view()) return t;
    if (g_grad_enabled && t.requires_grad()) {
        throw std::invalid_argument("A layer operand that requires a gradient must not be a transposed view.");
    }
    return Tensor(t.shape(), t.to_vector());
}

// The gradient buffer of `x`, created on first use; returns the beta to accumulate with.
float* grad_buffer(TensorImpl& x, float* beta) {
    *beta = x.grad ? 1.0f : 0.0f;
    if (!x.grad) {
        auto p = make_impl(x.shape, Storage(product(x.shape), 0.0f), false);
        x.grad = p;
    }
    return *beta == 0.0f ? x.grad->storage.device_write() : x.grad->storage.device_mut();
}

}  // namespace

void Window2d::validate(size_t in_h, size_t in_w) const {
    if (kernel_h == 0 || kernel_w == 0 || stride == 0) {
        throw std::invalid_argument("Window2d requires a kernel and a stride greater than zero.");
    }
    if (in_h + 2 * padding < kernel_h || in_w + 2 * padding < kernel_w) {
        throw std::invalid_argument("The window does not fit the padded input.");
    }
}

Tensor linear(const Tensor& input_, const Tensor& weight_, const Tensor* bias, bool relu) {
    if (input_.ndim() < 2) {
        throw std::invalid_argument("Linear expects at least 2 dimensions (..., in_features), received " +
                                    input_.shape_str() + ".");
    }
    if (weight_.ndim() != 2) throw std::invalid_argument("Linear expects a 2-D weight (in, out).");
    const size_t in_f = weight_.shape()[0], out_f = weight_.shape()[1];
    if (input_.shape().back() != in_f) {
        throw std::invalid_argument("Linear with in_features=" + std::to_string(in_f) + " received an input " +
                                    input_.shape_str() + ".");
    }
    if (bias != nullptr && bias->size() != out_f) {
        throw std::invalid_argument("Linear expects one bias value per output feature.");
    }
    const Tensor input = contiguous(input_), weight = contiguous(weight_);
    const size_t rows = input.size() / in_f;
    std::vector<size_t> out_shape = input.shape();
    out_shape.back() = out_f;
    const bool tracked = g_grad_enabled && !relu &&
                         (input.requires_grad() || weight.requires_grad() || (bias && bias->requires_grad()));
    Tensor out(out_shape, 0.0f, tracked);
    if (rows == 0) return out;

    b200_epilogue ep{};
    ep.bias = bias ? impl_of(*bias)->storage.device() : nullptr;
    ep.relu = relu ? 1 : 0;
    const int64_t m = static_cast<int64_t>(rows), k = static_cast<int64_t>(in_f), n = static_cast<int64_t>(out_f);
    const size_t ws_bytes = b200_gemm_f32_workspace(1, m, n, k);
    void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
    float* dst = impl_of(out)->storage.device_write();
    check_b200(b200_gemm_f32_fused(impl_of(input)->storage.device(), impl_of(weight)->storage.device(), dst, 1, m,
                                   n, k, 0, 0, k, n, n, 0, 0, m * n, 1.0f, 0.0f, current_precision(), &ep, ws,
                                   ws_bytes, nullptr),
               "linear");
    if (!tracked) return out;

    auto xi = impl_of(input), wi = impl_of(weight);
    std::shared_ptr<TensorImpl> bi = bias ? impl_of(*bias) : nullptr;
    impl_of(out)->parents = {xi, wi};
    if (bi) impl_of(out)->parents.push_back(bi);
    impl_of(out)->backward_fn = [xi, wi, bi, rows, in_f, out_f](const Tensor& grad_out) {
        const Tensor g = contiguous(grad_out);
        const float* pg = impl_of(g)->storage.device();
        float beta = 0.0f;
        if (xi->requires_grad) {  // dX (rows x in) = g (rows x out) x W^T
            float* o = grad_buffer(*xi, &beta);
            raw_gemm(pg, wi->storage.device(), o, 1, rows, out_f, in_f, false, true, 0, 0, beta);
        }
        if (wi->requires_grad) {  // dW (in x out) = X^T x g
            float* o = grad_buffer(*wi, &beta);
            raw_gemm(xi->storage.device(), pg, o, 1, in_f, rows, out_f, true, false, 0, 0, beta);
        }
        if (bi && bi->requires_grad) {  // db (1 x out) = ones (1 x rows) x g
            const Storage ones(rows, 1.0f);
            float* o = grad_buffer(*bi, &beta);
            raw_gemm(ones.device(), pg, o, 1, 1, rows, out_f, false, false, 0, 0, beta);
        }
    };
    return out;
}

Tensor conv2d(const Tensor& input_, const Tensor& weight_, const Tensor* bias, const Window2d& window) {
    if (input_.ndim() != 4) {
        throw std::invalid_argument("Conv2d expects a 4D volume (N, C, H, W), received " + input_.shape_str() + ".");
    }
    if (weight_.ndim() != 4 || weight_.shape()[2] != window.kernel_h || weight_.shape()[3] != window.kernel_w) {
        throw std::invalid_argument("Conv2d expects a weight (outC, C, kH, kW) matching the window.");
    }
    if (input_.shape()[1] != weight_.shape()[1]) {
        throw std::invalid_argument("Conv2d with in_channels=" + std::to_string(weight_.shape()[1]) +
                                    " received an input " + input_.shape_str() + ".");
    }
    const size_t N = input_.shape()[0], C = input_.shape()[1], H = input_.shape()[2], W = input_.shape()[3];
    const size_t out_c = weight_.shape()[0];
    window.validate(H, W);
    if (bias != nullptr && bias->size() != out_c) {
        throw std::invalid_argument("Conv2d expects one bias value per output channel.");
    }
    const Tensor input = contiguous(input_), weight = contiguous(weight_);
    const size_t oH = window.out_h(H), oW = window.out_w(W);
    const bool tracked = g_grad_enabled &&
                         (input.requires_grad() || weight.requires_grad() || (bias && bias->requires_grad()));
    Tensor out({N, out_c, oH, oW}, 0.0f, tracked);
    if (out.size() == 0) return out;
    const auto i64 = [](size_t v) { return static_cast<int64_t>(v); };
    check_b200(b200_conv2d_forward_f32(impl_of(input)->storage.device(), impl_of(weight)->storage.device(),
                                       bias ? impl_of(*bias)->storage.device() : nullptr,
                                       impl_of(out)->storage.device_write(), i64(N), i64(C), i64(H), i64(W),
                                       i64(out_c), i64(window.kernel_h), i64(window.kernel_w), i64(window.stride),
                                       i64(window.padding), 0, current_precision(), nullptr),
               "conv2d forward");
    if (!tracked) return out;

    auto xi = impl_of(input), wi = impl_of(weight);
    std::shared_ptr<TensorImpl> bi = bias ? impl_of(*bias) : nullptr;
    impl_of(out)->parents = {xi, wi};
    if (bi) impl_of(out)->parents.push_back(bi);
    const Window2d win = window;
    impl_of(out)->backward_fn = [xi, wi, bi, win, N, C, H, W, out_c](const Tensor& grad_out) {
        const Tensor g = contiguous(grad_out);
        const auto i64 = [](size_t v) { return static_cast<int64_t>(v); };
        // A gradient that already exists is accumulated into (Tensor::add_grad), a new one is
        // written: at most one call for each of the two cases.
        float* fresh[3] = {nullptr, nullptr, nullptr};
        float* accum[3] = {nullptr, nullptr, nullptr};
        TensorImpl* targets[3] = {xi->requires_grad ? xi.get() : nullptr, wi->requires_grad ? wi.get() : nullptr,
                                  bi && bi->requires_grad ? bi.get() : nullptr};
        for (int which = 0; which < 3; ++which) {
            if (targets[which] == nullptr) continue;
            float beta = 0.0f;
            float* buf = grad_buffer(*targets[which], &beta);
            (beta == 0.0f ? fresh : accum)[which] = buf;
        }
        auto run = [&](float* const o[3], float beta) {
            if (o[0] == nullptr && o[1] == nullptr && o[2] == nullptr) return;
            const size_t ws_bytes = o[1] ? b200_conv2d_backward_workspace(
                                               i64(N), i64(C), i64(H), i64(W), i64(out_c), i64(win.kernel_h),
                                               i64(win.kernel_w), i64(win.stride), i64(win.padding))
                                         : 0;
            void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
            check_b200(b200_conv2d_backward_f32(xi->storage.device(), wi->storage.device(),
                                                impl_of(g)->storage.device(), o[0], o[1], o[2], i64(N), i64(C),
                                                i64(H), i64(W), i64(out_c), i64(win.kernel_h), i64(win.kernel_w),
                                                i64(win.stride), i64(win.padding), beta, current_precision(), ws,
                                                ws_bytes, nullptr),
                       "conv2d backward");
        };
        run(fresh, 0.0f);
        run(accum, 1.0f);
    };
    return out;
}

namespace {

bool attention_tracked(const Tensor& q, const Tensor& k, const Tensor& v) {
    return g_grad_enabled && (q.requires_grad() || k.requires_grad() || v.requires_grad());
}

// Attaches the backward of the attention core: ONE kernel that recomputes the weights and fills
// the gradients of q, k and v (those that exist are accumulated into, Tensor::add_grad).
void attach_attention_backward(Tensor& out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask,
                               bool has_mask, size_t batch, size_t heads, size_t s_q, size_t s_k, size_t d_k,
                               size_t d_v, const int64_t (&qs)[3], const int64_t (&ks)[3], const int64_t (&vs)[3],
                               const int64_t (&os)[3], float scale) {
    auto qi = impl_of(q), ki = impl_of(k), vi = impl_of(v);
    std::shared_ptr<TensorImpl> mi = has_mask ? impl_of(mask) : nullptr;
    impl_of(out)->parents = {qi, ki, vi};
    struct Strides {
        int64_t q[3], k[3], v[3], o[3];
    } st{};
    for (int i = 0; i < 3; ++i) st.q[i] = qs[i], st.k[i] = ks[i], st.v[i] = vs[i], st.o[i] = os[i];
    impl_of(out)->backward_fn = [qi, ki, vi, mi, st, batch, heads, s_q, s_k, d_k, d_v, scale](const Tensor& grad_out) {
        const Tensor g = contiguous(grad_out);
        const auto i64 = [](size_t x) { return static_cast<int64_t>(x); };
        float* fresh[3] = {nullptr, nullptr, nullptr};
        float* accum[3] = {nullptr, nullptr, nullptr};
        TensorImpl* targets[3] = {qi->requires_grad ? qi.get() : nullptr, ki->requires_grad ? ki.get() : nullptr,
                                  vi->requires_grad ? vi.get() : nullptr};
        for (int which = 0; which < 3; ++which) {
            if (targets[which] == nullptr) continue;
            float beta = 0.0f;
            float* buf = grad_buffer(*targets[which], &beta);
            (beta == 0.0f ? fresh : accum)[which] = buf;
        }
        auto run = [&](float* const o[3], float beta) {
            if (o[0] == nullptr && o[1] == nullptr && o[2] == nullptr) return;
            // heads the fused kernel does not take run composed on the device and want scratch
            const size_t ws_bytes = b200_attention_any_workspace(i64(batch), i64(heads), i64(s_q), i64(s_k),
                                                                 i64(d_k), i64(d_v), 1);
            void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
            check_b200(b200_attention_backward_any_f32(
                           qi->storage.device(), ki->storage.device(), vi->storage.device(),
                           mi ? mi->storage.device() : nullptr, impl_of(g)->storage.device(), o[0], o[1], o[2],
                           i64(batch), i64(heads), i64(s_q), i64(s_k), i64(d_k), i64(d_v), st.q, st.k, st.v, st.o,
                           scale, beta, current_precision(), ws, ws_bytes, nullptr),
                       "attention backward");
        };
        run(fresh, 0.0f);
        run(accum, 1.0f);
    };
}

const float* mask_pointer(const Tensor* mask, size_t s_q, size_t s_k, Tensor* keep) {
    if (mask == nullptr) return nullptr;
    if (mask->ndim() != 2 || mask->shape()[0] != s_q || mask->shape()[1] != s_k) {
        throw std::invalid_argument("The attention mask must be (S_q, S_k), received " + mask->shape_str() + ".");
    }
    *keep = contiguous(*mask);
    return impl_of(*keep)->storage.device();
}

}  // namespace

Tensor scaled_dot_product_attention(const Tensor& query_, const Tensor& key_, const Tensor& value_,
                                    const Tensor* mask, Tensor* attention_weights) {
    if (query_.ndim() < 2 || key_.ndim() < 2 || value_.ndim() < 2) {
        throw std::invalid_argument("Attention needs at least 2 dimensions (seq, d_k).");
    }
    const size_t d_k = query_.shape().back();
    if (key_.shape().back() != d_k) {
        throw std::invalid_argument("Query and key must share d_k: " + query_.shape_str() + " and " +
                                    key_.shape_str() + ".");
    }
    const bool tracked = attention_tracked(query_, key_, value_);
    const Tensor q = contiguous(query_), k = contiguous(key_), v = contiguous(value_);
    const std::vector<size_t> lead(q.shape().begin(), q.shape().end() - 2);
    const size_t s_q = q.shape()[q.ndim() - 2], s_k = k.shape()[k.ndim() - 2], d_v = v.shape().back();
    if (std::vector<size_t>(k.shape().begin(), k.shape().end() - 2) != lead ||
        std::vector<size_t>(v.shape().begin(), v.shape().end() - 2) != lead || v.shape()[v.ndim() - 2] != s_k) {
        throw std::invalid_argument("Batched MatMul needs identical batch axes: " + q.shape_str() + ", " +
                                    k.shape_str() + " and " + v.shape_str() + ".");
    }
    Tensor mask_keep;
    const float* pm = mask_pointer(mask, s_q, s_k, &mask_keep);
    std::vector<size_t> out_shape = lead, w_shape = lead;
    out_shape.insert(out_shape.end(), {s_q, d_v});
    w_shape.insert(w_shape.end(), {s_q, s_k});
    Tensor out(out_shape, 0.0f, tracked);
    Tensor weights = attention_weights ? Tensor(w_shape, 0.0f, false) : Tensor();
    const size_t batch = product(lead);
    if (batch == 0) return out;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d_k));
    const auto i64 = [](size_t x) { return static_cast<int64_t>(x); };
    const int64_t qs[3] = {i64(s_q * d_k), 0, i64(d_k)}, ks[3] = {i64(s_k * d_k), 0, i64(d_k)};
    const int64_t vs[3] = {i64(s_k * d_v), 0, i64(d_v)}, os[3] = {i64(s_q * d_v), 0, i64(d_v)};
    {
        const size_t ws_bytes = attention_weights ? 0
                                                  : b200_attention_any_workspace(i64(batch), 1, i64(s_q), i64(s_k),
                                                                                 i64(d_k), i64(d_v), 0);
        void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
        check_b200(b200_attention_any_f32(impl_of(q)->storage.device(), impl_of(k)->storage.device(),
                                          impl_of(v)->storage.device(), pm, impl_of(out)->storage.device_write(),
                                          attention_weights ? impl_of(weights)->storage.device_write() : nullptr,
                                          i64(batch), 1, i64(s_q), i64(s_k), i64(d_k), i64(d_v), qs, ks, vs, os, scale,
                                          current_precision(), ws, ws_bytes, nullptr),
                   "scaled_dot_product_attention");
    }
    if (attention_weights) *attention_weights = weights;
    if (tracked) {
        attach_attention_backward(out, q, k, v, mask_keep, mask != nullptr, batch, 1, s_q, s_k, d_k, d_v, qs, ks, vs,
                                  os, scale);
    }
    return out;
}

Tensor multi_head_attention_core(const Tensor& query_, const Tensor& key_, const Tensor& value_,
                                 size_t num_heads, const Tensor* mask) {
    for (const Tensor* t : {&query_, &key_, &value_}) {
        if (t->ndim() != 3) {
            throw std::invalid_argument("MultiHeadAttention expects (batch, seq, d_model), received " +
                                        t->shape_str() + ".");
        }
    }
    const size_t batch = query_.shape()[0], s_q = query_.shape()[1], d_model = query_.shape()[2];
    if (num_heads == 0 || d_model % num_heads != 0 || value_.shape()[2] % num_heads != 0) {
        throw std::invalid_argument("d_model must be divisible by num_heads.");
    }
    if (key_.shape()[0] != batch || value_.shape()[0] != batch || key_.shape()[2] != d_model ||
        key_.shape()[1] != value_.shape()[1]) {
        throw std::invalid_argument("query, key and value need the same batch, key/value the same length and "
                                    "query/key the same width.");
    }
    const bool tracked = attention_tracked(query_, key_, value_);
    const Tensor q = contiguous(query_), k = contiguous(key_), v = contiguous(value_);
    const size_t s_k = k.shape()[1], d_k = d_model / num_heads, dv_model = v.shape()[2], d_v = dv_model / num_heads;
    Tensor mask_keep;
    const float* pm = mask_pointer(mask, s_q, s_k, &mask_keep);
    Tensor out({batch, s_q, dv_model}, 0.0f, tracked);
    if (batch == 0) return out;
    const auto i64 = [](size_t x) { return static_cast<int64_t>(x); };
    const int64_t qs[3] = {i64(s_q * d_model), i64(d_k), i64(d_model)};
    const int64_t ks[3] = {i64(s_k * d_model), i64(d_k), i64(d_model)};
    const int64_t vs[3] = {i64(s_k * dv_model), i64(d_v), i64(dv_model)};
    const int64_t os[3] = {i64(s_q * dv_model), i64(d_v), i64(dv_model)};
    const float scale = 1.0f / std::sqrt(static_cast<float>(d_k));
    {
        const size_t ws_bytes = b200_attention_any_workspace(i64(batch), i64(num_heads), i64(s_q), i64(s_k), i64(d_k),
                                                             i64(d_v), 0);
        void* ws = ws_bytes ? g_scratch.get(ws_bytes) : nullptr;
        check_b200(b200_attention_any_f32(impl_of(q)->storage.device(), impl_of(k)->storage.device(),
                                          impl_of(v)->storage.device(), pm, impl_of(out)->storage.device_write(),
                                          nullptr, i64(batch), i64(num_heads), i64(s_q), i64(s_k), i64(d_k), i64(d_v),
                                          qs, ks, vs, os, scale, current_precision(), ws, ws_bytes, nullptr),
                   "multi_head_attention_core");
    }
    if (tracked) {
        attach_attention_backward(out, q, k, v, mask_keep, mask != nullptr, batch, num_heads, s_q, s_k, d_k, d_v, qs,
                                  ks, vs, os, scale);
    }
    return out;
}

}  // namespace nn

// ------------------------------------------------------------------------------- load_tensors
std::vector<std::pair<std::string, Tensor>> load_tensors(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Cannot open " + path + ".");
    std::vector<char> raw((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    size_t off = 0;
    auto need = [&](size_t n) {
        if (off + n > raw.size()) throw std::runtime_error(path + ": truncated file.");
    };
    auto u32 = [&]() {
        need(4);
        uint32_t v;
        std::memcpy(&v, raw.data() + off, 4);
        off += 4;
        return v;
    };
    need(8);
    if (std::memcmp(raw.data(), "CPPAIENG", 8) != 0) throw std::runtime_error(path + ": bad signature.");
    off = 8;
    if (u32() != 1) throw std::runtime_error(path + ": unsupported version.");
    const uint32_t count = u32();
    std::vector<std::pair<std::string, Tensor>> out;
    for (uint32_t t = 0; t < count; ++t) {
        const uint32_t nlen = u32();
        need(nlen);
        std::string name(raw.data() + off, nlen);
        off += nlen;
        const uint32_t nd = u32();
        if (nd > 8) throw std::runtime_error(path + ": implausible rank.");
        std::vector<size_t> shape(nd);
        size_t n = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            need(8);
            uint64_t v;
            std::memcpy(&v, raw.data() + off, 8);
            off += 8;
            if (v != 0 && n > (raw.size() / 4) / v) throw std::runtime_error(path + ": size overflow.");
            shape[d] = static_cast<size_t>(v);
            n *= shape[d];
        }
        need(n * 4);
        std::vector<float> data(n);
        std::memcpy(data.data(), raw.data() + off, n * 4);
        off += n * 4;
        out.emplace_back(std::move(name), Tensor(shape, data));
    }
    return out;
}

}  // namespace engine
