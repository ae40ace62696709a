// C++17 host side of the B200 matmul path: the slice of the reference engine's public
// surface that its matrix product lives behind, re-stated over the C ABI in
// include/b200_gemm.h.  Same names, argument meaning and error behaviour as the reference:
//
//   engine::manual_seed / Tensor::rand / Tensor::randn    src/tensor.cpp:24-31, 117-135
//   engine::Storage  (host vector + lazy device mirror)   include/engine/detail/storage.hpp:99-117
//   engine::cuda::ops::matmul (the device seam)           include/engine/detail/cuda_ops.hpp:46-47
//   engine::cuda::transfer_stats / kernels_launched       include/engine/cuda.hpp:79-81, 209-218
//   engine::Tensor::matmul / transpose / reshape /        include/engine/tensor.hpp:157-198,
//           backward / grad                               src/tensor_ops.cpp:475-588
//   engine::nn::linear / conv2d / attention               the forward bodies of Linear (src/nn.cpp:101-130),
//                                                         Conv2d (src/conv.cpp:280-338) and
//                                                         scaled_dot_product_attention / MultiHeadAttention
//                                                         (src/transformer.cpp:279-304, 332-357), each as
//                                                         ONE kernel
//
// What differs, on purpose: there is no CPU loop (ops::matmul never returns false — it throws
// when the device cannot run the product), transpose() is a zero-copy view that the product
// consumes as a layout flag instead of a materialised buffer, and the backward pass calls the
// transposed forms directly.
#ifndef ENGINE_B200_HPP
#define ENGINE_B200_HPP

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace engine {

void manual_seed(uint64_t seed);

// A tensor's buffer and which side of the bus holds the valid copy.  Invariant: at least one
// of the two copies is valid at all times.
class Storage {
public:
    Storage();
    Storage(size_t count, float fill);
    explicit Storage(std::vector<float> values);

    size_t size() const { return buf_->count; }
    bool empty() const { return buf_->count == 0; }

    const std::vector<float>& host() const;  // downloads if the host copy is stale
    std::vector<float>& host_mut();          // same, and marks the device copy stale

    const float* device() const;  // uploads if the device copy is stale
    float* device_mut();          // same, and marks the host copy stale
    float* device_write();        // allocates without uploading; the kernel overwrites all of it
    void revert_device_write();   // undoes a device_write() whose kernel never launched
    bool resident_on_device() const { return buf_->device_valid; }

    Storage clone() const;  // independent copy that stays on whichever side the values live
    Storage share() const;  // second handle on the same buffer (what makes reshape a view)
    bool shares_with(const Storage& other) const { return buf_ == other.buf_; }

private:
    struct Buffer {
        std::vector<float> host;
        size_t count = 0;
        float fill = 0.0f;
        float* device = nullptr;
        bool host_valid = true;
        bool device_valid = false;
        bool reverted_host_valid = true;
        ~Buffer();
    };
    void materialise() const;
    void ensure_device_buffer() const;
    std::shared_ptr<Buffer> buf_;
};

namespace cuda {

bool available();
void synchronize();

struct TransferStats {
    size_t to_device_bytes = 0;
    size_t to_host_bytes = 0;
    size_t to_device_count = 0;
    size_t to_host_count = 0;
};
TransferStats transfer_stats();
void reset_transfer_stats();
size_t kernels_launched();

// Reduced precision is opt-in and never selected automatically (include/engine/cuda.hpp:153-177).
enum class MatmulKernel { Auto, TensorCore };
void set_matmul_kernel(MatmulKernel kernel);
MatmulKernel matmul_kernel();

// Throws std::runtime_error if a bounded device-side wait ran out in an earlier launch.
void check_device_status();

namespace ops {

// out = a x b + beta * out, batched; an unbatched operand is reused for every batch element.
// Returns true when the device did the work.  It always does, or throws std::runtime_error:
// there is no CPU path for the caller to fall back to.
bool matmul(const Storage& a, const Storage& b, Storage& out, size_t batch, size_t rows,
            size_t inner_dim, size_t cols, bool a_batched, bool b_batched, float beta = 0.0f);

// The same with operands that are stored transposed (a as inner_dim x rows, b as cols x
// inner_dim per batch element).  No reference counterpart: the reference materialises the
// transpose first (src/tensor_ops.cpp:576, :581).
bool matmul_ex(const Storage& a, const Storage& b, Storage& out, size_t batch, size_t rows,
               size_t inner_dim, size_t cols, bool a_batched, bool b_batched, bool a_transposed,
               bool b_transposed, float beta = 0.0f);

}  // namespace ops
}  // namespace cuda

struct TensorImpl;

class Tensor {
public:
    Tensor();
    explicit Tensor(const std::vector<size_t>& shape, float fill_value = 0.0f,
                    bool requires_grad = false);
    Tensor(const std::vector<size_t>& shape, const std::vector<float>& data,
           bool requires_grad = false);

    static Tensor zeros(const std::vector<size_t>& shape, bool requires_grad = false);
    static Tensor ones(const std::vector<size_t>& shape, bool requires_grad = false);
    static Tensor rand(const std::vector<size_t>& shape, float min_val = -1.0f, float max_val = 1.0f,
                       bool requires_grad = false);
    static Tensor randn(const std::vector<size_t>& shape, float mean = 0.0f, float stddev = 1.0f,
                        bool requires_grad = false);

    bool requires_grad() const;
    void set_requires_grad(bool requires_grad);
    Tensor grad() const;
    bool has_grad() const;
    void zero_grad();
    void add_grad(const Tensor& g);
    void backward();
    void backward(const Tensor& grad_output);

    const std::vector<size_t>& shape() const;
    size_t ndim() const;
    size_t size() const;
    std::string shape_str() const;

    // The elements in logical row-major order.  Reading downloads if the values live on the
    // device; on a transposed view the copy is made in logical order.
    std::vector<float> to_vector() const;
    float at(size_t flat_index) const;
    float operator()(size_t row, size_t col) const;

    // (M, K) x (K, N) -> (M, N); (B..., M, K) x (B..., K, N) -> (B..., M, N); a 2-D operand is
    // shared by every matrix of the other's batch.  Throws std::invalid_argument exactly where
    // the reference does (src/tensor_ops.cpp:476-503).
    Tensor matmul(const Tensor& other) const;
    // Swaps the last two axes.  A view: no data moves; a product consumes it as a layout flag.
    Tensor transpose() const;
    // Same elements, new shape (a view of a non-transposed tensor, a copy of a transposed one).
    Tensor reshape(const std::vector<size_t>& new_shape) const;
    Tensor detach() const;

    bool resident_on_device() const;
    bool is_transposed_view() const;

private:
    explicit Tensor(std::shared_ptr<TensorImpl> impl);
    std::shared_ptr<TensorImpl> impl_;
    friend struct TensorImpl;
};

namespace nn {

// include/engine/conv.hpp:12-26.
struct Window2d {
    size_t kernel_h;
    size_t kernel_w;
    size_t stride = 1;
    size_t padding = 0;

    Window2d(size_t k) : kernel_h(k), kernel_w(k) {}
    Window2d(size_t kh, size_t kw, size_t s = 1, size_t p = 0)
        : kernel_h(kh), kernel_w(kw), stride(s), padding(p) {}
    size_t out_h(size_t in_h) const { return (in_h + 2 * padding - kernel_h) / stride + 1; }
    size_t out_w(size_t in_w) const { return (in_w + 2 * padding - kernel_w) / stride + 1; }
    void validate(size_t in_h, size_t in_w) const;  // throws std::invalid_argument
};

// Linear::forward: input (..., in) x weight (in, out) + bias (out), optionally followed by ReLU
// (the feed-forward ff1(x).relu(), src/transformer.cpp:413) — product, broadcast add and
// activation in one kernel.  Gradients flow to input, weight and bias when relu is false (the
// bias gradient is the column sum of the incoming gradient, taken as a product with a row of
// ones); with relu the result does not track gradients.
Tensor linear(const Tensor& input, const Tensor& weight, const Tensor* bias = nullptr, bool relu = false);

// Conv2d::forward on (N, C, H, W) with weight (outC, C, kH, kW) and optional bias (outC): one
// implicit-GEMM kernel; its backward is one call that fills the three gradients without a
// column matrix (b200_conv2d_backward_f32).
Tensor conv2d(const Tensor& input, const Tensor& weight, const Tensor* bias, const Window2d& window);

// scaled_dot_product_attention over the leading (batch, head) axes: softmax(Q K^T / sqrt(d_k) +
// mask) V in one kernel; attention_weights, if given, receives the softmax output.  Gradients flow
// to query, key and value through ONE backward kernel that recomputes the weights.  Any size, like
// the reference's: heads beyond the fused kernels' tiles (S_q, S_k <= 128 and d_k, d_v <= 64 forward;
// the tiles of a head in one CTA's shared memory backward — S = 64 with d <= 64 fits, S = 128 does
// not) run composed on the device (b200_attention_any_f32: products with the scale and the mask in
// their store, owned softmax row kernels), never on the host.
Tensor scaled_dot_product_attention(const Tensor& query, const Tensor& key, const Tensor& value,
                                    const Tensor* mask = nullptr, Tensor* attention_weights = nullptr);

// The middle of MultiHeadAttention::forward: the three projections (B, S, d_model) in, the merged
// context (B, S, d_model) out; heads are split and merged by addressing, not by permute copies.
Tensor multi_head_attention_core(const Tensor& query, const Tensor& key, const Tensor& value,
                                 size_t num_heads, const Tensor* mask = nullptr);

}  // namespace nn

// Reads every tensor of a file in the reference's documented container format
// (include/engine/serialize.hpp:12-31: "CPPAIENG", u32 version, u32 count, then per tensor
// u32 name length, name, u32 ndim, u64 dims, f32 data; little-endian).
std::vector<std::pair<std::string, Tensor>> load_tensors(const std::string& path);

}  // namespace engine

#endif  // ENGINE_B200_HPP
