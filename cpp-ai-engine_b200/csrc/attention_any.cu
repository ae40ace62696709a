// scaled_dot_product_attention of any size (include/b200_gemm.h: b200_attention_any_f32 and its
// backward).  Heads whose tiles fit one CTA run in the fused kernels (attention_kernel.cuh,
// attention_bwd_kernel.cuh); every other shape runs here, composed on the device exactly as the
// reference composes it (src/transformer.cpp:279-304) but without its transposes and separate
// element-wise passes:
//   scores  = one batched product q x k^T with `* scale` and `+ mask` in its store (transB on k as stored)
//   weights = softmax over the rows, an owned kernel in the reference's order (row maximum, exp,
//             sum, divide: Tensor::softmax, src/tensor_ops.cpp:621-647)
//   out     = one batched product weights x v
// and for the gradients (the backward lambdas of those nodes, src/tensor_ops.cpp:570-585, 649-668):
//   dW = dout x v^T,  dv = W^T x dout,  dS = W o (dW - rowsum(dW o W)) * scale,  dq = dS x k,  dk = dS^T x q
// as four batched products through the transposed forms and one owned row kernel.
// The (batch, heads, S_q, S_k) weights live in caller workspace; nothing is allocated here.
#include "../../include/b200_gemm.h"

#include <cuda_runtime.h>

#include <cstdint>

namespace b200 {
void count_launch();                                                                          // gemm_sm100.cu
bool attention_backward_fits_one_cta(int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v);  // gemm_sm100.cu
}

namespace {

constexpr int kRowWarps = 8;  // rows per block: one warp each

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// In place over `rows` rows of `cols` floats: x <- exp(x - max(x)) / sum(exp(x - max(x))).
// One warp per row; lane j takes columns j, j + 32, ...; the row sum is the lanes' partial sums
// (each in ascending column order) added in a fixed shuffle tree — the same bits on every run.
__global__ void softmax_rows_kernel(float* __restrict__ x, long long rows, int cols) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    float* p = x + row * cols;
    float m = -INFINITY;
    for (int j = lane; j < cols; j += 32) m = fmaxf(m, p[j]);
    m = warp_max(m);
    float s = 0.f;
    for (int j = lane; j < cols; j += 32) {
        const float e = expf(p[j] - m);
        p[j] = e;
        s += e;
    }
    s = warp_sum(s);
    for (int j = lane; j < cols; j += 32) p[j] = p[j] / s;
}

// In place over d (rows x cols), with the softmax output y: d <- y o (d - rowsum(d o y)) * scale
// (Tensor::softmax's backward, src/tensor_ops.cpp:649-668, then the scalar multiply's).
__global__ void softmax_backward_rows_kernel(float* __restrict__ d, const float* __restrict__ y, long long rows,
                                             int cols, float scale) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    float* pd = d + row * cols;
    const float* py = y + row * cols;
    float dot = 0.f;
    for (int j = lane; j < cols; j += 32) dot += pd[j] * py[j];
    dot = warp_sum(dot);
    for (int j = lane; j < cols; j += 32) pd[j] = (py[j] * (pd[j] - dot)) * scale;
}

struct Layout {
    int64_t groups;     // launches: batch elements that cannot be folded into one strided batch
    int64_t per_group;  // matrices per launch
    int64_t q[2], k[2], v[2], o[2];  // (group stride, matrix stride) in floats
};

// Matrix (b, h) of a tensor lies at b * s[0] + h * s[1].  When b * s[0] + h * s[1] == (b * heads + h) * s[1]
// for all four tensors the whole (batch x heads) set is ONE strided batch; otherwise one launch per batch
// element walks its heads.
Layout fold(int64_t batch, int64_t heads, const int64_t* qs, const int64_t* ks, const int64_t* vs,
            const int64_t* os) {
    Layout l{};
    const bool one = heads == 1;
    const bool all = !one && qs[0] == heads * qs[1] && ks[0] == heads * ks[1] && vs[0] == heads * vs[1] &&
                     os[0] == heads * os[1];
    if (one || all) {
        l.groups = 1;
        l.per_group = batch * heads;
        const int idx = one ? 0 : 1;
        l.q[0] = l.k[0] = l.v[0] = l.o[0] = 0;
        l.q[1] = qs[idx], l.k[1] = ks[idx], l.v[1] = vs[idx], l.o[1] = os[idx];
    } else {
        l.groups = batch;
        l.per_group = heads;
        l.q[0] = qs[0], l.k[0] = ks[0], l.v[0] = vs[0], l.o[0] = os[0];
        l.q[1] = qs[1], l.k[1] = ks[1], l.v[1] = vs[1], l.o[1] = os[1];
    }
    return l;
}

int check_args(int64_t batch, int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
               const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os) {
    if (batch < 0 || heads <= 0 || s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return B200_EINVAL;
    if (qs == nullptr || ks == nullptr || vs == nullptr || os == nullptr) return B200_EINVAL;
    if (qs[2] < d_k || ks[2] < d_k || vs[2] < d_v || os[2] < d_v) return B200_EINVAL;
    if (s_k > 0x7fffffffll || batch * heads > 0x7fffffffll) return B200_ERANGE;
    return 0;
}

bool fused_forward_fits(int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v) {
    return s_q <= 128 && s_k <= 128 && d_k <= 64 && d_v <= 64;
}

// weights (per matrix s_q x s_k, contiguous) <- softmax(q x k^T * scale + mask), for one group
int scores_and_softmax(const float* q, const float* k, const float* mask, float* w, const Layout& l, int64_t s_q,
                       int64_t s_k, int64_t d_k, int64_t q_ld, int64_t k_ld, float scale, int precision,
                       cudaStream_t stream) {
    b200_epilogue ep{};
    ep.addend = mask;
    ep.ld_addend = s_k;
    int rc = b200_gemm_f32_fused(q, k, w, l.per_group, s_q, s_k, d_k, 0, 1, q_ld, k_ld, s_k, l.q[1], l.k[1],
                                 s_q * s_k, scale, 0.0f, precision, mask ? &ep : nullptr, nullptr, 0, stream);
    if (rc) return rc;
    const long long rows = static_cast<long long>(l.per_group) * s_q;
    const unsigned blocks = static_cast<unsigned>((rows + kRowWarps - 1) / kRowWarps);
    softmax_rows_kernel<<<blocks, kRowWarps * 32, 0, stream>>>(w, rows, static_cast<int>(s_k));
    b200::count_launch();
    return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

size_t b200_attention_any_workspace(int64_t batch, int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k,
                                    int64_t d_v, int backward) {
    if (batch <= 0 || heads <= 0 || s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return 0;
    const size_t one = static_cast<size_t>(batch) * heads * s_q * s_k * sizeof(float);
    if (!backward) return fused_forward_fits(s_q, s_k, d_k, d_v) ? 0 : one;
    // weights and their gradient, both (batch, heads, s_q, s_k)
    return b200::attention_backward_fits_one_cta(s_q, s_k, d_k, d_v) ? 0 : 2 * one;
}

int b200_attention_any_f32(const float* q, const float* k, const float* v, const float* mask, float* out,
                           float* weights, int64_t batch, int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k,
                           int64_t d_v, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3], float scale, int precision,
                           void* workspace, size_t workspace_bytes, void* stream_) {
    if (int rc = check_args(batch, heads, s_q, s_k, d_k, d_v, q_strides, k_strides, v_strides, out_strides)) return rc;
    if (fused_forward_fits(s_q, s_k, d_k, d_v))
        return b200_attention_f32_strided(q, k, v, mask, out, weights, batch, heads, s_q, s_k, d_k, d_v, q_strides,
                                          k_strides, v_strides, out_strides, scale, precision, stream_);
    if (batch == 0) return B200_OK;
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return B200_EINVAL;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t need = static_cast<size_t>(batch) * heads * s_q * s_k * sizeof(float);
    float* w = weights;  // the caller's attention_weights buffer doubles as the scratch
    if (w == nullptr) {
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15u))
            return B200_ENOSPACE;
        w = static_cast<float*>(workspace);
    }
    const Layout l = fold(batch, heads, q_strides, k_strides, v_strides, out_strides);
    const int64_t wg = l.per_group * s_q * s_k;
    for (int64_t g = 0; g < l.groups; ++g) {
        float* wgp = w + g * wg;
        int rc = scores_and_softmax(q + g * l.q[0], k + g * l.k[0], mask, wgp, l, s_q, s_k, d_k, q_strides[2],
                                    k_strides[2], scale, precision, stream);
        if (rc) return rc;
        rc = b200_gemm_f32(wgp, v + g * l.v[0], out + g * l.o[0], l.per_group, s_q, d_v, s_k, 0, 0, s_k, v_strides[2],
                           out_strides[2], s_q * s_k, l.v[1], l.o[1], 1.0f, 0.0f, precision, nullptr, 0, stream);
        if (rc) return rc;
    }
    return B200_OK;
}

int b200_attention_backward_any_f32(const float* q, const float* k, const float* v, const float* mask,
                                    const float* dout, float* dq, float* dk, float* dv, int64_t batch,
                                    int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
                                    const int64_t q_strides[3], const int64_t k_strides[3],
                                    const int64_t v_strides[3], const int64_t out_strides[3], float scale,
                                    float beta, int precision, void* workspace, size_t workspace_bytes,
                                    void* stream_) {
    if (int rc = check_args(batch, heads, s_q, s_k, d_k, d_v, q_strides, k_strides, v_strides, out_strides)) return rc;
    if (b200::attention_backward_fits_one_cta(s_q, s_k, d_k, d_v))
        return b200_attention_backward_f32_strided(q, k, v, mask, dout, dq, dk, dv, batch, heads, s_q, s_k, d_k, d_v,
                                                   q_strides, k_strides, v_strides, out_strides, scale, beta,
                                                   precision, stream_);
    int rc = 0;
    if (batch == 0) return B200_OK;
    if (q == nullptr || k == nullptr || v == nullptr || dout == nullptr) return B200_EINVAL;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t one = static_cast<size_t>(batch) * heads * s_q * s_k * sizeof(float);
    if (workspace == nullptr || workspace_bytes < 2 * one || (reinterpret_cast<uintptr_t>(workspace) & 15u))
        return B200_ENOSPACE;
    float* w_all = static_cast<float*>(workspace);
    float* d_all = w_all + one / sizeof(float);
    const Layout l = fold(batch, heads, q_strides, k_strides, v_strides, out_strides);
    const int64_t wg = l.per_group * s_q * s_k, mat = s_q * s_k;
    for (int64_t g = 0; g < l.groups; ++g) {
        float* w = w_all + g * wg;
        float* d = d_all + g * wg;
        const float* qg = q + g * l.q[0];
        const float* kg = k + g * l.k[0];
        const float* vg = v + g * l.v[0];
        const float* og = dout + g * l.o[0];
        // the attention weights again, with the forward's arithmetic
        rc = scores_and_softmax(qg, kg, mask, w, l, s_q, s_k, d_k, q_strides[2], k_strides[2], scale, precision, stream);
        if (rc) return rc;
        // dW = dout x v^T
        rc = b200_gemm_f32(og, vg, d, l.per_group, s_q, s_k, d_v, 0, 1, out_strides[2], v_strides[2], s_k, l.o[1],
                           l.v[1], mat, 1.0f, 0.0f, precision, nullptr, 0, stream);
        if (rc) return rc;
        // dv = W^T x dout
        if (dv != nullptr) {
            rc = b200_gemm_f32(w, og, dv + g * l.v[0], l.per_group, s_k, d_v, s_q, 1, 0, s_k, out_strides[2],
                               v_strides[2], mat, l.o[1], l.v[1], 1.0f, beta, precision, nullptr, 0, stream);
            if (rc) return rc;
        }
        if (dq == nullptr && dk == nullptr) continue;
        // dS = W o (dW - rowsum(dW o W)) * scale, in place over dW
        const long long rows = static_cast<long long>(l.per_group) * s_q;
        const unsigned blocks = static_cast<unsigned>((rows + kRowWarps - 1) / kRowWarps);
        softmax_backward_rows_kernel<<<blocks, kRowWarps * 32, 0, stream>>>(d, w, rows, static_cast<int>(s_k), scale);
        b200::count_launch();
        if ((rc = static_cast<int>(cudaGetLastError()))) return rc;
        // dq = dS x k
        if (dq != nullptr) {
            rc = b200_gemm_f32(d, kg, dq + g * l.q[0], l.per_group, s_q, d_k, s_k, 0, 0, s_k, k_strides[2],
                               q_strides[2], mat, l.k[1], l.q[1], 1.0f, beta, precision, nullptr, 0, stream);
            if (rc) return rc;
        }
        // dk = dS^T x q
        if (dk != nullptr) {
            rc = b200_gemm_f32(d, qg, dk + g * l.k[0], l.per_group, s_k, d_k, s_q, 1, 0, s_k, q_strides[2],
                               k_strides[2], mat, l.q[1], l.k[1], 1.0f, beta, precision, nullptr, 0, stream);
            if (rc) return rc;
        }
    }
    return B200_OK;
}

}  // extern "C"
