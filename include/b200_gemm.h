/* C ABI of the B200 (sm_100a) fp32 GEMM library — the drop-in for the reference engine's
 * matrix-product seam.
 *
 * The reference funnels every matrix product of the engine (Linear, attention, Conv2d via
 * im2col, and the autograd backward forms) through Tensor::matmul (src/tensor_ops.cpp:475-588),
 * which offers the work to one device entry point:
 *
 *     bool engine::cuda::ops::matmul(const Storage& a, const Storage& b, Storage& out,
 *                                    size_t batch, size_t rows, size_t inner_dim, size_t cols,
 *                                    bool a_batched, bool b_batched, float beta = 0.0f);
 *                                                   (include/engine/detail/cuda_ops.hpp:46-47,
 *                                                    implemented in src/cuda/kernels_matmul.cu:761-898)
 *
 * This header declares what a binding of that seam calls instead.  Plain pointers and sizes
 * only; every pointer is a DEVICE pointer unless the function name ends in _host.  Calls are
 * stream-ordered and never synchronise unless stated.  Return value: 0 on success, a negative
 * B200_E* code when the arguments were rejected (nothing was launched), a positive value for
 * a CUDA runtime error (cudaError_t) raised by the launch.
 *
 * Arithmetic: inputs and outputs are fp32.  Products run on the tcgen05 tensor cores in TF32
 * with the error-compensated three-product split ("3xTF32": a = a_hi + a_lo, b = b_hi + b_lo,
 * a*b ~ a_lo*b_hi + a_hi*b_lo + a_hi*b_hi) and partial sums are promoted to fp32 registers
 * every few k-steps, so results stay at fp32-level accuracy.  B200_PRECISION_TF32 is the
 * opt-in single-product mode (about 1e-3 relative error, like the reference's own
 * MatmulKernel::TensorCore, include/engine/cuda.hpp:153-177) and is never the default.
 *
 * Finite inputs only.  The reference's CPU loop skips every term whose A value is exactly zero
 * (src/tensor_ops.cpp:555), so it never forms 0 * Inf or 0 * NaN; for finite inputs the skip
 * changes nothing, and zeros in A give the same results here as there.  An infinite or NaN input,
 * however, makes every output that its row or column feeds non-finite here — NaN where the
 * reference may hold +-Inf (the split forms Inf - Inf), and also where the reference skipped the
 * term because the A value was zero and kept a finite result.  Outputs that the value does not
 * feed are unaffected.  Callers that may hold non-finite values must clean them first.
 *
 * Threads.  Like the reference's device layer (one dispatching thread, src/cuda/runtime.cu:159-160)
 * the library expects one thread per device to issue products.  Calls from several threads are
 * safe as far as the library's own state goes (first-use set-up is locked, and
 * b200_matmul_f32_host admits one call per device at a time), but b200_gemm_set_option changes
 * process-wide knobs without synchronisation: set options while no other thread is inside the
 * library.
 */
#ifndef B200_GEMM_H
#define B200_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_PRECISION_3XTF32 0 /* default: fp32-level accuracy */
#define B200_PRECISION_TF32 1   /* opt-in: one TF32 product per term */

#define B200_OK 0
#define B200_EINVAL (-1)    /* bad shape, stride, flag or null pointer */
#define B200_ERANGE (-2)    /* a dimension exceeds what the kernels index (2^31-1 rows/cols, 65535*... ) */
#define B200_ENOSPACE (-3)  /* workspace required but too small and no fallback possible */
#define B200_EDEVICE (-4)   /* no sm_100 device / driver entry point missing */
#define B200_ETIMEDOUT (-5) /* a device-side wait ran out (reported by b200_gemm_status) */

/* General form.  C[b] = alpha * op(A[b]) x op(B[b]) + beta * C[b] for b in [0, batch).
 * op(A) is M x K, op(B) is K x N, C is M x N; all matrices are row-major as stored:
 *   transA == 0: A stored M x K, element (i,k) at A[i*lda + k];  transA != 0: stored K x M.
 *   transB == 0: B stored K x N, element (k,j) at B[k*ldb + j];  transB != 0: stored N x K.
 * strideX is the element distance between consecutive batch matrices; 0 shares the operand
 * across the batch (the reference's a_batched / b_batched == false, src/tensor_ops.cpp:514-515).
 * The transposed forms replace the materialised Tensor::transpose() the reference performs
 * before its backward products (src/tensor_ops.cpp:576, :581) and in attention / Conv2d
 * (src/transformer.cpp:293, src/conv.cpp:322).
 * beta == 0 never reads C (it may hold anything, like Storage::device_write(),
 * src/storage.cpp:321-332).
 * workspace: device scratch for the deterministic split-K path (tall-skinny products); may be
 * NULL / 0, in which case the product runs unsplit.  Its contents need not be preserved.
 * stream: a cudaStream_t (NULL = the default stream). */
int b200_gemm_f32(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
                  int64_t K, int transA, int transB, int64_t lda, int64_t ldb, int64_t ldc,
                  int64_t strideA, int64_t strideB, int64_t strideC, float alpha, float beta,
                  int precision, void* workspace, size_t workspace_bytes, void* stream);

/* What the reference does in separate element-wise kernels right after a product, folded into
 * the product's own store (no reference counterpart as one call; the operations are
 * Linear's and Conv2d's bias broadcast add, src/nn.cpp:120-122 and src/conv.cpp:323; attention's
 * `* scale` then `+ mask`, src/transformer.cpp:292-297; the feed-forward ReLU,
 * src/transformer.cpp:413).  Applied in this order, each an fp32 operation on the fp32 result,
 * exactly as the separate kernels would:
 *     out = relu?( alpha * (op(A) x op(B)) + bias[col] + addend[row][col] + beta * out )
 * bias: N device floats or NULL.  addend: an M x N device matrix (leading dimension ld_addend >= N)
 * shared by every batch element, or NULL.  relu: 0 or 1. */
typedef struct b200_epilogue {
    const float* bias;
    const float* addend;
    int64_t ld_addend;
    int relu;
} b200_epilogue;

/* b200_gemm_f32 with the fused epilogue above (epilogue == NULL behaves like b200_gemm_f32). */
int b200_gemm_f32_fused(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
                        int64_t K, int transA, int transB, int64_t lda, int64_t ldb, int64_t ldc,
                        int64_t strideA, int64_t strideB, int64_t strideC, float alpha, float beta,
                        int precision, const b200_epilogue* epilogue, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Conv2d::forward as ONE kernel (src/conv.cpp:280-338 builds it from im2col, a product against
 * the transposed (out_c, K) weight view, a bias broadcast add and a (N, spatial, C) -> (N, C, H, W)
 * permute; src/cuda/kernels.cu:394-426 is the reference's im2col_gather kernel).  Implicit GEMM:
 * the column matrix is never written — the A tiles are gathered from x while they are loaded —
 * the weight is read as stored, and the store writes y in NCHW order with the bias (and an
 * optional ReLU) applied.
 * x: (n, c, h, w); weight: (out_c, c, kh, kw); bias: out_c values or NULL;
 * y: (n, out_c, oh, ow) with oh = (h + 2*pad - kh) / stride + 1, likewise ow.  All row-major. */
int b200_conv2d_forward_f32(const float* x, const float* weight, const float* bias, float* y,
                            int64_t n, int64_t c, int64_t h, int64_t w, int64_t out_c, int64_t kh,
                            int64_t kw, int64_t stride, int64_t pad, int relu, int precision,
                            void* stream);

/* The backward pass of Conv2d, without the column matrix, its transpose or col2im's scatter.
 * The reference derives it through autograd from the forward's pieces (src/conv.cpp:280-338):
 * the product's backward lambda (src/tensor_ops.cpp:570-585) materialises cols^T and W and runs
 * two products, im2col's backward scatters dCols with col2im (src/conv.cpp:152-222, 236-257;
 * its kernel: src/cuda/kernels.cu:428-466), the bias takes the column sums of the gradient.
 * Here, each optional (pass NULL to skip):
 *   dweight (out_c, c, kh, kw) = dOut^T x cols  — ONE implicit-GEMM kernel that gathers both operands
 *           (dy and the im2col view of x) while loading, contracting over the n*oh*ow output
 *           positions, split over the SMs with a deterministic reduction (second small kernel);
 *   dx (n, c, h, w)             — ONE gather kernel: dx[n][c][ih][iw] = sum over (o, i, j) of
 *           dy[n][o][(ih+pad-i)/stride][(iw+pad-j)/stride] * weight[o][c][i][j] (exact divisions
 *           that land inside dy only), stored in NCHW order;
 *   dbias (out_c)               — per-channel sums of dy.
 * beta = 0 overwrites the three gradients, beta = 1 accumulates into them (Tensor::add_grad,
 * src/tensor.cpp:168-203).  x may be NULL if dweight is, weight may be NULL if dx is.
 * workspace: b200_conv2d_backward_workspace() bytes, 16-byte aligned, for the weight gradient's
 * partial sums; without it that kernel runs unsplit (correct, slower). */
size_t b200_conv2d_backward_workspace(int64_t n, int64_t c, int64_t h, int64_t w, int64_t out_c, int64_t kh,
                                      int64_t kw, int64_t stride, int64_t pad);
int b200_conv2d_backward_f32(const float* x, const float* weight, const float* dy, float* dx,
                             float* dweight, float* dbias, int64_t n, int64_t c, int64_t h, int64_t w,
                             int64_t out_c, int64_t kh, int64_t kw, int64_t stride, int64_t pad,
                             float beta, int precision, void* workspace, size_t workspace_bytes,
                             void* stream);

/* scaled_dot_product_attention as ONE kernel (src/transformer.cpp:279-304 composes it from a batched
 * product against a materialised K^T, `* scale`, `+ mask`, Tensor::softmax, src/tensor_ops.cpp:621-647,
 * and a second batched product; its softmax kernels are src/cuda/kernels.cu:835-895):
 *     out[b] = softmax(q[b] x k[b]^T * scale + mask) x v[b]
 * One CTA per batch element (= per head); the scores live in tensor memory and registers only, two
 * threads per query row, and are normalised in the reference's order (max, exp, fp32 sum over the
 * columns in ascending order, divide).  q: (batch, s_q, d_k); k: (batch, s_k, d_k); v: (batch, s_k, d_v); mask: (s_q, s_k)
 * additive and shared by every batch element, or NULL; out: (batch, s_q, d_v); weights: optional
 * (batch, s_q, s_k) copy of the softmax output (the reference's attention_weights), or NULL.
 * Limits: s_q <= 128, s_k <= 128, d_k <= 64, d_v <= 64 (B200_ERANGE beyond; b200_attention_any_f32 takes every size). */
int b200_attention_f32(const float* q, const float* k, const float* v, const float* mask, float* out,
                       float* weights, int64_t batch, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
                       float scale, int precision, void* stream);

/* b200_attention_f32 on the head-split VIEW of the projections, writing the merged layout
 * (MultiHeadAttention::forward, src/transformer.cpp:339-357, materialises
 * reshape(B, S, H, hd).permute(0, 2, 1, 3) for q, k and v and the inverse permute for the result;
 * here both are addressing).  There are batch * heads matrices; element (row, e) of matrix (b, h) of
 * q lies at q[b * q_strides[0] + h * q_strides[1] + row * q_strides[2] + e] (strides in floats, the
 * last axis contiguous), likewise k, v and out.  For projections stored (B, S, H * hd):
 * strides = {S * H * hd, hd, H * hd}.  weights, if given, is (batch * heads, s_q, s_k) contiguous.
 * Same limits and errors as b200_attention_f32. */
int b200_attention_f32_strided(const float* q, const float* k, const float* v, const float* mask,
                               float* out, float* weights, int64_t batch, int64_t heads, int64_t s_q,
                               int64_t s_k, int64_t d_k, int64_t d_v, const int64_t q_strides[3],
                               const int64_t k_strides[3], const int64_t v_strides[3],
                               const int64_t out_strides[3], float scale, int precision, void* stream);

/* The backward pass of the attention core as ONE kernel.  The reference's autograd runs the
 * backward of each node of scaled_dot_product_attention (src/transformer.cpp:279-304): two product
 * backwards with materialised transposes (src/tensor_ops.cpp:570-585), the softmax backward
 * dX_ij = y_ij (dY_ij - sum_k dY_ik y_ik) (src/tensor_ops.cpp:649-668; kernel src/cuda/kernels.cu),
 * the scalar multiply's and the transpose's.  Here, per head, the scores are recomputed (same
 * arithmetic as the forward kernel), and
 *     dW = dout x v^T,  dv = W^T x dout,  dS = W o (dW - rowsum(dW o W)) * scale,
 *     dq = dS x k,      dk = dS^T x q
 * run as five tensor-core products around the row arithmetic; nothing of size (S_q, S_k) reaches
 * global memory.  dq, dk, dv (any may be NULL) are addressed like q, k, v; dout like the forward's
 * out; beta = 0 overwrites, beta = 1 accumulates (Tensor::add_grad, src/tensor.cpp:168-203).
 * Limits: those of the forward kernel AND the tiles of a head must fit one CTA's shared memory
 * (S = 64 with d <= 64 does; S = 128 does not): B200_ERANGE otherwise — b200_attention_backward_any_f32
 * takes every size. */
int b200_attention_backward_f32(const float* q, const float* k, const float* v, const float* mask,
                                const float* dout, float* dq, float* dk, float* dv, int64_t batch,
                                int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v, float scale, float beta,
                                int precision, void* stream);
int b200_attention_backward_f32_strided(const float* q, const float* k, const float* v, const float* mask,
                                        const float* dout, float* dq, float* dk, float* dv, int64_t batch,
                                        int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
                                        const int64_t q_strides[3], const int64_t k_strides[3],
                                        const int64_t v_strides[3], const int64_t out_strides[3],
                                        float scale, float beta, int precision, void* stream);

/* scaled_dot_product_attention and its backward for heads of ANY size (the reference's take any S and d,
 * src/transformer.cpp:279-304).  Same arguments as the _strided forms plus a workspace.  Heads that fit the
 * fused kernels run there and need no workspace.  Every other shape runs composed on the device, as the
 * reference composes it but without its transposes and separate element-wise passes: the scores as one
 * batched product on k as stored with `* scale` and `+ mask` in its store, an owned row-softmax kernel in
 * the reference's order (maximum, exp, sum, divide: src/tensor_ops.cpp:621-647), weights x v; for the
 * gradients the weights again, dW = dout x v^T, dv = W^T x dout, the softmax backward
 * dS = W o (dW - rowsum(dW o W)) * scale as one row kernel (src/tensor_ops.cpp:649-668), dq = dS x k,
 * dk = dS^T x q.  When (batch, heads) fold into one stride the products are single launches over
 * batch * heads matrices, otherwise one launch per batch element over its heads.
 * workspace: b200_attention_any_workspace() bytes (0 when the fused kernel takes the shape), 16-byte
 * aligned; too little is B200_ENOSPACE.  The forward uses `weights`, when given, instead of workspace. */
size_t b200_attention_any_workspace(int64_t batch, int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k,
                                    int64_t d_v, int backward);
int b200_attention_any_f32(const float* q, const float* k, const float* v, const float* mask, float* out,
                           float* weights, int64_t batch, int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k,
                           int64_t d_v, const int64_t q_strides[3], const int64_t k_strides[3],
                           const int64_t v_strides[3], const int64_t out_strides[3], float scale, int precision,
                           void* workspace, size_t workspace_bytes, void* stream);
int b200_attention_backward_any_f32(const float* q, const float* k, const float* v, const float* mask,
                                    const float* dout, float* dq, float* dk, float* dv, int64_t batch,
                                    int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
                                    const int64_t q_strides[3], const int64_t k_strides[3],
                                    const int64_t v_strides[3], const int64_t out_strides[3], float scale,
                                    float beta, int precision, void* workspace, size_t workspace_bytes,
                                    void* stream);

/* Bytes of workspace with which b200_gemm_f32 can use split-K for this shape (0 when it would
 * not split).  Replaces the reference's scratch_buffer for its split-K partials
 * (src/cuda/kernels_matmul.cu:866-893, src/cuda/kernels.cu:593-604). */
size_t b200_gemm_f32_workspace(int64_t batch, int64_t M, int64_t N, int64_t K);

/* What b200_gemm_f32 would do with TMA-legal operands of this shape and `workspace_bytes` of
 * workspace: the tile width, whether tiles run on CTA pairs, the deterministic K-split (1 = none;
 * as deep as the workspace holds, never deeper than the planner wants), the K-split of a mostly
 * empty last wave, the kernels one call launches and the workspace bytes it writes.  Works
 * without a device (148 SMs are assumed then).  The counterpart of the reference's
 * resolve_matmul_kernel (src/cuda/runtime.cu:293-298) made visible to callers and tests. */
typedef struct b200_plan_info {
    int tile_n, pair, split_k, tail_tiles, tail_split, kernels;
    size_t workspace_used;
} b200_plan_info;
int b200_gemm_f32_plan(int64_t batch, int64_t M, int64_t N, int64_t K, size_t workspace_bytes,
                       b200_plan_info* out);

/* The reference seam itself, argument for argument (include/engine/detail/cuda_ops.hpp:46-47):
 * out = a x b + beta * out over `batch` contiguous row-major matrices, a is (rows x inner_dim),
 * b is (inner_dim x cols); an unbatched operand is reused for every batch element. */
int b200_matmul_f32(const float* a, const float* b, float* out, size_t batch, size_t rows,
                    size_t inner_dim, size_t cols, int a_batched, int b_batched, float beta,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Same product from HOST buffers: uploads a and b, runs the kernel, downloads out, and returns
 * after the result is on the host — the whole cost a caller holding host tensors pays, as when
 * the reference's Storage uploads stale operands and a later data() downloads the result
 * (src/storage.cpp:281-307).  Device staging buffers are cached per device between calls.
 * A large single product (rows, cols >= 4096) is run as a wavefront of blocks whose uploads,
 * kernels and downloads overlap on streams of their own; pass page-locked host buffers to get the
 * overlap (pageable ones work, serialised). */
int b200_matmul_f32_host(const float* a, const float* b, float* out, size_t batch, size_t rows,
                         size_t inner_dim, size_t cols, int a_batched, int b_batched, float beta);

/* N-column-sharded product for large GEMMs on g GPUs of one node (no reference counterpart:
 * the reference is single-device, src/cuda/runtime.cu:83).  This rank computes columns
 * [col0, col0 + cols) of C = A x B from its full A (M x K, lda) and the same columns of the full
 * B (K x N, ldb), and stores every finished tile at the same position of each of the
 * n_dest row-major M x N buffers in dest[] (host array of DEVICE pointers: this rank's own C
 * first and, for the fused all-gather, the peers' C mapped into this process): the worker warps
 * store each tile into dest[0], two otherwise idle warps copy it on to dest[1..].  Plain stores over
 * NVLink; no multicast.  This is the building block of b200_gemm_f32_sharded, which adds the
 * barriers: called directly, the caller orders it across ranks itself — before (a peer must be done
 * reading the C this call overwrites) and after (a barrier once the stream is idle). */
int b200_gemm_f32_colshard(const float* A, const float* B, float* const* dest, int n_dest,
                           int64_t M, int64_t N, int64_t K, int64_t col0, int64_t cols, int64_t lda,
                           int64_t ldb, int64_t ldc, int precision, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The sharded product behind one handle (no reference counterpart, src/cuda/runtime.cu:83).
 *
 * One rank per GPU of one node — a process per GPU, or one thread per GPU in one process; never two
 * ranks on one GPU (the barrier kernels of the ranks wait for one another).  A communicator belongs
 * to the device that was current when it was created, holds no pointer it owns except its own
 * staging buffers, and is used by one thread at a time.
 *
 *   b200_shard_comm_create     rank in [0, world), world <= 8.
 *   b200_shard_comm_set_peers  enables B200_SHARD_FUSED.  c_bufs[r]: rank r's full M x N result buffer
 *                              and flags[r]: rank r's block of `world` 32-bit words, both as DEVICE
 *                              pointers valid in THIS process (own memory at [rank]; the peers' through
 *                              peer access inside one process, or CUDA IPC / symmetric memory between
 *                              processes).  Every flag block must be zero before the first call and is
 *                              owned by the library from then on.
 *   b200_shard_comm_set_nccl   enables B200_SHARD_NCCL and b200_matmul_f32_host_sharded.  nccl_comm is the
 *                              caller's ncclComm_t of the same ranks; the library resolves NCCL at run
 *                              time from the libnccl.so.2 already in the process (else the system's)
 *                              and has no link-time dependency on it.  B200_EDEVICE if none is found.
 */
typedef struct b200_shard_comm b200_shard_comm;
int b200_shard_comm_create(b200_shard_comm** comm, int rank, int world);
int b200_shard_comm_set_peers(b200_shard_comm* comm, float* const* c_bufs, uint32_t* const* flags);
int b200_shard_comm_set_nccl(b200_shard_comm* comm, void* nccl_comm);
int b200_shard_comm_destroy(b200_shard_comm* comm);

/* The columns [*col0, *col0 + *cols) of an N-column result that rank `rank` of `world` computes:
 * equal blocks rounded up to 32 columns, the last ranks taking what is left. */
void b200_shard_columns(int64_t N, int world, int rank, int64_t* col0, int64_t* cols);

#define B200_SHARD_FUSED 0 /* tiles are stored into every rank's C by the product kernel itself */
#define B200_SHARD_NCCL 1  /* local columns, then one ncclAllGather of packed column blocks */

/* C = A x B with B and C split by column blocks over the ranks; every rank passes all of A (M x K),
 * all of B (K x N; only its own columns are read) and its full-size C, and ends with ALL of C.
 * Stream-ordered like every other call; collective: all ranks call it with the same shape.
 *
 * B200_SHARD_FUSED: [entry barrier] [product kernel] [exit barrier] on `stream`.  The product
 *   kernel's worker warps store each finished tile into this rank's C and two otherwise idle warps
 *   copy it from there into every peer's C with plain stores over NVLink while the next tiles are
 *   multiplied (no multicast, no TMA on peer memory).  C must be the buffer registered as
 *   c_bufs[rank].  Hazard that the barriers close: a peer's kernel writes into THIS rank's C.  The
 *   entry barrier holds every rank's stores back until all ranks have reached the call in stream
 *   order — so work queued earlier on `stream` that still reads the previous result is safe — and the
 *   exit barrier completes only when every rank's product kernel has finished, so work queued after
 *   the call sees all columns.  Readers on OTHER streams must be ordered against `stream` by the caller.
 * B200_SHARD_NCCL: product into a packed staging block, ncclAllGather in place, copies into C.
 *
 * A barrier wait that runs out (a peer that never arrives) is bounded at two seconds and reported
 * by b200_gemm_status as B200_ETIMEDOUT; C is then incomplete. */
int b200_gemm_f32_sharded(b200_shard_comm* comm, int mode, const float* A, const float* B, float* C,
                          int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                          int precision, void* stream);

/* The same sharded product from HOST buffers, and nothing is uploaded twice: rank r holds the rows
 * [r * M / world, (r + 1) * M / world) of A (a_rows, M / world x K), its own columns of B packed
 * (b_cols, K x cols) and receives its own columns of C packed (c_cols, M x cols, ALL rows), cols as
 * b200_shard_columns gives them.  Per rank the bus carries 1/world of A, 1/world of B and 1/world
 * of C.  Pipeline, on four streams: B's columns go up first; A's rows go up in `chunks` pieces
 * (0 = automatic, at most 16; M / world must divide); each piece is all-gathered over NVLink into
 * local memory (ncclAllGather, in place) as soon as it has landed; the strip of world * chunk rows
 * is multiplied as one product as soon as its gather is done; its rows go back to the host while
 * the next strip is multiplied.  Needs b200_shard_comm_set_nccl when world > 1; M % world == 0.
 * Returns after the result is on the host; pass page-locked buffers to get the overlap.
 * Collective: all ranks call it with the same M, N, K and chunks. */
#define B200_SHARD_MAX_CHUNKS 16
typedef struct b200_shard_host_layout {
    int chunks;
    int64_t rows_per_rank, chunk_rows;
} b200_shard_host_layout;
int b200_shard_host_plan(int64_t M, int world, int chunks, b200_shard_host_layout* out);
int b200_matmul_f32_host_sharded(b200_shard_comm* comm, const float* a_rows, const float* b_cols, float* c_cols,
                                 int64_t M, int64_t N, int64_t K, int chunks);

/* b200_gemm_f32 for callers that must not allocate device memory.  (No counterpart in the
 * reference: its split-K path always takes its partials from a growable scratch buffer,
 * src/cuda/kernels.cu:593-604.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits — a latency-critical loop that
 * cannot take cudaMalloc's implicit device synchronisation, a memory-budgeted process whose
 * device memory was handed out once at start-up, or a program under an arena allocator that
 * owns the whole GPU and offers no hook for a library to ask for more.
 * Such a caller can still pass A, B and C, but has nowhere to get the scratch that the
 * deterministic split-K path (tall-skinny products such as dW = X^T x dY) writes its partial
 * sums to.  Here that scratch is a fixed 4 MiB array inside the library's device image, present on
 * every GPU that loads the library until the process exits.  The call performs no cudaMalloc,
 * cudaFree or other allocating call.
 *
 * Same arguments and arithmetic as b200_gemm_f32; results are identical to what that function
 * returns when it is handed a workspace of the same 4 MiB.  Differences:
 *   - a shape whose split-K plan needs more than 4 MiB of partials is refused with
 *     B200_ENOSPACE (the automatic plan never needs more than about 2.4 MB on a B200; forced
 *     "split_k" / "tile_n" options can);
 *   - device_status: optional DEVICE pointer to an int, zeroed by the caller, that receives the
 *     bits of any bounded device-side wait that ran out (non-zero = treat results as invalid).
 *     With NULL those bits go to a word inside the library that b200_gemm_status does not read;
 *   - the first call on each device looks up the device addresses of the library's scratch and
 *     status word.  Make that first call with the device current and before any stream capture
 *     begins;
 *   - all calls on a device share the one scratch array, which keeps whatever the last call left
 *     in it (nothing in it needs to start at zero).  Two calls that may run at the same time on
 *     one GPU — different streams, or different threads — race on it: keep such calls on one
 *     stream or order them yourself. */
int b200_gemm_f32_static_scratch(const float* A, const float* B, float* C, int64_t batch, int64_t M,
                                 int64_t N, int64_t K, int transA, int transB, int64_t lda,
                                 int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB,
                                 int64_t strideC, float alpha, float beta, int precision,
                                 int* device_status, void* stream);

/* Device-side health of the launches so far on the current device: synchronises the device,
 * returns 0 or B200_ETIMEDOUT if any bounded wait inside a kernel ran out, and clears the flag.
 * Covers the launches of b200_gemm_f32_static_scratch that were given no status pointer too.
 * (The reference counts failed launches, src/cuda/kernels.cu:81-157; its kernels have no waits.) */
int b200_gemm_status(void);

/* Test aid for the failure-detection path: launches one warp that waits, with a budget of
 * budget_us microseconds (1 .. 100000), on a barrier nobody arrives at.  The wait runs out exactly
 * as a lost copy or a lost tensor-core completion would make a product kernel's wait run out: it
 * records a status bit and raises the abort flag, and the kernel returns normally — nothing traps
 * or faults, and the context stays usable.  Synchronises the device.  observed_host (optional,
 * two ints): [0] = threads whose wait wrongly reported completion (0 expected), [1] = the abort
 * flag (1 expected).  Afterwards b200_gemm_status() returns B200_ETIMEDOUT once.  Allocates a few
 * bytes of device memory for the duration of the call. */
int b200_gemm_selftest_timeout(unsigned budget_us, int* observed_host);

/* Number of kernels this library has launched in this process (all devices). */
uint64_t b200_gemm_launch_count(void);

/* Tuning knobs for benchmarking; unknown names return B200_EINVAL.
 *   "tile_n"        0 = automatic, else 32 / 64 / 128 / 256
 *   "split_k"       0 = automatic, 1 = never split, n = force n splits (needs workspace)
 *   "promote_every" k-blocks (32 k each) accumulated in TMEM before promotion to fp32 registers;
 *                   0 (default) = automatic: 1 in the fp32-accurate mode, 8 in TF32 mode
 *   "force_ldg"     1 = always use the register-staged loader instead of TMA
 *   "group_m"       tile rows per scheduling band (0 = automatic: 8 for pair tiles, 16 otherwise)
 *   "tail_split"    1 (default) = when the last wave of tiles would leave most SMs idle, run its
 *                   tiles split along K in a second launch (needs workspace), 0 = never
 *   "host_pipeline" 1 (default) = b200_matmul_f32_host overlaps transfers and math (12 panels per
 *                   side), 2..16 = the same with that many panels, 0 = one upload, one kernel,
 *                   one download
 *   "tf32_round"    B200_PRECISION_TF32 only: 1 (default) = operands are rounded to nearest TF32 first, as
 *                   the reference's tensor-core kernel converts them (wmma::__float_to_tf32); 0 = the
 *                   tensor core truncates them itself, which saves a pass over every tile (twice the
 *                   operand error, biased towards zero)
 *   "pair_mode"     0 = automatic, 1 = never, 2 = whenever legal: run 256 x 256 tiles on pairs of
 *                   CTAs (tcgen05 cta_group::2)
 *   "head_mode"     3xTF32 with the TMA loader: 0 (default) = the workers round every value to its
 *                   nearest TF32 head and write head and tail; 1 = the tensor core's own truncation
 *                   of the raw tile is the head and only the tail is written (one shared-memory
 *                   store pass less; representation error 2^-21 instead of 2^-22 per operand)
 *   "block_k"       values of k per pipeline stage: 0 / 32 = 32 (default), 64 = two 128-byte swizzle rows side by
 *                   side for tiles up to 64 columns wide with the TMA loader (half the barrier hand-overs of the
 *                   k-loop; measured 3-5 % faster at K >= 384, slower at K = 96, error 1.2-1.6x: not the default)
 *   "pair_workers"  worker warps per CTA of the CTA-pair kernel: 8 (default) or 16 (same bits; measured 3-5 %
 *                   slower on a B200)
 *   "split_warps"   CTA-pair kernel: 0 (default) = the eight worker warps split each landed stage and drain the
 *                   accumulator in turn; 8 = eight more warps per CTA only split, the workers only drain and
 *                   store (same bits; on a B200 1-2 % slower at 4096^3 and 8192^3, ~1 % faster at 16384^3)
 *   "pdl"           1 (default) = kernels are launched with programmatic stream serialization: the
 *                   set-up of a product overlaps the end of the kernel before it; 0 = plain launches
 *   "map_cache"     1 (default) = encoded TMA tensor maps are reused between calls with the same
 *                   pointers and shapes, 0 = every call encodes its own */
int b200_gemm_set_option(const char* name, long value);

/* Static description of a code, never NULL. */
const char* b200_gemm_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
