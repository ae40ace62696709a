// Fused attention core for sm_100a:  out = softmax(Q x K^T * scale + mask) x V  per head, without
// ever writing the (S_q x S_k) scores to global memory.
//
// The reference builds it from five kernels — a batched product against a materialised K^T,
// a scalar multiply, a broadcast add of the mask, a row softmax and a second batched product
// (scaled_dot_product_attention, src/transformer.cpp:279-304; softmax: src/tensor_ops.cpp:621-647).
// Here one CTA handles one (batch, head) matrix:
//
//   workers (4 warps)  load Q, K, V with plain loads, split them into TF32 head/tail tiles
//                      (the 3xTF32 scheme of the GEMM kernel) in K-major swizzled shared memory;
//   MMA lane           S = Q x K^T into TMEM (tcgen05.mma kind::tf32, M = 128, rows past S_q are
//                      zero padding);
//   workers            each thread pulls ITS row of S from TMEM (one TMEM lane = one query row),
//                      so scale, mask, max, exp, sum and divide are thread-local — in the
//                      reference's order, fp32 — then writes the row of P, split, back to shared
//                      memory over the Q/K tiles that are no longer needed;
//   MMA lane           O = P x V into TMEM;
//   workers            store their row of O.
//
// Limits of this kernel: S_q <= 128, S_k <= 128, d_k <= 64, d_v <= 64 (the engine's models use
// S = 64 and 24-wide heads).  Larger shapes go through the separate products.
#pragma once

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kAttnThreads = 160;  // warp 0: MMA issue + TMEM; warps 1..4: one thread per query row
constexpr int kAttnMaxSk = 128;
constexpr int kAttnMaxD = 64;

struct AttnParams {
    const float* q;     // (batch, s_q, d_k)
    const float* k;     // (batch, s_k, d_k)
    const float* v;     // (batch, s_k, d_v)
    const float* mask;  // (s_q, s_k) additive, shared by every batch element, or null
    float* out;         // (batch, s_q, d_v)
    float* weights;     // (batch, s_q, s_k) softmax output, or null
    int batch, s_q, s_k, d_k, d_v;
    int sk_pad, dk_pad, dv_pad;  // s_k rounded to 32, d_k to 32, d_v to 16
    float scale;
    int precision;
    int* status;
};

// Byte offset of element (row r, k) in a K-major, 128-byte-swizzled tile made of k-blocks of 32
// floats; k-block kb of a tile with `rows` rows starts at kb * rows * 128.
__device__ __forceinline__ uint32_t kmajor_offset(int rows, int r, int k) {
    const int kb = k >> 5, c = (k >> 2) & 7;
    return (uint32_t)kb * (uint32_t)rows * 128u + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u +
           (uint32_t)((c ^ (r & 7)) << 4) + (uint32_t)(k & 3) * 4u;
}

// Loads a (rows_valid x k_valid) matrix into a K-major tile of `rows` x `k_pad`, zero padded,
// split into head and tail.  k_contig: element (r, k) at src[r * ld + k], else at src[k * ld + r].
__device__ __forceinline__ void attn_load_tile(const float* __restrict__ src, long long ld, bool k_contig,
                                               int rows, int rows_valid, int k_pad, int k_valid,
                                               uint8_t* hi, uint8_t* lo, bool want_lo, int tid, int nthreads) {
    const int chunks = k_pad >> 2;  // groups of 4 k
    const int units = rows * chunks;
    for (int unit = tid; unit < units; unit += nthreads) {
        int r, c;
        if (k_contig) {
            r = unit / chunks;
            c = unit - r * chunks;
        } else {
            c = unit / rows;
            r = unit - c * rows;
        }
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < rows_valid) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = c * 4 + e;
                if (kk < k_valid) x[e] = __ldg(k_contig ? src + (long long)r * ld + kk : src + (long long)kk * ld + r);
            }
        }
        float4 h, l;
        tf32_split(x[0], h.x, l.x);
        tf32_split(x[1], h.y, l.y);
        tf32_split(x[2], h.z, l.z);
        tf32_split(x[3], h.w, l.w);
        const uint32_t off = kmajor_offset(rows, r, c * 4);
        *reinterpret_cast<float4*>(hi + off) = h;
        if (want_lo) *reinterpret_cast<float4*>(lo + off) = l;
    }
}

// Issues the products of one (A tile) x (B tile)^T over k_pad values of k into TMEM column `dcol`.
__device__ __forceinline__ void attn_issue(uint32_t tmem_d, uint32_t a_hi, uint32_t a_lo, int a_rows,
                                           uint32_t b_hi, uint32_t b_lo, int b_rows, int k_pad, int n,
                                           bool prec3) {
    const uint32_t idesc = make_idesc_tf32(128, n, 0, 0);
    uint32_t accumulate = 0;
    for (int pass = prec3 ? 0 : 2; pass < 3; ++pass) {  // tail x head, head x tail, head x head
        for (int kb = 0; kb < (k_pad >> 5); ++kb) {
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t ao = kb * a_rows * 128 + ks * 32, bo = kb * b_rows * 128 + ks * 32;
                const uint64_t ad = make_smem_desc((pass == 0 ? a_lo : a_hi) + ao, 16, 1024, kLayoutSw128);
                const uint64_t bd = make_smem_desc((pass == 1 ? b_lo : b_hi) + bo, 16, 1024, kLayoutSw128);
                mma_tf32_ss(tmem_d, ad, bd, idesc, accumulate);
                accumulate = 1;
            }
        }
    }
}

__global__ void __launch_bounds__(kAttnThreads, 1) attention_fwd_kernel(const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool worker = warp >= 1;
    const int wtid = threadIdx.x - 32;  // 0..127 for workers
    const int row = (warp & 3) * 32 + lane;  // worker's query row = its TMEM lane
    const bool prec3 = p.precision == 0;

    // shared memory: [ Q hi | Q lo | K hi | K lo ] later reused as [ P hi | P lo ], then [ V hi | V lo ]
    const uint32_t q_bytes = 128u * p.dk_pad * 4u, k_bytes = (uint32_t)p.sk_pad * p.dk_pad * 4u;
    const uint32_t p_bytes = 128u * p.sk_pad * 4u, v_bytes = (uint32_t)p.dv_pad * p.sk_pad * 4u;
    const uint32_t region1 = max(2 * (q_bytes + k_bytes), 2 * p_bytes);
    uint8_t* q_hi = smem;
    uint8_t* q_lo = q_hi + q_bytes;
    uint8_t* k_hi = q_lo + q_bytes;
    uint8_t* k_lo = k_hi + k_bytes;
    uint8_t* p_hi = smem;
    uint8_t* p_lo = p_hi + p_bytes;
    uint8_t* v_hi = smem + region1;
    uint8_t* v_lo = v_hi + v_bytes;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        abort_s = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(&tmem_base_s), 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;
    volatile int* abort_flag = &abort_s;

    uint32_t phase = 0;
    for (int b = blockIdx.x; b < p.batch; b += gridDim.x, phase ^= 1) {
        // ---- 1. operands into shared memory
        if (worker) {
            attn_load_tile(p.q + (long long)b * p.s_q * p.d_k, p.d_k, true, 128, p.s_q, p.dk_pad, p.d_k, q_hi,
                           q_lo, prec3, wtid, 128);
            attn_load_tile(p.k + (long long)b * p.s_k * p.d_k, p.d_k, true, p.sk_pad, p.s_k, p.dk_pad, p.d_k,
                           k_hi, k_lo, prec3, wtid, 128);
            // V is the B operand of P x V: tile rows = value feature, k = key index
            attn_load_tile(p.v + (long long)b * p.s_k * p.d_v, p.d_v, false, p.dv_pad, p.d_v, p.sk_pad, p.s_k,
                           v_hi, v_lo, prec3, wtid, 128);
            fence_proxy_async_smem();
        }
        __syncthreads();
        // ---- 2. S = Q x K^T
        if (threadIdx.x == 0) {
            tc_fence_after_sync();
            attn_issue(tmem_s, smem_u32(q_hi), smem_u32(q_lo), 128, smem_u32(k_hi), smem_u32(k_lo), p.sk_pad,
                       p.dk_pad, p.sk_pad, prec3);
            tc_commit(smem_u32(&bars[0]));
        }
        // ---- 3. softmax of one row per thread, P back to shared memory
        bool ok = true;
        if (worker) {
            ok = mbar_wait(smem_u32(&bars[0]), phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, 16);
                *abort_flag = 1;
            } else {
                tc_fence_after_sync();
                float s[kAttnMaxSk];
                const uint32_t t0 = tmem_s + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll
                for (int g = 0; g < kAttnMaxSk / 32; ++g) {
                    if (g * 32 < p.sk_pad) {
                        uint32_t v32[32];
                        tmem_ld_x32(t0 + g * 32, v32);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) s[g * 32 + j] = __uint_as_float(v32[j]);
                    }
                }
                tc_fence_before_sync();
                // scores = (q . k) * scale + mask; then the reference's softmax loop, all fp32
                const bool valid_row = row < p.s_q;
                float max_v = -INFINITY;
#pragma unroll
                for (int j = 0; j < kAttnMaxSk; ++j) {
                    if (j < p.s_k) {
                        float x = s[j] * p.scale;
                        if (p.mask && valid_row) x += __ldg(p.mask + (long long)row * p.s_k + j);
                        s[j] = x;
                        max_v = fmaxf(max_v, x);
                    }
                }
                float denom = 0.f;
#pragma unroll
                for (int j = 0; j < kAttnMaxSk; ++j) {
                    if (j < p.s_k) {
                        const float e = expf(s[j] - max_v);
                        s[j] = e;
                        denom += e;
                    }
                }
#pragma unroll
                for (int j = 0; j < kAttnMaxSk; ++j) {
                    if (j < p.s_k) {
                        s[j] = s[j] / denom;
                    } else {
                        s[j] = 0.f;
                    }
                }
                if (p.weights && valid_row) {
                    float* wrow = p.weights + ((long long)b * p.s_q + row) * p.s_k;
#pragma unroll
                    for (int j = 0; j < kAttnMaxSk; ++j)
                        if (j < p.s_k) wrow[j] = s[j];
                }
                // P tile: row = this thread, k = key index
#pragma unroll
                for (int j = 0; j < kAttnMaxSk; j += 4) {
                    if (j < p.sk_pad) {
                        float4 h, l;
                        tf32_split(valid_row ? s[j] : 0.f, h.x, l.x);
                        tf32_split(valid_row ? s[j + 1] : 0.f, h.y, l.y);
                        tf32_split(valid_row ? s[j + 2] : 0.f, h.z, l.z);
                        tf32_split(valid_row ? s[j + 3] : 0.f, h.w, l.w);
                        const uint32_t off = kmajor_offset(128, row, j);
                        *reinterpret_cast<float4*>(p_hi + off) = h;
                        if (prec3) *reinterpret_cast<float4*>(p_lo + off) = l;
                    }
                }
                fence_proxy_async_smem();
            }
        }
        __syncthreads();
        if (*abort_flag) break;
        // ---- 4. O = P x V
        if (threadIdx.x == 0) {
            tc_fence_after_sync();
            attn_issue(tmem_o, smem_u32(p_hi), smem_u32(p_lo), 128, smem_u32(v_hi), smem_u32(v_lo), p.dv_pad,
                       p.sk_pad, p.dv_pad, prec3);
            tc_commit(smem_u32(&bars[1]));
        }
        // ---- 5. store the rows of O
        if (worker) {
            ok = mbar_wait(smem_u32(&bars[1]), phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, 32);
                *abort_flag = 1;
            } else {
                tc_fence_after_sync();
                const uint32_t t0 = tmem_o + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll
                for (int g = 0; g < kAttnMaxD / 16; ++g) {
                    if (g * 16 < p.dv_pad) {
                        uint32_t v16[16];
                        tmem_ld_x16(t0 + g * 16, v16);
                        tmem_ld_wait();
                        if (row < p.s_q) {
                            float* orow = p.out + ((long long)b * p.s_q + row) * p.d_v;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (g * 16 + j < p.d_v) orow[g * 16 + j] = __uint_as_float(v16[j]);
                        }
                    }
                }
                tc_fence_before_sync();
            }
        }
        __syncthreads();  // shared memory and TMEM are reused by the next head
        if (*abort_flag) break;
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace b200
