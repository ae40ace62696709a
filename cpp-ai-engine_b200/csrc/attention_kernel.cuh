// Fused attention core for sm_100a:  out = softmax(Q x K^T * scale + mask) x V  per head, without
// ever writing the (S_q x S_k) scores to global memory.
//
// The reference builds it from five kernels — a batched product against a materialised K^T,
// a scalar multiply, a broadcast add of the mask, a row softmax and a second batched product
// (scaled_dot_product_attention, src/transformer.cpp:279-304; softmax: src/tensor_ops.cpp:621-647).
// Here one CTA handles one (batch, head) matrix:
//
//   workers (8 warps)  load Q, K and V with plain loads, split them into TF32 head/tail tiles
//                      (the 3xTF32 scheme of the GEMM kernel) in K-major swizzled shared memory;
//   MMA lane           S = Q x K^T into TMEM (tcgen05.mma kind::tf32, M = 128; rows past S_q are
//                      never read back);
//   workers            load their part of the mask while that product runs; then two threads
//                      share each row of S (one TMEM lane = one query row, each thread takes half
//                      of its columns): scale, mask, max, exp, sum and divide in fp32, the sum in
//                      the reference's column order (the first half hands its partial sum to the
//                      second), with the row maximum and the sums exchanged through shared memory;
//                      the row of P goes back, split, to shared memory over the Q/K tiles;
//   MMA lane           O = P x V into TMEM;
//   workers            store their row of O.
//
// Limits of this kernel: S_q <= 128, S_k <= 128, d_k <= 64, d_v <= 64 (the engine's models use
// S = 64 and 24-wide heads).  Larger shapes go through the separate products.
#pragma once

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kAttnWorkers = 256;               // warps 1..8: two threads per query row
constexpr int kAttnThreads = 32 + kAttnWorkers;  // warp 0: MMA issue + TMEM
// Nine warps put three on one of the SM's four register files (16384 registers each), so a thread
// can have 168 registers at most: a larger per-thread cap compiles but cannot be launched.
constexpr int kAttnMaxSk = 128;
constexpr int kAttnMaxD = 64;

struct AttnParams {
    // Matrix i of the batch is (i / heads, i % heads); element (row, e) of its Q lies at
    // q[(i / heads) * q_bs + (i % heads) * q_hs + row * q_ld + e], and likewise for K, V and out, so
    // the split into heads and the merge back are addressing, not copies.
    const float* q;     // s_q x d_k per matrix
    const float* k;     // s_k x d_k per matrix
    const float* v;     // s_k x d_v per matrix
    const float* mask;  // (s_q, s_k) additive, shared by every matrix, or null
    float* out;         // s_q x d_v per matrix
    float* weights;     // (batch, s_q, s_k) contiguous softmax output, or null
    long long q_bs, q_hs, q_ld, k_bs, k_hs, k_ld, v_bs, v_hs, v_ld, o_bs, o_hs, o_ld;
    int batch, heads, s_q, s_k, d_k, d_v;
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

// Operand tiles are K-major, `rows` x `k_pad`, zero padded along k, split into head and tail.
// A (rows_valid x k_valid) matrix is fetched in units of 4 consecutive k: element (r, k) at
// src[r * ld + k] if k_contig, else at src[k * ld + r].  Rows past rows_valid are zero filled only
// if fill_rows (an A operand's spare rows may hold anything: they feed accumulator rows that are
// never read).  Fetching (global loads into registers) and committing (split + shared-memory
// stores) are separate steps so that the loads of all three operands of a head are in flight
// together: a head costs one memory round trip, not one per tile.
#ifndef B200_ATTN_FETCH_BATCH
#define B200_ATTN_FETCH_BATCH 4
#endif
constexpr int kAttnFetchBatch = B200_ATTN_FETCH_BATCH;

struct AttnFetch {
    float4 x[kAttnFetchBatch];
    int off[kAttnFetchBatch];  // byte offset in the tile, or -1: nothing to store
};

__device__ __forceinline__ void attn_fetch(AttnFetch& f, const float* __restrict__ src, long long ld,
                                           bool k_contig, int rows, int rows_valid, bool fill_rows, int k_pad,
                                           int k_valid, int base, int nthreads) {
    const int chunks = k_pad >> 2;  // groups of 4 k
    const int units = rows * chunks;
    const bool vec = k_contig && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
#pragma unroll
    for (int u = 0; u < kAttnFetchBatch; ++u) {
        const int unit = base + u * nthreads;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        int off = -1;
        if (unit < units) {
            int r, c;
            if (k_contig) {
                r = unit / chunks;
                c = unit - r * chunks;
            } else {
                c = unit / rows;
                r = unit - c * rows;
            }
            const int k0 = c * 4;
            if (fill_rows || r < rows_valid) off = static_cast<int>(kmajor_offset(rows, r, k0));
            if (r < rows_valid && k0 < k_valid) {
                if (k_contig) {
                    const float* ptr = src + (long long)r * ld + k0;
                    if (vec && k0 + 3 < k_valid) {
                        v = __ldg(reinterpret_cast<const float4*>(ptr));
                    } else {
                        v.x = __ldg(ptr);
                        if (k0 + 1 < k_valid) v.y = __ldg(ptr + 1);
                        if (k0 + 2 < k_valid) v.z = __ldg(ptr + 2);
                        if (k0 + 3 < k_valid) v.w = __ldg(ptr + 3);
                    }
                } else {
                    const float* ptr = src + (long long)k0 * ld + r;
                    v.x = __ldg(ptr);
                    if (k0 + 1 < k_valid) v.y = __ldg(ptr + ld);
                    if (k0 + 2 < k_valid) v.z = __ldg(ptr + 2 * ld);
                    if (k0 + 3 < k_valid) v.w = __ldg(ptr + 3 * ld);
                }
            }
        }
        f.x[u] = v;
        f.off[u] = off;
    }
}

__device__ __forceinline__ void attn_commit(const AttnFetch& f, uint8_t* hi, uint8_t* lo, bool want_lo) {
#pragma unroll
    for (int u = 0; u < kAttnFetchBatch; ++u) {
        if (f.off[u] < 0) continue;
        float4 h, l;
        tf32_split(f.x[u].x, h.x, l.x);
        tf32_split(f.x[u].y, h.y, l.y);
        tf32_split(f.x[u].z, h.z, l.z);
        tf32_split(f.x[u].w, h.w, l.w);
        *reinterpret_cast<float4*>(hi + f.off[u]) = h;
        if (want_lo) *reinterpret_cast<float4*>(lo + f.off[u]) = l;
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

// Named barrier of the worker warps only (the MMA warp does not take part).
__device__ __forceinline__ void attn_worker_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kAttnWorkers) : "memory");
}

// CH = s_k rounded up to 32, divided by 32: every worker owns CH * 16 score columns of its row.
template <int CH>
__global__ void __launch_bounds__(kAttnThreads, 1) attention_fwd_kernel(const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ float red_max[2][128];
    __shared__ float red_sum[2][128];

    constexpr int kCols = CH * 16;  // score columns per worker
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool worker = warp >= 1;
    const int wtid = threadIdx.x - 32;       // 0..255 for workers
    const int half = (warp - 1) >> 2;        // which half of the row's columns (workers only)
    const int row = (warp & 3) * 32 + lane;  // worker's query row = its TMEM lane
    const int col0 = half * kCols;
    const bool prec3 = p.precision == 0;
    // rows past s_q hold whatever shared memory held: a row of an accumulator depends on that row
    // of the A operand only, and those rows are never stored.  Warps made of such rows only skip
    // the arithmetic (not the barriers).
    const bool warp_has_rows = (warp & 3) * 32 < p.s_q;
    const bool valid_row = row < p.s_q;

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
    const bool mask_vec = p.mask != nullptr && (p.s_k & 3) == 0 && (reinterpret_cast<uintptr_t>(p.mask) & 15u) == 0;

    uint32_t phase = 0;
    for (int b = blockIdx.x; b < p.batch; b += gridDim.x, phase ^= 1) {
        const int bb = b / p.heads, bh = b - bb * p.heads;
        // ---- 1. Q, K and V (the B operand of P x V: tile rows = value feature, k = key index) into
        //         shared memory
        if (worker) {
            const int units_q = 128 * (p.dk_pad >> 2), units_k = p.sk_pad * (p.dk_pad >> 2);
            const int units_v = p.dv_pad * (p.sk_pad >> 2);
            const int units_max = max(units_q, max(units_k, units_v));
            for (int base = wtid; base < units_max; base += kAttnWorkers * kAttnFetchBatch) {
                AttnFetch fq, fk, fv;
                attn_fetch(fq, p.q + bb * p.q_bs + bh * p.q_hs, p.q_ld, true, 128, p.s_q, false, p.dk_pad, p.d_k,
                           base, kAttnWorkers);
                attn_fetch(fk, p.k + bb * p.k_bs + bh * p.k_hs, p.k_ld, true, p.sk_pad, p.s_k, true, p.dk_pad,
                           p.d_k, base, kAttnWorkers);
                attn_fetch(fv, p.v + bb * p.v_bs + bh * p.v_hs, p.v_ld, false, p.dv_pad, p.d_v, true, p.sk_pad,
                           p.s_k, base, kAttnWorkers);
                attn_commit(fq, q_hi, q_lo, prec3);
                attn_commit(fk, k_hi, k_lo, prec3);
                attn_commit(fv, v_hi, v_lo, prec3);
            }
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
        // ---- 3. softmax: each row is shared by two workers (one per half of its columns)
        bool ok = true;
        if (worker) {
            // while the product runs: this thread's part of the mask row
            float s[kCols];
            float m[kCols];
#pragma unroll
            for (int j = 0; j < kCols; ++j) m[j] = 0.f;
            if (p.mask != nullptr && valid_row) {
                const float* mrow = p.mask + (long long)row * p.s_k + col0;
#pragma unroll
                for (int j = 0; j < kCols; j += 4) {
                    if (mask_vec && col0 + j + 3 < p.s_k) {
                        const float4 t = __ldg(reinterpret_cast<const float4*>(mrow + j));
                        m[j] = t.x, m[j + 1] = t.y, m[j + 2] = t.z, m[j + 3] = t.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (col0 + j + e < p.s_k) m[j + e] = __ldg(mrow + j + e);
                    }
                }
            }
            ok = mbar_wait(smem_u32(&bars[0]), phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, 16);
                *abort_flag = 1;
            }
            tc_fence_after_sync();
            const uint32_t t0 = tmem_s + (static_cast<uint32_t>((warp & 3) * 32) << 16) + col0;
            float max_v = -INFINITY;
            if (ok && warp_has_rows) {
#pragma unroll
                for (int g = 0; g < CH; ++g) {
                    uint32_t v16[16];
                    tmem_ld_x16(t0 + g * 16, v16);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) s[g * 16 + j] = __uint_as_float(v16[j]);
                }
                // scores = (q . k) * scale, then + mask: two roundings, as the reference's two ops;
                // columns past s_k become -inf, so their exp is an exact 0
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    float x = __fmul_rn(s[j], p.scale);
                    if (p.mask != nullptr) x = __fadd_rn(x, m[j]);
                    if (col0 + j >= p.s_k) x = -INFINITY;
                    s[j] = x;
                    max_v = fmaxf(max_v, x);
                }
            }
            tc_fence_before_sync();
            red_max[half][row] = max_v;
            attn_worker_sync();
            max_v = fmaxf(red_max[0][row], red_max[1][row]);
            // the sum runs over the columns in ascending order, as the reference's loop: the first
            // half hands its partial sum to the second
            float sum = 0.f;
            if (ok && warp_has_rows) {
#pragma unroll
                for (int j = 0; j < kCols; ++j) s[j] = expf(s[j] - max_v);
            }
            if (half == 0) {
                if (ok && warp_has_rows) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) sum += s[j];
                }
                red_sum[0][row] = sum;
            }
            attn_worker_sync();
            if (half == 1) {
                sum = red_sum[0][row];
                if (ok && warp_has_rows) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) sum += s[j];
                }
                red_sum[1][row] = sum;
            }
            attn_worker_sync();
            if (ok && warp_has_rows) {
                // e / denom, correctly rounded: a rounded reciprocal, one product and one residual
                // correction (the division's own fast path, without its range checks: 0 <= e <= 1 and
                // 1 <= denom <= 128 here)
                const float denom = red_sum[1][row];
                const float inv = __frcp_rn(denom);
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    const float q0 = s[j] * inv;
                    const float r = fmaf(-q0, denom, s[j]);
                    s[j] = fmaf(r, inv, q0);
                }
                if (p.weights && valid_row) {
                    float* wrow = p.weights + ((long long)b * p.s_q + row) * p.s_k + col0;
                    const bool wvec = (p.s_k & 3) == 0 && (reinterpret_cast<uintptr_t>(p.weights) & 15u) == 0;
#pragma unroll
                    for (int j = 0; j < kCols; j += 4) {
                        if (wvec && col0 + j + 3 < p.s_k) {
                            *reinterpret_cast<float4*>(wrow + j) = make_float4(s[j], s[j + 1], s[j + 2], s[j + 3]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (col0 + j + e < p.s_k) wrow[j + e] = s[j + e];
                        }
                    }
                }
                // P tile: row = this thread, k = key index
#pragma unroll
                for (int j = 0; j < kCols; j += 4) {
                    float4 h, l;
                    tf32_split(s[j], h.x, l.x);
                    tf32_split(s[j + 1], h.y, l.y);
                    tf32_split(s[j + 2], h.z, l.z);
                    tf32_split(s[j + 3], h.w, l.w);
                    const uint32_t off = kmajor_offset(128, row, col0 + j);
                    *reinterpret_cast<float4*>(p_hi + off) = h;
                    if (prec3) *reinterpret_cast<float4*>(p_lo + off) = l;
                }
            }
            fence_proxy_async_smem();
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
        // ---- 5. store the rows of O: the 16-column groups alternate between a row's two workers
        if (worker) {
            ok = mbar_wait(smem_u32(&bars[1]), phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, 32);
                *abort_flag = 1;
            } else if (warp_has_rows) {
                tc_fence_after_sync();
                const uint32_t t0 = tmem_o + (static_cast<uint32_t>((warp & 3) * 32) << 16);
                float* obase = p.out + bb * p.o_bs + bh * p.o_hs;
                const bool ovec = (p.o_ld & 3) == 0 && (reinterpret_cast<uintptr_t>(obase) & 15u) == 0;
#pragma unroll
                for (int g = 0; g < kAttnMaxD / 16; ++g) {
                    if ((g & 1) == half && g * 16 < p.dv_pad) {
                        uint32_t v16[16];
                        tmem_ld_x16(t0 + g * 16, v16);
                        tmem_ld_wait();
                        if (valid_row) {
                            float* orow = obase + row * p.o_ld + g * 16;
#pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                if (ovec && g * 16 + j + 3 < p.d_v) {
                                    *reinterpret_cast<float4*>(orow + j) =
                                        make_float4(__uint_as_float(v16[j]), __uint_as_float(v16[j + 1]),
                                                    __uint_as_float(v16[j + 2]), __uint_as_float(v16[j + 3]));
                                } else {
#pragma unroll
                                    for (int e = 0; e < 4; ++e)
                                        if (g * 16 + j + e < p.d_v) orow[j + e] = __uint_as_float(v16[j + e]);
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
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
