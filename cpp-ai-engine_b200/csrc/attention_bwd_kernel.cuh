// Backward pass of the fused attention core for sm_100a: for one head,
//
//     W  = softmax(Q x K^T * scale + mask)          recomputed, never stored
//     dW = dO x V^T
//     dV = W^T x dO
//     dS = W o (dW - rowsum(dW o W)) * scale        softmax's and the scale's backward
//     dQ = dS x K,    dK = dS^T x Q
//
// which the reference's autograd derives from the five nodes of scaled_dot_product_attention
// (src/transformer.cpp:279-304): two product backwards (src/tensor_ops.cpp:570-585, each with a
// materialised transpose), the softmax backward dX_ij = y_ij (dY_ij - sum_k dY_ik y_ik)
// (src/tensor_ops.cpp:649-668), the scalar multiply's and the K^T transpose's.  Here one CTA per
// head runs five tcgen05 products and the row arithmetic between them:
//
//   workers   Q, dO (A operands) and K, V (B operands) into shared memory, split for 3xTF32 —
//             one round trip;
//   MMA lane  S = Q x K^T and dW = dO x V^T into two TMEM regions;
//   workers   two threads per row: W as in the forward kernel (same arithmetic, same order),
//             then dot = sum_j dW_j W_j in ascending j (the first half hands its partial sum to
//             the second), dS; they write dS (rows = queries) and the TRANSPOSED W and dS (rows =
//             keys) as A operands, and load the transposed B operands dO^T, K^T, Q^T, all over the
//             dead Q / K / V / dO tiles;
//   MMA lane  dV = W^T x dO, dQ = dS x K, dK = dS^T x Q;
//   workers   store the rows (beta = 1 accumulates into existing gradients).
//
// An A tile only holds the rows that exist (rounded up to 8): the products read 128 rows, the
// rest is whatever follows in shared memory and lands in accumulator rows that are never read.
// The host lays the tiles out, checks that they fit and leaves 16 KB of slack after the last.
#pragma once

#include "attention_kernel.cuh"

namespace b200 {

struct AttnBwdParams {
    const float* q;
    const float* k;
    const float* v;
    const float* mask;   // (s_q, s_k) or null
    const float* dout;   // gradient of the output, addressed like the forward's out
    float* dq;           // addressed like q
    float* dk;           // addressed like k
    float* dv;           // addressed like v
    long long q_bs, q_hs, q_ld, k_bs, k_hs, k_ld, v_bs, v_hs, v_ld, o_bs, o_hs, o_ld;
    int batch, heads, s_q, s_k, d_k, d_v;
    int sq_pad, sk_pad;    // rounded to 32: contraction lengths of the transposed products
    int dk_pad, dv_pad;    // rounded to 32: contraction lengths of S and dW
    int dk_n, dv_n;        // rounded to 16: widths of dQ / dK and dV
    int rows_q, rows_k;    // rows held by the A tiles indexed by query / key (rounded to 8)
    // byte offsets of the head tiles in shared memory; each tail tile follows its head tile
    uint32_t off_qa, off_kb, off_vb, off_doa;   // first two products (dead afterwards)
    uint32_t off_wt, off_ds, off_dst;           // A operands of the last three, over the dead tiles
    uint32_t off_dot, off_kt, off_qt;           // transposed B operands of the last three, likewise
    uint32_t sz_qa, sz_kb, sz_vb, sz_doa, sz_wt, sz_ds, sz_dst, sz_dot, sz_kt, sz_qt;
    float scale;
    float beta;
    int precision;
    int* status;
};

template <int CH>
__global__ void __launch_bounds__(kAttnThreads, 1) attention_bwd_kernel(const AttnBwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ float red_a[2][128];
    __shared__ float red_b[2][128];

    constexpr int kCols = CH * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool worker = warp >= 1;
    const int wtid = threadIdx.x - 32;
    const int half = (warp - 1) >> 2;
    const int row = (warp & 3) * 32 + lane;  // TMEM lane: a query row, later a key row
    const int col0 = half * kCols;
    const bool prec3 = p.precision == 0;
    const bool warp_has_q = (warp & 3) * 32 < p.s_q;
    const bool valid_q = row < p.s_q;

    uint8_t* qa = smem + p.off_qa;
    uint8_t* kb = smem + p.off_kb;
    uint8_t* vb = smem + p.off_vb;
    uint8_t* doa = smem + p.off_doa;
    uint8_t* wt = smem + p.off_wt;
    uint8_t* ds = smem + p.off_ds;
    uint8_t* dst = smem + p.off_dst;
    uint8_t* dot_t = smem + p.off_dot;
    uint8_t* kt = smem + p.off_kt;
    uint8_t* qt = smem + p.off_qt;

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
    const uint32_t tmem_s = tmem, tmem_g = tmem + 128;                    // S and dW
    const uint32_t tmem_dv = tmem, tmem_dq = tmem + 64, tmem_dk = tmem + 128;  // afterwards
    volatile int* abort_flag = &abort_s;
    const bool mask_vec = p.mask != nullptr && (p.s_k & 3) == 0 && (reinterpret_cast<uintptr_t>(p.mask) & 15u) == 0;

    uint32_t phase = 0;
    for (int b = blockIdx.x; b < p.batch; b += gridDim.x, phase ^= 1) {
        const int bb = b / p.heads, bh = b - bb * p.heads;
        const float* gq = p.q + bb * p.q_bs + bh * p.q_hs;
        const float* gk = p.k + bb * p.k_bs + bh * p.k_hs;
        const float* gv = p.v + bb * p.v_bs + bh * p.v_hs;
        const float* gdo = p.dout + bb * p.o_bs + bh * p.o_hs;

        // ---- 1. the operand tiles of the first two products
        if (worker) {
            int units_max = 128 * (p.dk_pad >> 2);                       // Q as A
            units_max = max(units_max, 128 * (p.dv_pad >> 2));           // dO as A
            units_max = max(units_max, p.sk_pad * (p.dk_pad >> 2));      // K as B
            units_max = max(units_max, p.sk_pad * (p.dv_pad >> 2));      // V as B
            for (int base = wtid; base < units_max; base += kAttnWorkers * kAttnFetchBatch) {
                AttnFetch f0, f1, f2, f3;
                attn_fetch(f0, gq, p.q_ld, true, 128, p.s_q, false, p.dk_pad, p.d_k, base, kAttnWorkers);
                attn_fetch(f1, gdo, p.o_ld, true, 128, p.s_q, false, p.dv_pad, p.d_v, base, kAttnWorkers);
                attn_fetch(f2, gk, p.k_ld, true, p.sk_pad, p.s_k, true, p.dk_pad, p.d_k, base, kAttnWorkers);
                attn_fetch(f3, gv, p.v_ld, true, p.sk_pad, p.s_k, true, p.dv_pad, p.d_v, base, kAttnWorkers);
                attn_commit(f0, qa, qa + p.sz_qa, prec3);
                attn_commit(f1, doa, doa + p.sz_doa, prec3);
                attn_commit(f2, kb, kb + p.sz_kb, prec3);
                attn_commit(f3, vb, vb + p.sz_vb, prec3);
            }
            fence_proxy_async_smem();
        }
        __syncthreads();
        // ---- 2. S = Q x K^T, dW = dO x V^T
        if (threadIdx.x == 0) {
            tc_fence_after_sync();
            attn_issue(tmem_s, smem_u32(qa), smem_u32(qa + p.sz_qa), 128, smem_u32(kb), smem_u32(kb + p.sz_kb),
                       p.sk_pad, p.dk_pad, p.sk_pad, prec3);
            attn_issue(tmem_g, smem_u32(doa), smem_u32(doa + p.sz_doa), 128, smem_u32(vb), smem_u32(vb + p.sz_vb),
                       p.sk_pad, p.dv_pad, p.sk_pad, prec3);
            tc_commit(smem_u32(&bars[0]));
        }
        // ---- 3. the row arithmetic
        bool ok = true;
        if (worker) {
            ok = mbar_wait(smem_u32(&bars[0]), phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, 64);
                *abort_flag = 1;
            }
            tc_fence_after_sync();
            float s[kCols];
            float g[kCols];
            const bool active = ok && warp_has_q;
            float max_v = -INFINITY;
            if (active) {
                const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    uint32_t v16[16];
                    tmem_ld_x16(tmem_s + lane_off + col0 + c * 16, v16);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) s[c * 16 + j] = __uint_as_float(v16[j]);
                    tmem_ld_x16(tmem_g + lane_off + col0 + c * 16, v16);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) g[c * 16 + j] = __uint_as_float(v16[j]);
                }
                const float* mrow = p.mask != nullptr && valid_q ? p.mask + (long long)row * p.s_k + col0 : nullptr;
#pragma unroll
                for (int j = 0; j < kCols; j += 4) {
                    float m4[4] = {0.f, 0.f, 0.f, 0.f};
                    if (mrow != nullptr) {
                        if (mask_vec && col0 + j + 3 < p.s_k) {
                            const float4 t = __ldg(reinterpret_cast<const float4*>(mrow + j));
                            m4[0] = t.x, m4[1] = t.y, m4[2] = t.z, m4[3] = t.w;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (col0 + j + e < p.s_k) m4[e] = __ldg(mrow + j + e);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float x = __fmul_rn(s[j + e], p.scale);
                        if (p.mask != nullptr) x = __fadd_rn(x, m4[e]);
                        if (col0 + j + e >= p.s_k) x = -INFINITY;
                        s[j + e] = x;
                        max_v = fmaxf(max_v, x);
                    }
                }
            }
            tc_fence_before_sync();
            red_a[half][row] = max_v;
            attn_worker_sync();
            max_v = fmaxf(red_a[0][row], red_a[1][row]);
            float sum = 0.f;
            if (active) {
#pragma unroll
                for (int j = 0; j < kCols; ++j) s[j] = expf(s[j] - max_v);
            }
            if (half == 0) {
                if (active) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) sum += s[j];
                }
                red_b[0][row] = sum;
            }
            attn_worker_sync();
            if (half == 1) {
                sum = red_b[0][row];
                if (active) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) sum += s[j];
                }
                red_b[1][row] = sum;
            }
            attn_worker_sync();
            float dot = 0.f;
            if (active) {
                const float denom = red_b[1][row];
                const float inv = __frcp_rn(denom);
#pragma unroll
                for (int j = 0; j < kCols; ++j) {  // W, rounded like the forward kernel's division
                    const float q0 = s[j] * inv;
                    const float r = fmaf(-q0, denom, s[j]);
                    s[j] = fmaf(r, inv, q0);
                }
            }
            // dot = sum_j dW_j W_j, ascending j: one rounding for the product, one for the sum
            if (half == 0) {
                if (active) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) dot = __fadd_rn(dot, __fmul_rn(g[j], s[j]));
                }
                red_a[0][row] = dot;  // the maxima were consumed before the last barrier
            }
            attn_worker_sync();
            if (half == 1) {
                dot = red_a[0][row];
                if (active) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) dot = __fadd_rn(dot, __fmul_rn(g[j], s[j]));
                }
                red_a[1][row] = dot;
            }
            attn_worker_sync();
            if (ok) {
                dot = red_a[1][row];
                const bool live = active && valid_q;
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    // dS = (W (dW - dot)) * scale; rows and columns that do not exist give zeros
                    const float w = live ? s[j] : 0.f;
                    const float d = live ? __fmul_rn(__fmul_rn(w, __fsub_rn(g[j], dot)), p.scale) : 0.f;
                    s[j] = w;
                    g[j] = d;
                }
                // dS as an A operand: row = this query, k = key
                if (live) {
#pragma unroll
                    for (int j = 0; j < kCols; j += 4) {
                        float4 h, l;
                        tf32_split(g[j], h.x, l.x);
                        tf32_split(g[j + 1], h.y, l.y);
                        tf32_split(g[j + 2], h.z, l.z);
                        tf32_split(g[j + 3], h.w, l.w);
                        const uint32_t off = kmajor_offset(p.rows_q, row, col0 + j);
                        *reinterpret_cast<float4*>(ds + off) = h;
                        if (prec3) *reinterpret_cast<float4*>(ds + p.sz_ds + off) = l;
                    }
                }
                // W^T and dS^T as A operands: row = key, k = this query (zeros up to sq_pad)
                if (row < p.sq_pad) {
#pragma unroll
                    for (int j = 0; j < kCols; ++j) {
                        const int key = col0 + j;
                        if (key < p.rows_k) {
                            const uint32_t off = kmajor_offset(p.rows_k, key, row);
                            float h, l;
                            tf32_split(s[j], h, l);
                            *reinterpret_cast<float*>(wt + off) = h;
                            if (prec3) *reinterpret_cast<float*>(wt + p.sz_wt + off) = l;
                            tf32_split(g[j], h, l);
                            *reinterpret_cast<float*>(dst + off) = h;
                            if (prec3) *reinterpret_cast<float*>(dst + p.sz_dst + off) = l;
                        }
                    }
                }
            }
            // the transposed B operands of the last three products (tile rows = feature, k = query /
            // key index), over tiles of the first two products that are dead now
            if (ok) {
                int units_max = p.dv_n * (p.sq_pad >> 2);                // dO^T
                units_max = max(units_max, p.dk_n * (p.sk_pad >> 2));    // K^T
                units_max = max(units_max, p.dk_n * (p.sq_pad >> 2));    // Q^T
                for (int base = wtid; base < units_max; base += kAttnWorkers * kAttnFetchBatch) {
                    AttnFetch f0, f1, f2;
                    attn_fetch(f0, gdo, p.o_ld, false, p.dv_n, p.d_v, true, p.sq_pad, p.s_q, base, kAttnWorkers);
                    attn_fetch(f1, gk, p.k_ld, false, p.dk_n, p.d_k, true, p.sk_pad, p.s_k, base, kAttnWorkers);
                    attn_fetch(f2, gq, p.q_ld, false, p.dk_n, p.d_k, true, p.sq_pad, p.s_q, base, kAttnWorkers);
                    attn_commit(f0, dot_t, dot_t + p.sz_dot, prec3);
                    attn_commit(f1, kt, kt + p.sz_kt, prec3);
                    attn_commit(f2, qt, qt + p.sz_qt, prec3);
                }
            }
            fence_proxy_async_smem();
        }
        __syncthreads();
        if (*abort_flag) break;
        // ---- 4. dV = W^T x dO, dQ = dS x K, dK = dS^T x Q
        if (threadIdx.x == 0) {
            tc_fence_after_sync();
            attn_issue(tmem_dv, smem_u32(wt), smem_u32(wt + p.sz_wt), p.rows_k, smem_u32(dot_t),
                       smem_u32(dot_t + p.sz_dot), p.dv_n, p.sq_pad, p.dv_n, prec3);
            attn_issue(tmem_dq, smem_u32(ds), smem_u32(ds + p.sz_ds), p.rows_q, smem_u32(kt), smem_u32(kt + p.sz_kt),
                       p.dk_n, p.sk_pad, p.dk_n, prec3);
            attn_issue(tmem_dk, smem_u32(dst), smem_u32(dst + p.sz_dst), p.rows_k, smem_u32(qt),
                       smem_u32(qt + p.sz_qt), p.dk_n, p.sq_pad, p.dk_n, prec3);
            tc_commit(smem_u32(&bars[1]));
        }
        // ---- 5. store the gradient rows: 16-column groups alternate between a row's two workers
        if (worker) {
            ok = mbar_wait(smem_u32(&bars[1]), phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, 128);
                *abort_flag = 1;
            } else {
                tc_fence_after_sync();
                const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
                auto store_rows = [&](uint32_t tcol, int rows_valid, int width, int width_pad, float* base,
                                      long long ld) {
                    if ((warp & 3) * 32 >= rows_valid) return;  // warp-uniform
                    const bool vec = (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
#pragma unroll
                    for (int c = 0; c < kAttnMaxD / 16; ++c) {
                        if ((c & 1) == half && c * 16 < width_pad) {
                            uint32_t v16[16];
                            tmem_ld_x16(tcol + lane_off + c * 16, v16);
                            tmem_ld_wait();
                            if (row < rows_valid) {
                                float* orow = base + row * ld + c * 16;
#pragma unroll
                                for (int j = 0; j < 16; j += 4) {
                                    if (vec && c * 16 + j + 3 < width) {
                                        float4 o = make_float4(__uint_as_float(v16[j]), __uint_as_float(v16[j + 1]),
                                                               __uint_as_float(v16[j + 2]), __uint_as_float(v16[j + 3]));
                                        if (p.beta != 0.f) {
                                            const float4 old = *reinterpret_cast<const float4*>(orow + j);
                                            o.x += p.beta * old.x, o.y += p.beta * old.y;
                                            o.z += p.beta * old.z, o.w += p.beta * old.w;
                                        }
                                        *reinterpret_cast<float4*>(orow + j) = o;
                                    } else {
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            if (c * 16 + j + e < width) {
                                                float o = __uint_as_float(v16[j + e]);
                                                if (p.beta != 0.f) o += p.beta * orow[j + e];
                                                orow[j + e] = o;
                                            }
                                        }
                                    }
                                }
                            }
                        }
                    }
                };
                if (p.dv != nullptr)
                    store_rows(tmem_dv, p.s_k, p.d_v, p.dv_n, p.dv + bb * p.v_bs + bh * p.v_hs, p.v_ld);
                if (p.dq != nullptr)
                    store_rows(tmem_dq, p.s_q, p.d_k, p.dk_n, p.dq + bb * p.q_bs + bh * p.q_hs, p.q_ld);
                if (p.dk != nullptr)
                    store_rows(tmem_dk, p.s_k, p.d_k, p.dk_n, p.dk + bb * p.k_bs + bh * p.k_hs, p.k_ld);
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
