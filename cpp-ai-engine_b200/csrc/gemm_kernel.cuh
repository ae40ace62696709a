// The fp32-accurate GEMM kernel for sm_100a.
//
//   C[b] = alpha * op(A[b]) x op(B[b]) + beta * C[b]          (row-major storage, fp32 in/out)
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Inside a CTA:
//
//   warp 0      TMA producer   one lane issues cp.async.bulk.tensor loads of the raw fp32
//                              A/B tiles of a k-block (BK = 32 or 16 values of k) into a
//                              shared-memory stage; transposed operands are loaded in their
//                              stored orientation and described to the tensor core as
//                              MN-major, so no transpose is ever materialised.
//   warps 4..11 workers        split every fp32 value of the stage IN PLACE into its TF32
//                              head (written back over the raw value) and TF32 tail (written
//                              to the second half of the stage).  The split is layout-blind:
//                              it never needs to know the swizzle or the orientation.
//                              The same warps later drain the TMEM accumulator.
//   warp 1      MMA issuer     one lane issues, per 8 values of k, three tcgen05.mma
//                              kind::tf32 products (tail x head, head x tail, head x head)
//                              into a TMEM accumulator, and commits to mbarriers.
//
// The tensor core's fp32 accumulator truncates: a chain of thousands of MMAs into one TMEM
// accumulator drifts (measured 2.9e-5 relative at K = 2048).  So the chain is cut every
// `promote_every` k-blocks: the MMA warp switches to the second TMEM accumulator while the
// workers pull the finished partial tile with tcgen05.ld and add it to fp32 registers with
// ordinary round-to-nearest adds.  The epilogue then writes alpha * acc + beta * C from
// registers.
//
// When an operand cannot be described to TMA (base not 16-byte aligned, leading dimension not a
// multiple of 4 floats: K = 9 im2col, N = 121 / 10 heads) the workers load it with plain
// global loads, split in registers and store straight into the K-major swizzled layout; the
// TMA warp idles.  Same MMA and epilogue code.
//
// Pair mode (kPair): two CTAs of a cluster form one 256 x BN tile.  Each CTA loads and splits
// 128 rows of A and HALF of the tile's B columns, and the leader CTA's MMA lane issues
// cta_group::2 products that read both CTAs' shared memory and write 128 accumulator rows
// into each CTA's TMEM.  Per CTA that cuts the shared-memory traffic of a k-block (raw tile
// in, head/tail out, operand fetches) by a third and the stage to 64 KB, so three stages fit.
// No TMA load is multicast: every CTA fetches only what it alone needs.
//
// Every wait is bounded (see sm100_ptx.cuh).  A wait that runs out records a bit in
// *status, raises a CTA-wide abort flag that all other waits poll, and every role falls
// through to the common exit where TMEM is released.
#pragma once

#include <type_traits>

#include "sm100_ptx.cuh"

namespace b200 {

constexpr int kBM = 128;          // tile rows = MMA M
constexpr int kWorkerWarps = 8;   // split + promote + epilogue
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kFirstWorkerWarp = 4;  // warps 0..3 form the control warpgroup (two of them idle)
constexpr int kThreads = kFirstWorkerWarp * 32 + kWorkerThreads;
constexpr int kMaxDest = 8;

// status bits (device-side wait that ran out, by role)
constexpr int kStatProducer = 1;
constexpr int kStatMma = 2;
constexpr int kStatWorkerFull = 4;
constexpr int kStatWorkerAcc = 8;
constexpr int kStatForwarder = 16;
constexpr int kStatSelfTest = 32;

struct GemmParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, kblocks, split_k, kb_per_split, group_m, total_work;
    const float* A;
    const float* B;
    float* dest[kMaxDest];  // dest[0] = C; further entries receive the same tiles (column-shard gather)
    int n_dest;
    long long lda, ldb, ldc, strideA, strideB, strideC;
    int transA, transB;
    float alpha, beta;
    int precision;      // 0 = 3xTF32, 1 = TF32
    // Multipliers that replace the scheduler's integer divisions (fast_div below): by split_k, by
    // the tiles of one matrix, by the tiles of one band, by the rows of a full band and of the last.
    unsigned long long fd_split, fd_tiles, fd_band, fd_rows, fd_rows_last;
    int promote_every;  // k-blocks per TMEM accumulation chain
    int tf32_round;     // TF32 mode with the TMA loader: 1 = workers round the tile to nearest first
    int trunc_hi;       // 3xTF32 with the TMA loader: 1 = the head is the tensor core's own truncation
    float* partial;     // split-K partials [split][batch][M][N] (split_k > 1)
    // fused epilogue: out = act(alpha*acc + beta*out + bias[col] + addend[row][col])
    const float* bias;    // N values, or null
    const float* addend;  // M x N (ld_addend), shared by every batch element, or null
    long long ld_addend;
    int relu;
    // implicit-GEMM convolution (conv kernels only): A is gathered from an NCHW input instead of a
    // stored column matrix, and the output is stored NCHW
    int cv_c, cv_h, cv_w, cv_kh, cv_kw, cv_stride, cv_pad, cv_oh, cv_ow;
    int cv_oc;        // output channels of the convolution (gradient kernels)
    int cv_table;     // 1: the gather runs from the per-CTA k tables (K <= kConvTableMax, offsets fit 32 bits)
    int cv_ones_col;  // weight gradient: this column of the column matrix is all ones (bias sums), or -1
    int cv_store_hw;  // pixels per image and channel of the tensor the NCHW store writes
    int tile_offset;    // first tile of this launch (tail-wave launches start past the full waves)
    int tail_tiles;     // > 0: partials are compact, [split][tail tile][tile rows][BN]
    int* status;
    // tensor-core view of the shared-memory tiles
    // k-step ks (8 values of k) of an operand tile starts (ks / 4) * ksub + (ks % 4) * kstep bytes into it:
    // a K-major tile wider than one 128-byte swizzle row (BK = 64) is two 32-wide sub-tiles side by side
    uint32_t a_lbo, a_sbo, a_kstep, a_ksub, a_layout;
    uint32_t b_lbo, b_sbo, b_kstep, b_ksub, b_layout;
    uint32_t idesc;
    // loader / epilogue fast paths
    int a_vec_ok, b_vec_ok, c_vec_ok;
};

template <int BN, int BK, bool kPair = false, int kWW = kWorkerWarps>
struct TileCfg {
    static_assert(kWW == 8 || kWW == 16, "eight or sixteen worker warps");
    static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
    static_assert(BK == 16 || BK == 32 || BK == 64, "unsupported k-block");
    static constexpr uint32_t kABytes = kBM * BK * 4;
    static constexpr int kBCols = kPair ? BN / 2 : BN;  // B columns held by one CTA
    static constexpr uint32_t kBBytes = kBCols * BK * 4;
    static constexpr uint32_t kHalf = kABytes + kBBytes;  // raw / head tiles; tails follow
    static constexpr uint32_t kStageBytes = 2 * kHalf;
    static constexpr int kMaxStages = (227 * 1024 - 2048 - kWorkerWarps * 4096) / kStageBytes;
    static constexpr int kStages = kMaxStages > 4 ? 4 : kMaxStages;
    static constexpr uint32_t kEpilogueBytes = kWorkerWarps * 4096;  // one 32 x 32 block per warp
    static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpilogueBytes + 1024;  // + alignment slack
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;           // two accumulators
    // Four warps cover the 128 accumulator rows (a warp reads the 32 TMEM lanes of its quarter), so
    // kWW / 4 warps share a row and split its columns.
    static constexpr int kColParts = kWW / 4;
    static constexpr int kCols = BN / kColParts;                          // columns per worker
    static constexpr int kWorkerThreadsCfg = kWW * 32;
    static constexpr int kThreadsCfg = kFirstWorkerWarp * 32 + kWW * 32;
    // the epilogue's staging area (kEpilogueBytes in all) is cut into one slot per worker warp:
    // 32 rows x kStageCols floats
    static constexpr int kStageCols = (kEpilogueBytes / kWW) / (32 * 4);
    static_assert(kStageCols == 32 || kStageCols == 16, "staging slot of 32 x 32 or 32 x 16 floats");
};

struct Work {
    int b, mt, nt, sp, kb0, kb1;
    int tile;  // linear tile index (batch included)
};

// n / d for 0 <= n < 2^31 as one 64 x 64 -> high-64 multiply by m = ceil(2^64 / d), exact for every
// 32-bit n (d = 1 is stored as m = 0).  The tile scheduler runs once per tile in three warps of
// every CTA; a small product executes it cold, and a hardware-free division is ~20 instructions.
__host__ __device__ inline unsigned long long fast_div_magic(int d) {
    return d <= 1 ? 0ull : (~0ull) / static_cast<unsigned long long>(d) + 1ull;
}
__device__ __forceinline__ int fast_div(int n, unsigned long long m) {
    return m ? static_cast<int>(__umul64hi(m, static_cast<unsigned long long>(static_cast<unsigned>(n)))) : n;
}

// Fills the multipliers from split_k, tiles_m, tiles_n and group_m (host side, before a launch).
inline void fill_schedule(GemmParams& p) {
    const int rows_last = p.tiles_m % p.group_m;
    p.fd_split = fast_div_magic(p.split_k);
    p.fd_tiles = fast_div_magic(p.tiles_m * p.tiles_n);
    p.fd_band = fast_div_magic(p.group_m * p.tiles_n);
    p.fd_rows = fast_div_magic(p.tiles_m < p.group_m ? p.tiles_m : p.group_m);
    p.fd_rows_last = fast_div_magic(rows_last ? rows_last : p.group_m);
}

__device__ __forceinline__ Work decode_work(const GemmParams& p, int w) {
    Work r;
    const int q = fast_div(w, p.fd_split);
    r.sp = w - q * p.split_k;
    int t = q + p.tile_offset;
    r.tile = t;
    const int tiles = p.tiles_m * p.tiles_n;
    r.b = fast_div(t, p.fd_tiles);
    t -= r.b * tiles;
    // Tiles are walked in bands of group_m tile-rows so that the CTAs running at one time
    // cover a near-square patch of C and share A and B tiles through L2.
    const int per_group = p.group_m * p.tiles_n;
    const int g = fast_div(t, p.fd_band);
    const int first_m = g * p.group_m;
    const int gsize = min(p.tiles_m - first_m, p.group_m);
    const int in_g = t - g * per_group;
    r.nt = fast_div(in_g, first_m + p.group_m <= p.tiles_m ? p.fd_rows : p.fd_rows_last);
    r.mt = first_m + in_g - r.nt * gsize;
    r.kb0 = r.sp * p.kb_per_split;
    r.kb1 = min(p.kblocks, r.kb0 + p.kb_per_split);
    return r;
}

// kCluster: the barrier is also arrived on by the peer CTA, whose writes must be acquired.
template <bool kCluster = false>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                         int* status, int code, uint64_t budget_ns = kWaitBudgetNs) {
    auto probe = [&]() { return kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (probe()) return true;
    const uint64_t start = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (probe()) return true;
        }
        if (*abort_flag) return false;
        if (global_timer_ns() - start > budget_ns) {
            atomicOr(status, code);
            *abort_flag = 1;
            return false;
        }
    }
}

// The fused part of the epilogue, in the order the reference applies its separate operations
// to a product: bias broadcast add (src/nn.cpp:120-122, src/conv.cpp:323), additive mask
// (src/transformer.cpp:296); then the accumulation into an existing output; ReLU last
// (src/transformer.cpp:413).
__device__ __forceinline__ float add_bias_mask(const GemmParams& p, float v, int row, int col) {
    if (p.bias) v += __ldg(p.bias + col);
    if (p.addend) v += __ldg(p.addend + (long long)row * p.ld_addend + col);
    return v;
}
__device__ __forceinline__ float finish_output(const GemmParams& p, float scaled, float old, int row,
                                               int col) {
    float v = add_bias_mask(p, scaled, row, col);
    if (p.beta != 0.f) v += p.beta * old;
    return p.relu ? fmaxf(v, 0.0f) : v;
}

// Loads a ROWS x 32 tile of one operand with plain global loads, splits it and stores the
// head / tail tiles in the K-major 128-byte-swizzled layout.  `k_contig`: k is the contiguous
// index of the stored matrix (A not transposed, B transposed).
template <int ROWS, bool kLoad, bool kStore>
__device__ __forceinline__ void ldg_split_store(const float* __restrict__ base, long long ld,
                                                bool k_contig, bool vec_ok, int row0, int row_max,
                                                int k0, int K, uint8_t* hi, uint8_t* lo,
                                                bool want_lo, int wtid, float4* v) {
    constexpr int kChunks = 8;  // 16-byte chunks per 128-byte row
    constexpr int kUnits = ROWS * kChunks;
    constexpr int kPer = kUnits / kWorkerThreads;
    static_assert(kUnits % kWorkerThreads == 0, "tile does not divide over the workers");
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            int r, c;
            if (k_contig) {
                r = unit / kChunks;
                c = unit % kChunks;
            } else {
                r = unit % ROWS;
                c = unit / ROWS;
            }
            const int gr = row0 + r;
            const int gk = k0 + c * 4;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gr < row_max && gk < K) {
                if (k_contig) {
                    const float* src = base + (long long)gr * ld + gk;
                    if (vec_ok && gk + 3 < K) {
                        x = __ldg(reinterpret_cast<const float4*>(src));
                    } else {
                        x.x = __ldg(src);
                        if (gk + 1 < K) x.y = __ldg(src + 1);
                        if (gk + 2 < K) x.z = __ldg(src + 2);
                        if (gk + 3 < K) x.w = __ldg(src + 3);
                    }
                } else {
                    const float* src = base + (long long)gk * ld + gr;
                    x.x = __ldg(src);
                    if (gk + 1 < K) x.y = __ldg(src + ld);
                    if (gk + 2 < K) x.z = __ldg(src + 2 * ld);
                    if (gk + 3 < K) x.w = __ldg(src + 3 * ld);
                }
            }
            v[u] = x;
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            int r, c;
            if (k_contig) {
                r = unit / kChunks;
                c = unit % kChunks;
            } else {
                r = unit % ROWS;
                c = unit / ROWS;
            }
            const uint32_t off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u +
                                 (uint32_t)((c ^ (r & 7)) << 4);
            float4 h, l;
            tf32_split(v[u].x, h.x, l.x);
            tf32_split(v[u].y, h.y, l.y);
            tf32_split(v[u].z, h.z, l.z);
            tf32_split(v[u].w, h.w, l.w);
            *reinterpret_cast<float4*>(hi + off) = h;
            if (want_lo) *reinterpret_cast<float4*>(lo + off) = l;
        }
    }
}

// Implicit im2col: the 128 x 32 A tile of a convolution, gathered straight from the NCHW input
// (what nn::im2col would have written to row m = (n, oh, ow), column k = (c, kh, kw),
// src/conv.cpp:61-150; zero outside the padded border), split and stored like any A tile.
// Consecutive threads take consecutive output pixels, which are consecutive input addresses
// for stride 1.
template <bool kLoad, bool kStore>
__device__ __forceinline__ void conv_gather_split_store(const GemmParams& p, int row0, int k0,
                                                        uint8_t* hi, uint8_t* lo, bool want_lo,
                                                        int wtid, float4* v) {
    constexpr int kUnits = kBM * 8;
    constexpr int kPer = kUnits / kWorkerThreads;
    const int ohw = p.cv_oh * p.cv_ow;
    const int khw = p.cv_kh * p.cv_kw;
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit % kBM, c = unit / kBM;
            const int gr = row0 + r;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
            if (gr < p.M) {
                const int img = gr / ohw, pix = gr - img * ohw;
                const int oh = pix / p.cv_ow, ow = pix - oh * p.cv_ow;
                const int ih0 = oh * p.cv_stride - p.cv_pad, iw0 = ow * p.cv_stride - p.cv_pad;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int gk = k0 + c * 4 + e;
                    if (gk < p.K) {
                        const int ci = gk / khw, rem = gk - ci * khw;
                        const int kh = rem / p.cv_kw, kw = rem - kh * p.cv_kw;
                        const int ih = ih0 + kh, iw = iw0 + kw;
                        if (ih >= 0 && ih < p.cv_h && iw >= 0 && iw < p.cv_w) {
                            x4[e] = __ldg(p.A + (((long long)img * p.cv_c + ci) * p.cv_h + ih) * p.cv_w + iw);
                        }
                    }
                }
            }
            v[u] = make_float4(x4[0], x4[1], x4[2], x4[3]);
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit % kBM, c = unit / kBM;
            const uint32_t off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u +
                                 (uint32_t)((c ^ (r & 7)) << 4);
            float4 h, l;
            tf32_split(v[u].x, h.x, l.x);
            tf32_split(v[u].y, h.y, l.y);
            tf32_split(v[u].z, h.z, l.z);
            tf32_split(v[u].w, h.w, l.w);
            *reinterpret_cast<float4*>(hi + off) = h;
            if (want_lo) *reinterpret_cast<float4*>(lo + off) = l;
        }
    }
}

// Stores one unit (4 consecutive k of one tile row) of a K-major swizzled tile, split.
__device__ __forceinline__ void store_unit_split(uint8_t* hi, uint8_t* lo, bool want_lo, int r, int c,
                                                 const float4& v) {
    const uint32_t off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u + (uint32_t)((c ^ (r & 7)) << 4);
    float4 h, l;
    tf32_split(v.x, h.x, l.x);
    tf32_split(v.y, h.y, l.y);
    tf32_split(v.z, h.z, l.z);
    tf32_split(v.w, h.w, l.w);
    *reinterpret_cast<float4*>(hi + off) = h;
    if (want_lo) *reinterpret_cast<float4*>(lo + off) = l;
}

// Table-driven gather of a convolution's A tile (forward: from x; input gradient with stride 1:
// from dy).  Element (row, k) of the tile is  src[row.base + koff[k]]  when
// 0 <= row.y + dy[k] < ymax and 0 <= row.x + dx[k] < xmax, else zero, where
//   forward:         row = (n, oh, ow):  base = n*C*H*W + y*W + x,  (y, x) = (oh*s - pad, ow*s - pad);
//                    k = (c, kh, kw):    koff = c*H*W + kh*W + kw,  (dy, dx) = (kh, kw);  limits (H, W)
//   input gradient:  row = (n, ih, iw):  base = n*O*oH*oW + y*oW + x,  (y, x) = (ih + pad, iw + pad);
//                    k = (o, kh, kw):    koff = o*oH*oW - kh*oW - kw,  (dy, dx) = (-kh, -kw);  limits (oH, oW).
// The k side is the same for every row of every tile: each CTA writes it once into two tables in
// the epilogue's staging area (these kernels store NCHW straight from registers and leave it
// free); the row side is computed once per tile.  What is left per element is two adds and two
// unsigned compares instead of four divisions.
constexpr int kConvTableMax = kWorkerWarps * 4096 / 8;  // k values the two tables hold
constexpr int kConvDeltaBias = 32768;                   // (dy, dx) are stored + bias in 16 bits each

struct ConvRow {
    long long base;
    int y, x;  // already minus kConvDeltaBias; a row past M gets a y that fails every compare
};

template <bool kLoad, bool kStore>
__device__ __forceinline__ void conv_table_gather_split_store(const float* __restrict__ src, const int* koff,
                                                              const uint32_t* kdelta, const ConvRow& row,
                                                              uint32_t ymax, uint32_t xmax, int k0, int K,
                                                              uint8_t* hi, uint8_t* lo, bool want_lo, int wtid,
                                                              float4* v) {
    constexpr int kPer = kBM * 8 / kWorkerThreads;
    static_assert(kWorkerThreads % kBM == 0, "a worker keeps one tile row");
    const int r = wtid % kBM;
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int c = wtid / kBM + u * (kWorkerThreads / kBM);
            const int gk = k0 + c * 4;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
            if (gk < K) {  // the tables are padded to a multiple of 4 with entries that fail the compares
                const int4 ko = *reinterpret_cast<const int4*>(koff + gk);
                const uint4 kd = *reinterpret_cast<const uint4*>(kdelta + gk);
                const int ko4[4] = {ko.x, ko.y, ko.z, ko.w};
                const uint32_t kd4[4] = {kd.x, kd.y, kd.z, kd.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t ty = static_cast<uint32_t>(row.y + static_cast<int>(kd4[e] >> 16));
                    const uint32_t tx = static_cast<uint32_t>(row.x + static_cast<int>(kd4[e] & 0xffffu));
                    if (ty < ymax && tx < xmax) x4[e] = __ldg(src + row.base + ko4[e]);
                }
            }
            v[u] = make_float4(x4[0], x4[1], x4[2], x4[3]);
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            store_unit_split(hi, lo, want_lo, r, wtid / kBM + u * (kWorkerThreads / kBM), v[u]);
        }
    }
}


// Weight gradient of a convolution, dW (outC x C*kH*kW) = dOut^T x cols, with neither dOut^T nor
// cols ever written (the reference's backward of `cols.matmul(W^T)`, src/tensor_ops.cpp:570-585,
// materialises cols^T and multiplies by the (N*spatial, outC) gradient).  The contraction runs
// over the output positions m = (n, oh, ow).
//
// A tile: row = output channel o, k = m, read from dy (N, outC, oH, oW): for one channel,
// consecutive m of an image are consecutive floats.  Rows past outC are left as they are: they
// feed accumulator rows that are never stored.
template <bool kLoad, bool kStore>
__device__ __forceinline__ void conv_dy_rows_split_store(const GemmParams& p, int row0, int k0, uint8_t* hi,
                                                         uint8_t* lo, bool want_lo, int wtid, float4* v) {
    constexpr int kPer = kBM * 8 / kWorkerThreads;
    const int ohw = p.cv_oh * p.cv_ow;
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit >> 3, c = unit & 7;
            const int o = row0 + r, m0 = k0 + c * 4;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
            if (o < p.M && m0 < p.K) {
                const int img = m0 / ohw, sp = m0 - img * ohw;
                const float* src = p.A + ((long long)img * p.M + o) * ohw + sp;
                if (p.a_vec_ok) {  // ohw % 4 == 0: the four positions lie in one image, 16-byte aligned
                    const float4 t = __ldg(reinterpret_cast<const float4*>(src));
                    x4[0] = t.x, x4[1] = t.y, x4[2] = t.z, x4[3] = t.w;
                } else {
                    int ii = img, ss = sp;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (m0 + e < p.K) x4[e] = __ldg(p.A + ((long long)ii * p.M + o) * ohw + ss);
                        if (++ss == ohw) ss = 0, ++ii;
                    }
                }
            }
            v[u] = make_float4(x4[0], x4[1], x4[2], x4[3]);
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit >> 3, c = unit & 7;
            if (row0 + r < p.M) store_unit_split(hi, lo, want_lo, r, c, v[u]);
        }
    }
}

// B tile of the weight gradient: row = column kc = (c, kh, kw) of the column matrix, k = m,
// gathered from x (N, C, H, W) exactly as nn::im2col would have filled cols[m][kc]
// (src/conv.cpp:61-150).  Rows past C*kH*kW are left as they are (columns that are never stored).
template <int ROWS, bool kLoad, bool kStore>
__device__ __forceinline__ void conv_cols_T_split_store(const GemmParams& p, int row0, int k0, uint8_t* hi,
                                                        uint8_t* lo, bool want_lo, int wtid, float4* v) {
    constexpr int kPer = ROWS * 8 / kWorkerThreads;
    const int ohw = p.cv_oh * p.cv_ow, khw = p.cv_kh * p.cv_kw;
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit >> 3, c = unit & 7;
            const int kc = row0 + r, m0 = k0 + c * 4;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
            if (kc == p.cv_ones_col) {
                // the bias gradient rides along as one more column of the column matrix: dOut^T x 1
#pragma unroll
                for (int e = 0; e < 4; ++e) x4[e] = (m0 + e < p.K) ? 1.0f : 0.0f;
            } else if (kc < p.N && m0 < p.K) {
                const int ci = kc / khw, rem = kc - ci * khw;
                const int kh = rem / p.cv_kw, kw = rem - kh * p.cv_kw;
                int img = m0 / ohw;
                const int pix = m0 - img * ohw;
                int oh = pix / p.cv_ow, ow = pix - oh * p.cv_ow;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (m0 + e < p.K) {
                        const int ih = oh * p.cv_stride - p.cv_pad + kh, iw = ow * p.cv_stride - p.cv_pad + kw;
                        if (ih >= 0 && ih < p.cv_h && iw >= 0 && iw < p.cv_w)
                            x4[e] = __ldg(p.B + (((long long)img * p.cv_c + ci) * p.cv_h + ih) * p.cv_w + iw);
                    }
                    if (++ow == p.cv_ow) {
                        ow = 0;
                        if (++oh == p.cv_oh) oh = 0, ++img;
                    }
                }
            }
            v[u] = make_float4(x4[0], x4[1], x4[2], x4[3]);
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit >> 3, c = unit & 7;
            if (row0 + r < p.N) store_unit_split(hi, lo, want_lo, r, c, v[u]);
        }
    }
}

// Input gradient of a convolution as ONE gather product (the reference forms dCols = dOut x W and
// scatters it with col2im, src/conv.cpp:152-222, summing the overlaps):
//   dx[n][c][ih][iw] = sum over (o, kh, kw) of dy[n][o][(ih+pad-kh)/s][(iw+pad-kw)/s] * W[o][c][kh][kw]
// taken over the terms whose divisions are exact and land inside dy.
//
// A tile: row = input pixel m' = (n, ih, iw), k = (o, kh, kw), gathered from dy.
template <bool kLoad, bool kStore>
__device__ __forceinline__ void conv_dx_gather_split_store(const GemmParams& p, int row0, int k0, uint8_t* hi,
                                                           uint8_t* lo, bool want_lo, int wtid, float4* v) {
    constexpr int kPer = kBM * 8 / kWorkerThreads;
    const int hw = p.cv_h * p.cv_w, khw = p.cv_kh * p.cv_kw;
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit % kBM, c = unit / kBM;
            const int gr = row0 + r;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
            if (gr < p.M) {
                const int img = gr / hw, pix = gr - img * hw;
                const int ih = pix / p.cv_w, iw = pix - ih * p.cv_w;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int gk = k0 + c * 4 + e;
                    if (gk < p.K) {
                        const int o = gk / khw, rem = gk - o * khw;
                        const int kh = rem / p.cv_kw, kw = rem - kh * p.cv_kw;
                        int ty = ih + p.cv_pad - kh, tx = iw + p.cv_pad - kw;
                        bool hit = ty >= 0 && tx >= 0;
                        if (p.cv_stride != 1 && hit) {
                            const int oy = ty / p.cv_stride, ox = tx / p.cv_stride;
                            hit = oy * p.cv_stride == ty && ox * p.cv_stride == tx;
                            ty = oy, tx = ox;
                        }
                        if (hit && ty < p.cv_oh && tx < p.cv_ow)
                            x4[e] = __ldg(p.A + (((long long)img * p.cv_oc + o) * p.cv_oh + ty) * p.cv_ow + tx);
                    }
                }
            }
            v[u] = make_float4(x4[0], x4[1], x4[2], x4[3]);
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            store_unit_split(hi, lo, want_lo, unit % kBM, unit / kBM, v[u]);
        }
    }
}

// B tile of the input gradient: row = input channel c, k = (o, kh, kw), read from the weight
// (outC, C, kH, kW) as it is stored.  Rows past C are left as they are.
template <int ROWS, bool kLoad, bool kStore>
__device__ __forceinline__ void conv_weight_T_split_store(const GemmParams& p, int row0, int k0, uint8_t* hi,
                                                          uint8_t* lo, bool want_lo, int wtid, float4* v) {
    constexpr int kPer = ROWS * 8 / kWorkerThreads;
    const int khw = p.cv_kh * p.cv_kw;
    if constexpr (kLoad) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit >> 3, c = unit & 7;
            const int ci = row0 + r;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
            if (ci < p.N) {
                int gk = k0 + c * 4;
                int o = gk / khw, q = gk - o * khw;
#pragma unroll
                for (int e = 0; e < 4; ++e, ++gk) {
                    if (gk < p.K) x4[e] = __ldg(p.B + ((long long)o * p.cv_c + ci) * khw + q);
                    if (++q == khw) q = 0, ++o;
                }
            }
            v[u] = make_float4(x4[0], x4[1], x4[2], x4[3]);
        }
    }
    if constexpr (kStore) {
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int unit = wtid + u * kWorkerThreads;
            const int r = unit >> 3, c = unit & 7;
            if (row0 + r < p.N) store_unit_split(hi, lo, want_lo, r, c, v[u]);
        }
    }
}

// Splits one landed stage in place: the raw fp32 tile becomes the head tile, the tail tile is written
// kHalf bytes further on.  kN4 16-byte chunks are shared out over kT threads.  A thread's chunks are
// loaded first, up to kMaxBatch at a time, and split and stored afterwards: written as one loop
// (load, split, store, next chunk) the stores of one chunk may alias the load of the next as far as
// the compiler can tell, and every chunk would pay a full shared-memory round trip.
template <int kN4, int kT, int kMaxBatch>
__device__ __forceinline__ void split_stage(float4* hi, float4* lo, int tid, bool prec3, bool tail_only) {
    constexpr int kPer = (kN4 + kT - 1) / kT;  // chunks per thread
    constexpr int kBatch = kPer < kMaxBatch ? kPer : kMaxBatch;
#pragma unroll
    for (int u0 = 0; u0 < kPer; u0 += kBatch) {
        float4 x[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int q = tid + (u0 + u) * kT;
            if (u0 + u < kPer && ((u0 + u + 1) * kT <= kN4 || q < kN4)) x[u] = hi[q];
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int q = tid + (u0 + u) * kT;
            if (u0 + u < kPer && ((u0 + u + 1) * kT <= kN4 || q < kN4)) {
                if (tail_only) {
                    // The raw tile stays as it is: the tensor core drops the low 13 mantissa bits of
                    // what it reads, so its head is trunc(x); only the tail x - trunc(x) (exact in
                    // fp32, then rounded to TF32) is written — one pass of shared-memory stores
                    // instead of two.
                    lo[q] = make_float4(tf32_tail_of_truncated(x[u].x), tf32_tail_of_truncated(x[u].y),
                                        tf32_tail_of_truncated(x[u].z), tf32_tail_of_truncated(x[u].w));
                } else {
                    float4 h, l;
                    tf32_split(x[u].x, h.x, l.x);
                    tf32_split(x[u].y, h.y, l.y);
                    tf32_split(x[u].z, h.z, l.z);
                    tf32_split(x[u].w, h.w, l.w);
                    hi[q] = h;
                    if (prec3) lo[q] = l;
                }
            }
        }
    }
}

// kConv: 0 a plain product; 1 convolution forward (A gathered from x, NCHW store); 2 weight
// gradient (both operands gathered, contraction over the output positions, plain store);
// 3 input gradient (A gathered from dy, B from the weight, NCHW store).
// kWW: worker warps (8, or 16 for the large pair tiles: twice the warps per scheduler to hide the
// latency of the split's and the drain's dependent instruction chains, half the accumulators each).
// kSW: warps that do nothing but split the landed stages (0, or 8 for the pair tiles).  With them the kWW
// worker warps only drain the accumulator and store: the two dependent chains of a k-block — split,
// hand over to the tensor core; wait for it, add its partial sum into registers — run side by side
// on different warps instead of one after the other in each worker.
template <int BN, int BK, bool kTma, bool kPair = false, int kConv = 0, int kWW = kWorkerWarps, int kSW = 0>
__global__ void __launch_bounds__((kFirstWorkerWarp + kWW + kSW) * 32, 1)
gemm_tf32_kernel(const GemmParams p, const __grid_constant__ CUtensorMap mapA,
                 const __grid_constant__ CUtensorMap mapB) {
    using Cfg = TileCfg<BN, BK, kPair, kWW>;
    constexpr int kWT = kWW * 32;  // worker threads
    static_assert(kWW == kWorkerWarps || (kTma && kConv == 0), "sixteen workers: TMA loader, plain product");
    static_assert(kSW == 0 || (kSW == 8 && kWW == 8 && kTma && kConv == 0 && BN == 256),
                  "split warps: TMA loader, plain product, 256-wide tiles");
    // registers per thread at launch (what ptxas reports for the launch bounds) and of a split warp
    constexpr int kLaunchRegs = (kSW > 0 || kWW == 16) ? 96 : 168;
    constexpr int kSplitRegs = 40;
    constexpr int kSplitters = kSW > 0 ? kSW : kWW;  // warps that hand a split stage to the tensor core
    constexpr int kStages = Cfg::kStages;
    constexpr int kCols = Cfg::kCols;
    constexpr int kTileM = kPair ? 2 * kBM : kBM;        // rows of C per tile
    constexpr int kArrivals = kPair ? 2 * kWW : kWW;
    constexpr int kSplitArrivals = kPair ? 2 * kSplitters : kSplitters;
    static_assert(kTma || BK == 32, "the register-staged loader writes 128-byte rows");
    static_assert(!kPair || kTma, "pair mode loads with TMA");
    static_assert(kConv == 0 || !kTma, "the convolution gathers its operands in registers");
    // the workers of the widest tiles (and of the register-staged loader, which also holds the next
    // k-block in registers) take the control warpgroup's spare registers
    constexpr bool kMoveRegs = BN == 256 || (!kTma && BN == 128);

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    __shared__ __align__(8) uint64_t full_bar[kStages];   // TMA bytes landed
    __shared__ __align__(8) uint64_t split_bar[kStages];  // head/tail tiles ready for the MMA
    __shared__ __align__(8) uint64_t empty_bar[kStages];  // MMAs reading the stage finished
    __shared__ __align__(8) uint64_t accf_bar[2];         // accumulator chain finished
    __shared__ __align__(8) uint64_t acce_bar[2];         // accumulator drained
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ uint32_t fwd_count_s;  // worker warps that have stored their part of a tile (column-shard gather)

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &abort_s;
    // In pair mode the two CTAs of a cluster walk the same tiles; CTA 0 is the leader.
    const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
    const int first_work = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int work_stride = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&split_bar[s]), kSplitArrivals);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&accf_bar[b]), 1);
            mbar_init(smem_u32(&acce_bar[b]), kArrivals);
        }
        abort_s = 0;
        fwd_count_s = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        __syncwarp();
        if constexpr (kPair) {
            tmem_alloc_pair(smem_u32(&tmem_base_s), Cfg::kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(&tmem_base_s), Cfg::kTmemCols);
            tmem_relinquish();
        }
    }
    if (kTma && warp == 0 && lane == 0) {
        tma_prefetch_desc(&mapA);
        tma_prefetch_desc(&mapB);
    }
    tc_fence_before_sync();
    if constexpr (kPair) {
        __syncwarp();
        cluster_sync();  // both CTAs' barriers exist before either signals the other
    } else {
        __syncthreads();
    }
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    // Everything above (barriers, tensor memory, descriptor prefetch) touched no global data and may
    // have run while the previous kernel of the stream was still finishing; from here on this
    // kernel reads and writes memory that kernel may own.
    grid_dependency_wait();
    const bool prec3 = (p.precision == 0);
    const int promote_every = p.promote_every;

    // The 128 x 256 tile keeps 128 accumulators per worker thread in registers: hand the
    // control warpgroup's registers to the two worker warpgroups.
    if (warp < kFirstWorkerWarp) {
      if constexpr (kMoveRegs) reg_dealloc<40>();
      if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (kTma && lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int w = first_work; w < p.total_work && ok; w += work_stride) {
                const Work wk = decode_work(p, w);
                const int za = p.strideA ? wk.b : 0;
                const int zb = p.strideB ? wk.b : 0;
                for (int kb = wk.kb0; kb < wk.kb1; ++kb, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    {
                        const bool got = wait_bar(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag,
                                                  p.status, kStatProducer);
                        if (!got) {
                            ok = false;
                            break;
                        }
                    }
                    const uint32_t full = smem_u32(&full_bar[s]);
                    const uint32_t sa = smem_u32(smem) + s * Cfg::kStageBytes;
                    const uint32_t sb = sa + Cfg::kABytes;
                    mbar_arrive_expect_tx(full, Cfg::kHalf);
                    const int row0 = wk.mt * kTileM + static_cast<int>(cta_rank) * kBM;
                    const int col0 = wk.nt * BN + static_cast<int>(cta_rank) * Cfg::kBCols;
                    if (!p.transA) {  // K-major: one box of 32 k per 128-byte swizzle row
#pragma unroll
                        for (int h = 0; h < (BK + 31) / 32; ++h)
                            tma_load_3d(sa + h * (kBM * 128), &mapA, full, kb * BK + h * 32, row0, za);
                    } else {
#pragma unroll
                        for (int j = 0; j < kBM / 32; ++j)
                            tma_load_3d(sa + j * (BK * 128), &mapA, full, row0 + j * 32, kb * BK, za);
                    }
                    if (p.transB) {
#pragma unroll
                        for (int h = 0; h < (BK + 31) / 32; ++h)
                            tma_load_3d(sb + h * (Cfg::kBCols * 128), &mapB, full, kb * BK + h * 32, col0, zb);
                    } else {
#pragma unroll
                        for (int j = 0; j < Cfg::kBCols / 32; ++j)
                            tma_load_3d(sb + j * (BK * 128), &mapB, full, col0 + j * 32, kb * BK, zb);
                    }
                }
            }
            if (!ok) {
                // Leave no bulk copy in flight behind an exiting CTA: give the loads already
                // issued a short while to land.
                for (uint32_t back = 1; back <= (uint32_t)kStages && back <= it; ++back) {
                    const uint32_t j = it - back;
                    mbar_wait(smem_u32(&full_bar[j % kStages]), (j / kStages) & 1, 20000000ull);
                }
            }
        }
      } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && cta_rank == 0) {
            const uint32_t s0 = smem_u32(smem);
            const uint64_t dA_hi = make_smem_desc(s0, p.a_lbo, p.a_sbo, p.a_layout);
            const uint64_t dB_hi = make_smem_desc(s0 + Cfg::kABytes, p.b_lbo, p.b_sbo, p.b_layout);
            // descriptor offset (16-byte units) of k-step ks within an operand tile
            const uint32_t a_kstep = p.a_kstep >> 4, a_ksub = p.a_ksub >> 4;
            const uint32_t b_kstep = p.b_kstep >> 4, b_ksub = p.b_ksub >> 4;
            auto a_off = [&](int ks) { return static_cast<uint32_t>(ks >> 2) * a_ksub + static_cast<uint32_t>(ks & 3) * a_kstep; };
            auto b_off = [&](int ks) { return static_cast<uint32_t>(ks >> 2) * b_ksub + static_cast<uint32_t>(ks & 3) * b_kstep; };
            constexpr uint32_t kLoOff = Cfg::kHalf >> 4;
            const uint32_t idesc = p.idesc;
            auto issue_mma = [](uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t accum) {
                if constexpr (kPair) {
                    mma_tf32_ss_pair(d, a, b, id, accum);
                } else {
                    mma_tf32_ss(d, a, b, id, accum);
                }
            };
            // completion of everything issued so far -> the barrier at this offset in the CTA
            // (in both CTAs of a pair)
            auto signal_done = [](uint32_t bar) {
                if constexpr (kPair) {
                    tc_commit_pair(bar, 3);
                } else {
                    tc_commit(bar);
                }
            };
            uint32_t it = 0, chain = 0;
            bool ok = true;
            for (int w = first_work; w < p.total_work && ok; w += work_stride) {
                const Work wk = decode_work(p, w);
                const int nkb = wk.kb1 - wk.kb0;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    const bool chain_start = (i % promote_every) == 0;
                    const bool chain_end = ((i + 1) % promote_every) == 0 || i == nkb - 1;
                    const uint32_t buf = chain & 1;
                    if (chain_start) {
                        const bool got = wait_bar<kPair>(smem_u32(&acce_bar[buf]),
                                                         ((chain >> 1) & 1) ^ 1, abort_flag,
                                                         p.status, kStatMma);
                        if (!got) {
                            ok = false;
                            break;
                        }
                    }
                    {
                        const bool got = wait_bar<kPair>(smem_u32(&split_bar[s]), ph, abort_flag,
                                                         p.status, kStatMma);
                        if (!got) {
                            ok = false;
                            break;
                        }
                    }
                    tc_fence_after_sync();
                    const uint32_t d = tmem + buf * BN;
                    const uint32_t soff = (s * Cfg::kStageBytes) >> 4;
                    uint32_t accumulate = chain_start ? 0u : 1u;
                    if (prec3) {
                        // The accumulator truncates after every MMA, by an amount relative to
                        // its magnitude.  The two correction products are ~2^-11 of the head
                        // product: issue all of them first, while the accumulator is still
                        // tiny, so that only the BK/8 head products truncate at full scale.
#pragma unroll
                        for (int ks = 0; ks < BK / 8; ++ks) {
                            const uint64_t ah = dA_hi + (soff + a_off(ks));
                            const uint64_t bh = dB_hi + (soff + b_off(ks));
                            issue_mma(d, ah + kLoOff, bh, idesc, accumulate);
                            issue_mma(d, ah, bh + kLoOff, idesc, 1u);
                            accumulate = 1u;
                        }
                    }
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ++ks) {
                        const uint64_t ah = dA_hi + (soff + a_off(ks));
                        const uint64_t bh = dB_hi + (soff + b_off(ks));
                        issue_mma(d, ah, bh, idesc, accumulate);
                        accumulate = 1u;
                    }
                    signal_done(smem_u32(&empty_bar[s]));
                    if (chain_end) {
                        signal_done(smem_u32(&accf_bar[buf]));
                        ++chain;
                    }
                }
            }
        }
      } else if constexpr (kConv == 0) {
        // ------------------------------------------------------------------ forwarders (warps 2, 3)
        // Column-shard gather: the workers store a finished tile into this GPU's own C and go
        // straight back to splitting; these two otherwise idle warps then copy the tile from
        // there (it is still in L2) into every peer's C with plain stores over NVLink.  A store
        // to a peer is posted, but an SM can only keep so many in flight: issued by the workers,
        // seven remote copies per tile stalled the whole pipeline once per tile.  The source is
        // global memory that nobody overwrites during the launch, so the forwarders may fall
        // any number of tiles behind; they catch up under the next tiles' math.
        if (p.n_dest > 1) {
            const int ftid = static_cast<int>(threadIdx.x) - 64;
            const uint32_t cnt = smem_u32(&fwd_count_s);
            uint32_t target = 0;
            bool ok = true;
            for (int w = first_work; w < p.total_work && ok; w += work_stride) {
                const Work wk = decode_work(p, w);
                target += kWW;
                if (smem_load_acquire(cnt) < target) {
                    const uint64_t start = global_timer_ns();
                    for (;;) {
                        if (smem_load_acquire(cnt) >= target) break;
                        if (*abort_flag) {
                            ok = false;
                            break;
                        }
                        if (global_timer_ns() - start > kWaitBudgetNs) {
                            atomicOr(p.status, kStatForwarder);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        __nanosleep(256);
                    }
                    if (!ok) break;
                }
                const int row0 = wk.mt * kTileM + static_cast<int>(cta_rank) * kBM;
                const int col0 = wk.nt * BN;
                const long long boff = (long long)wk.b * p.strideC;
                if (p.c_vec_ok && (p.N & 3) == 0) {
                    constexpr int kC4 = BN / 4;              // 16-byte chunks per tile row
                    constexpr int kPasses = kBM * kC4 / 64;  // chunks per forwarder thread
                    static_assert(kPasses % 2 == 0, "the copy loop is unrolled by two");
                    // (the control warps run on 40 registers: two chunks in flight per thread)
#pragma unroll 1
                    for (int i0 = 0; i0 < kPasses; i0 += 2) {
                        const int u0 = ftid + i0 * 64, u1 = u0 + 64;
                        const int r0 = row0 + u0 / kC4, c0 = col0 + (u0 % kC4) * 4;
                        const int r1 = row0 + u1 / kC4, c1 = col0 + (u1 % kC4) * 4;
                        const bool in0 = r0 < p.M && c0 < p.N, in1 = r1 < p.M && c1 < p.N;
                        const long long off0 = boff + (long long)r0 * p.ldc + c0;
                        const long long off1 = boff + (long long)r1 * p.ldc + c1;
                        float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
                        if (in0) v0 = __ldcg(reinterpret_cast<const float4*>(p.dest[0] + off0));
                        if (in1) v1 = __ldcg(reinterpret_cast<const float4*>(p.dest[0] + off1));
#pragma unroll 1
                        for (int dd = 1; dd < p.n_dest; ++dd) {
                            float* dst = p.dest[dd];
                            if (in0) *reinterpret_cast<float4*>(dst + off0) = v0;
                            if (in1) *reinterpret_cast<float4*>(dst + off1) = v1;
                        }
                    }
                } else {
                    for (int u = ftid; u < kBM * BN; u += 64) {
                        const int row = row0 + u / BN, col = col0 + u % BN;
                        if (row < p.M && col < p.N) {
                            const long long off = boff + (long long)row * p.ldc + col;
                            const float v = __ldcg(p.dest[0] + off);
                            for (int dd = 1; dd < p.n_dest; ++dd) p.dest[dd][off] = v;
                        }
                    }
                }
            }
        }
      }
    } else if (kSW > 0 && warp >= kFirstWorkerWarp + kWW) {
        // ------------------------------------------------------------------ split warps
        if constexpr (kSW > 0) {
            reg_dealloc<kSplitRegs>();
            constexpr int kST = kSW * 32;
            const int stid = static_cast<int>(threadIdx.x) - (kFirstWorkerWarp + kWW) * 32;
            uint32_t it = 0;
            bool ok = true;
            for (int w = first_work; w < p.total_work && ok; w += work_stride) {
                const Work wk = decode_work(p, w);
                for (int kb = wk.kb0; kb < wk.kb1; ++kb, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    bool got = wait_bar(smem_u32(&full_bar[s]), ph, abort_flag, p.status, kStatWorkerFull);
                    got = __all_sync(0xffffffffu, got);
                    if (!got) {
                        ok = false;
                        break;
                    }
                    uint8_t* stage = smem + s * Cfg::kStageBytes;
                    constexpr int kN4 = Cfg::kHalf / 16;
                    if (prec3 || p.tf32_round)
                        split_stage<kN4, kST, 4>(reinterpret_cast<float4*>(stage),
                                                 reinterpret_cast<float4*>(stage + Cfg::kHalf), stid, prec3,
                                                 prec3 && p.trunc_hi);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (kPair) {
                            mbar_arrive_cluster(map_to_cta(smem_u32(&split_bar[s]), 0));
                        } else {
                            mbar_arrive(smem_u32(&split_bar[s]));
                        }
                    }
                }
            }
            grid_launch_dependents();
        }
    } else {
        // ------------------------------------------------------------------ workers
        // setmaxnreg.inc can only take what setmaxnreg.dec released INSIDE THIS CTA (the pool is per CTA,
        // not the SM's free registers), and blocks until it gets it: what the control warpgroup (and the
        // split warps) give up must cover the workers' increase.
        //   8 workers, 168 at launch: 128 x 128 = 16384 = 256 x (232 - 168)
        //  16 workers,  96 at launch: 128 x 56  =  7168 >= 512 x (104 - 96) = 4096   (112 would need 8192: a hang)
        //   8 workers + 8 split warps, 96 at launch: 128 x 56 + 256 x 56 = 21504 >= 256 x (176 - 96) = 20480
        constexpr int kWorkerRegs = kSW > 0 ? 176 : kWW == 16 ? 104 : 232;
        static_assert(kFirstWorkerWarp * 32 * (kLaunchRegs - 40) + kSW * 32 * (kLaunchRegs - kSplitRegs) >=
                          kWT * (kWorkerRegs - kLaunchRegs),
                      "the workers' register increase exceeds what the other warps release");
        if constexpr (kMoveRegs) reg_alloc<kWorkerRegs>();
        const int wid = warp - kFirstWorkerWarp;
        const int wtid = threadIdx.x - kFirstWorkerWarp * 32;
        const int quarter = warp & 3;  // TMEM lanes this warp may touch: 32*quarter .. +31
        const int half = wid >> 2;     // which part of the tile's columns (kWW / 4 parts)
        float acc[kCols];
        uint32_t it = 0, chain = 0;
        bool ok = true;

        // Convolution gathers: the k side of the addressing, once per CTA (see
        // conv_table_gather_split_store).
        const int* koff = nullptr;
        const uint32_t* kdelta = nullptr;
        if constexpr (kConv == 1 || kConv == 3) {
            if (p.cv_table) {
                int* t_off = reinterpret_cast<int*>(smem + kStages * Cfg::kStageBytes);
                uint32_t* t_del = reinterpret_cast<uint32_t*>(t_off + kConvTableMax);
                const int khw = p.cv_kh * p.cv_kw;
                const int padded = (p.K + 3) & ~3;
                for (int k = wtid; k < padded; k += kWorkerThreads) {
                    const int ch = k / khw, rem = k - ch * khw;
                    const int kh = rem / p.cv_kw, kw = rem - kh * p.cv_kw;
                    if (k >= p.K) {
                        t_off[k] = 0;
                        t_del[k] = 0;  // delta -32768: no row passes the compare
                    } else if constexpr (kConv == 1) {
                        t_off[k] = (ch * p.cv_h + kh) * p.cv_w + kw;
                        t_del[k] = (static_cast<uint32_t>(kConvDeltaBias + kh) << 16) |
                                   static_cast<uint32_t>(kConvDeltaBias + kw);
                    } else {
                        t_off[k] = (ch * p.cv_oh - kh) * p.cv_ow - kw;
                        t_del[k] = (static_cast<uint32_t>(kConvDeltaBias - kh) << 16) |
                                   static_cast<uint32_t>(kConvDeltaBias - kw);
                    }
                }
                asm volatile("bar.sync 2, %0;" ::"n"(kWorkerThreads) : "memory");
                koff = t_off;
                kdelta = t_del;
            }
        }

        // split_bar / acce_bar are waited on by the MMA lane of the leader CTA only.
        auto arrive_at_leader = [&](uint32_t bar) {
            if constexpr (kPair) {
                mbar_arrive_cluster(map_to_cta(bar, 0));
            } else {
                mbar_arrive(bar);
            }
        };

        // Adds the finished TMEM partial of accumulator chain `c` into the fp32 registers.
        auto promote = [&](uint32_t c) -> bool {
            const uint32_t buf = c & 1;
            bool got;
            {
                got = wait_bar(smem_u32(&accf_bar[buf]), (c >> 1) & 1, abort_flag, p.status,
                               kStatWorkerAcc);
                got = __all_sync(0xffffffffu, got);
            }
            if (!got) return false;
            tc_fence_after_sync();
            const uint32_t t0 = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN +
                                half * kCols;
            if constexpr (kCols >= 32 && kWW == 16) {
                // 104 registers per thread: sixteen columns at a time
#pragma unroll
                for (int g = 0; g < kCols / 16; ++g) {
                    uint32_t v[16];
                    tmem_ld_x16(t0 + g * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[g * 16 + j] += __uint_as_float(v[j]);
                }
            } else if constexpr (kCols >= 64 && kSW == 0) {
                // Two 32-column loads in flight per wait: the load's latency is paid once per 64 columns
                // (the registers allow no more beside 128 accumulators).
#pragma unroll
                for (int g = 0; g < kCols / 64; ++g) {
                    uint32_t v0[32], v1[32];
                    tmem_ld_x32(t0 + g * 64, v0);
                    tmem_ld_x32(t0 + g * 64 + 32, v1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[g * 64 + j] += __uint_as_float(v0[j]);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[g * 64 + 32 + j] += __uint_as_float(v1[j]);
                }
            } else if constexpr (kCols >= 32) {
#pragma unroll
                for (int g = 0; g < kCols / 32; ++g) {
                    uint32_t v[32];
                    tmem_ld_x32(t0 + g * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[g * 32 + j] += __uint_as_float(v[j]);
                }
            } else {
                uint32_t v[16];
                tmem_ld_x16(t0, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(v[j]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) arrive_at_leader(smem_u32(&acce_bar[buf]));
            return true;
        };

        // Register-staged loader: one k-block of both operands, as a load phase (global -> registers)
        // and a store phase (split, registers -> shared memory), so that the loads of k-block i + 1
        // are in flight while k-block i is multiplied and drained.
        [[maybe_unused]] float4 va[kBM * 8 / kWorkerThreads];
        [[maybe_unused]] float4 vb[BN * 8 / kWorkerThreads];
        [[maybe_unused]] ConvRow crow{0, 0, 0};
        [[maybe_unused]] auto ldg_phase = [&](auto load_c, auto store_c, const Work& wk, int kb, uint8_t* stage) {
            constexpr bool L = decltype(load_c)::value, S = decltype(store_c)::value;
            const int k0 = kb * BK;
            uint8_t* a_hi = stage;
            uint8_t* a_lo = stage + Cfg::kHalf;
            uint8_t* b_hi = stage + Cfg::kABytes;
            uint8_t* b_lo = stage + Cfg::kHalf + Cfg::kABytes;
            if constexpr (kConv == 1) {
                if (koff != nullptr) {
                    conv_table_gather_split_store<L, S>(p.A, koff, kdelta, crow, p.cv_h, p.cv_w, k0, p.K, a_hi, a_lo,
                                                        prec3, wtid, va);
                } else {
                    conv_gather_split_store<L, S>(p, wk.mt * kBM, k0, a_hi, a_lo, prec3, wtid, va);
                }
            } else if constexpr (kConv == 2) {
                conv_dy_rows_split_store<L, S>(p, wk.mt * kBM, k0, a_hi, a_lo, prec3, wtid, va);
            } else if constexpr (kConv == 3) {
                if (koff != nullptr) {
                    conv_table_gather_split_store<L, S>(p.A, koff, kdelta, crow, p.cv_oh, p.cv_ow, k0, p.K, a_hi,
                                                        a_lo, prec3, wtid, va);
                } else {
                    conv_dx_gather_split_store<L, S>(p, wk.mt * kBM, k0, a_hi, a_lo, prec3, wtid, va);
                }
            } else {
                ldg_split_store<kBM, L, S>(p.A + (long long)wk.b * p.strideA, p.lda, !p.transA, p.a_vec_ok != 0,
                                           wk.mt * kBM, p.M, k0, p.K, a_hi, a_lo, prec3, wtid, va);
            }
            if constexpr (kConv == 2) {
                conv_cols_T_split_store<BN, L, S>(p, wk.nt * BN, k0, b_hi, b_lo, prec3, wtid, vb);
            } else if constexpr (kConv == 3) {
                conv_weight_T_split_store<BN, L, S>(p, wk.nt * BN, k0, b_hi, b_lo, prec3, wtid, vb);
            } else {
                ldg_split_store<BN, L, S>(p.B + (long long)wk.b * p.strideB, p.ldb, p.transB != 0, p.b_vec_ok != 0,
                                          wk.nt * BN, p.N, k0, p.K, b_hi, b_lo, prec3, wtid, vb);
            }
        };

        for (int w = first_work; w < p.total_work && ok; w += work_stride) {
            const Work wk = decode_work(p, w);
            const int nkb = wk.kb1 - wk.kb0;
#pragma unroll
            for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
            if constexpr (kConv == 1 || kConv == 3) {
                if (koff != nullptr) {
                    const int gr = wk.mt * kBM + wtid % kBM;
                    if (gr >= p.M) {
                        crow.y = -2 * kConvDeltaBias - (1 << 20);  // fails every compare
                        crow.x = 0;
                    } else if constexpr (kConv == 1) {
                        const int ohw = p.cv_oh * p.cv_ow;
                        const int img = gr / ohw, pix = gr - img * ohw;
                        const int oh = pix / p.cv_ow, ow = pix - oh * p.cv_ow;
                        const int y = oh * p.cv_stride - p.cv_pad, x = ow * p.cv_stride - p.cv_pad;
                        crow.base = ((long long)img * p.cv_c * p.cv_h + y) * p.cv_w + x;
                        crow.y = y - kConvDeltaBias;
                        crow.x = x - kConvDeltaBias;
                    } else {
                        const int hw = p.cv_h * p.cv_w;
                        const int img = gr / hw, pix = gr - img * hw;
                        const int ih = pix / p.cv_w, iw = pix - ih * p.cv_w;
                        const int y = ih + p.cv_pad, x = iw + p.cv_pad;
                        crow.base = ((long long)img * p.cv_oc * p.cv_oh + y) * p.cv_ow + x;
                        crow.y = y - kConvDeltaBias;
                        crow.x = x - kConvDeltaBias;
                    }
                }
            }

            if constexpr (!kTma) {
                if (nkb > 0) ldg_phase(std::true_type{}, std::false_type{}, wk, wk.kb0, nullptr);
            }
            for (int i = 0; i < nkb && ok; ++i, ++it) {
                const uint32_t s = it % kStages;
                const uint32_t ph = (it / kStages) & 1;
                uint8_t* stage = smem + s * Cfg::kStageBytes;
                if constexpr (kSW > 0) {
                    // the split warps hand the stages over; these warps only drain
                } else if constexpr (kTma) {
                    bool got;
                    {
                        got = wait_bar(smem_u32(&full_bar[s]), ph, abort_flag, p.status,
                                       kStatWorkerFull);
                        got = __all_sync(0xffffffffu, got);
                    }
                    if (!got) {
                        ok = false;
                        break;
                    }
                    float4* hi = reinterpret_cast<float4*>(stage);
                    float4* lo = reinterpret_cast<float4*>(stage + Cfg::kHalf);
                    constexpr int kN4 = Cfg::kHalf / 16;
                    // TF32 mode without rounding: the tensor core reads the fp32 tile as it is
                    // (it drops the low 13 mantissa bits), so the workers only pass the stage on.
                    const int n4 = (prec3 || p.tf32_round) ? kN4 : 0;
                    if (n4 != 0) split_stage<kN4, kWT, 8>(hi, lo, wtid, prec3, prec3 && p.trunc_hi);
                } else {
                    bool got;
                    {
                        got = wait_bar(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status,
                                       kStatWorkerFull);
                        got = __all_sync(0xffffffffu, got);
                    }
                    if (!got) {
                        ok = false;
                        break;
                    }
                    ldg_phase(std::false_type{}, std::true_type{}, wk, wk.kb0 + i, stage);
                }
                if constexpr (kSW == 0) {
                    // generic-proxy writes -> visible to the tensor core's async-proxy reads
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) arrive_at_leader(smem_u32(&split_bar[s]));
                }
                if constexpr (!kTma) {
                    // the next k-block's global loads fly while the accumulator is drained
                    if (i + 1 < nkb) ldg_phase(std::true_type{}, std::false_type{}, wk, wk.kb0 + i + 1, nullptr);
                }

                // Drain the chain that ended one k-block ago (its MMAs have had a whole
                // k-block of time to finish, so this rarely waits).
                if (i >= 1 && ((i % promote_every) == 0)) {
                    if (!promote(chain)) {
                        ok = false;
                        break;
                    }
                    ++chain;
                }
            }
            if (!ok) break;
            if (!promote(chain)) {  // the last chain of the tile
                ok = false;
                break;
            }
            ++chain;

            // ---------------------------------------------------------------- epilogue
            // Last tile of this CTA: what is left is the store, so the next kernel's set-up can run
            // under it (it still waits for this kernel to complete before it touches memory).
            if (w + work_stride >= p.total_work) grid_launch_dependents();
            // A thread holds kCols consecutive columns of ONE row; stored as it stands, every
            // store instruction of a warp would touch 32 different rows with 16 bytes each.
            // Each warp therefore turns 32 x 32 blocks through its own 4 KB of shared memory
            // (16-byte chunks XOR-swizzled by row, conflict-free both ways) and stores rows:
            // one instruction writes four full 128-byte row segments — what HBM and, for the
            // peers' copies of C, NVLink want.
            if constexpr (kConv == 1 || kConv == 3) {
                // The product's row m = (n, pixel) and column ch go to t[n][ch][pixel]: for one
                // column, the 32 rows a warp holds are 32 consecutive floats, so the threads store
                // their own registers directly and the (N, spatial, C) -> (N, C, H, W) permute of
                // Conv2d::forward (src/conv.cpp:335-337) — or, for the input gradient, col2im's
                // scatter — never happens as a separate pass.
                const int row = wk.mt * kBM + quarter * 32 + lane;
                const int col_base = wk.nt * BN + half * kCols;
                if (row < p.M) {
                    const int ohw = p.cv_store_hw;
                    const int img = row / ohw, pix = row - img * ohw;
                    float* ybase = p.dest[0] + (long long)img * p.N * ohw + pix;
#pragma unroll
                    for (int j = 0; j < kCols; ++j) {
                        const int col = col_base + j;
                        if (col < p.N) {
                            float o = p.alpha * acc[j];
                            if (p.bias) o += __ldg(p.bias + col);
                            if (p.beta != 0.f) o += p.beta * ybase[(long long)col * ohw];
                            if (p.relu) o = fmaxf(o, 0.f);
                            ybase[(long long)col * ohw] = o;
                        }
                    }
                }
            } else {
                // staging slot of this warp: 32 rows x kSC floats, rows of kSC4 16-byte chunks
                constexpr int kSC = Cfg::kStageCols;
                constexpr int kSC4 = kSC / 4;
                constexpr int kRowsPerStore = 32 / kSC4;  // rows one store instruction of the warp covers
                constexpr int kStoreIters = 32 / kRowsPerStore;
                float4* tile = reinterpret_cast<float4*>(smem + kStages * Cfg::kStageBytes) + wid * (8 * kSC);
                const int row_base = wk.mt * kTileM + static_cast<int>(cta_rank) * kBM + quarter * 32;
                const int col_base = wk.nt * BN + half * kCols;
                const int sub_row = lane / kSC4;  // row within the group one store instruction covers
                const int chunk = lane % kSC4;    // 16-byte chunk of the row segment
                const bool split_out = p.split_k > 1;
                const float alpha = split_out ? 1.0f : p.alpha;
                const float beta = split_out ? 0.0f : p.beta;
                const bool compact = split_out && p.tail_tiles > 0;
                const long long ld_out = compact ? (long long)BN : split_out ? (long long)p.N : p.ldc;
                const bool vec = compact ? true : split_out ? ((p.N & 3) == 0) : (p.c_vec_ok != 0);
                const bool fuse = !split_out && (p.bias != nullptr || p.addend != nullptr);
                const bool relu = !split_out && p.relu != 0;
                const bool plain = beta == 0.f;
                // compact: element (row, col) of tail tile t lives at
                //   ((sp * tail_tiles + t) * kTileM + row - tile_row0) * BN + col - tile_col0
                const long long base_off =
                    compact ? (((long long)wk.sp * p.tail_tiles + (wk.tile - p.tile_offset)) * kTileM -
                               (long long)wk.mt * kTileM) * BN - (long long)wk.nt * BN
                    : split_out ? ((long long)wk.sp * p.batch + wk.b) * (long long)p.M * p.N
                                : (long long)wk.b * p.strideC;
#pragma unroll
                for (int g = 0; g < kCols / kSC + (kCols < kSC ? 1 : 0); ++g) {
                    constexpr int kChunkCols = kCols < kSC ? kCols : kSC;
                    constexpr int kChunks = kChunkCols / 4;
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < kChunks; ++j) {
                        tile[lane * kSC4 + (j ^ (lane & (kSC4 - 1)))] =
                            make_float4(acc[g * kSC + 4 * j], acc[g * kSC + 4 * j + 1],
                                        acc[g * kSC + 4 * j + 2], acc[g * kSC + 4 * j + 3]);
                    }
                    __syncwarp();
                    const int col = col_base + g * kSC + chunk * 4;
                    if (chunk < kChunks && col < p.N && plain) {
                        // The common store — one destination (C or the split-K partials), no beta —
                        // apart from the general one below: a small product is one tile per
                        // CTA and fetches every instruction it executes cold, so the path it walks
                        // is short.
                        float* dst0 = (split_out ? p.partial : p.dest[0]) + base_off + col;
                        const bool whole = vec && col + 3 < p.N;  // an aligned 16-byte chunk
                        float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);  // the same for every row
                        if (fuse && p.bias != nullptr) {
                            bias4.x = __ldg(p.bias + col);
                            if (col + 1 < p.N) bias4.y = __ldg(p.bias + col + 1);
                            if (col + 2 < p.N) bias4.z = __ldg(p.bias + col + 2);
                            if (col + 3 < p.N) bias4.w = __ldg(p.bias + col + 3);
                        }
#pragma unroll 1
                        for (int it = 0; it < kStoreIters; ++it) {
                            const int rr = it * kRowsPerStore + sub_row;
                            const int row = row_base + rr;
                            if (row >= p.M) continue;
                            float4 v = tile[rr * kSC4 + (chunk ^ (rr & (kSC4 - 1)))];
                            v.x *= alpha;
                            v.y *= alpha;
                            v.z *= alpha;
                            v.w *= alpha;
                            if (fuse) {  // bias, then mask, then ReLU: the order of the separate ops
                                if (p.bias != nullptr) {
                                    v.x += bias4.x;
                                    v.y += bias4.y;
                                    v.z += bias4.z;
                                    v.w += bias4.w;
                                }
                                if (p.addend != nullptr) {
                                    const float* ad = p.addend + (long long)row * p.ld_addend + col;
                                    v.x += __ldg(ad);
                                    if (col + 1 < p.N) v.y += __ldg(ad + 1);
                                    if (col + 2 < p.N) v.z += __ldg(ad + 2);
                                    if (col + 3 < p.N) v.w += __ldg(ad + 3);
                                }
                            }
                            if (relu) {
                                v.x = fmaxf(v.x, 0.f);
                                v.y = fmaxf(v.y, 0.f);
                                v.z = fmaxf(v.z, 0.f);
                                v.w = fmaxf(v.w, 0.f);
                            }
                            float* dst = dst0 + (long long)row * ld_out;
                            if (whole) {
                                *reinterpret_cast<float4*>(dst) = v;
                            } else {
                                dst[0] = v.x;
                                if (col + 1 < p.N) dst[1] = v.y;
                                if (col + 2 < p.N) dst[2] = v.z;
                                if (col + 3 < p.N) dst[3] = v.w;
                            }
                        }
                    } else if (chunk < kChunks && col < p.N) {
                        // Not unrolled on purpose: 32 copies of the store path (4 column groups x
                        // 8 row groups) made the kernel 20 % slower at 4096^3 — the k-loop's
                        // code no longer stayed in the instruction cache.
#pragma unroll 1
                        for (int it = 0; it < kStoreIters; ++it) {
                            const int rr = it * kRowsPerStore + sub_row;
                            const int row = row_base + rr;
                            if (row >= p.M) continue;
                            float4 v = tile[rr * kSC4 + (chunk ^ (rr & (kSC4 - 1)))];
                            v.x *= alpha;
                            v.y *= alpha;
                            v.z *= alpha;
                            v.w *= alpha;
                            if (fuse) {  // bias / mask do not depend on the destination
                                if (col + 0 < p.N) v.x = add_bias_mask(p, v.x, row, col + 0);
                                if (col + 1 < p.N) v.y = add_bias_mask(p, v.y, row, col + 1);
                                if (col + 2 < p.N) v.z = add_bias_mask(p, v.z, row, col + 2);
                                if (col + 3 < p.N) v.w = add_bias_mask(p, v.w, row, col + 3);
                            }
                            const long long off = base_off + (long long)row * ld_out + col;
                            {
                                float* dst = (split_out ? p.partial : p.dest[0]) + off;
                                if (vec && col + 3 < p.N) {
                                    float4 o = v;
                                    if (beta != 0.f) {
                                        const float4 old = *reinterpret_cast<const float4*>(dst);
                                        o.x += beta * old.x;
                                        o.y += beta * old.y;
                                        o.z += beta * old.z;
                                        o.w += beta * old.w;
                                    }
                                    if (relu) {
                                        o.x = fmaxf(o.x, 0.f);
                                        o.y = fmaxf(o.y, 0.f);
                                        o.z = fmaxf(o.z, 0.f);
                                        o.w = fmaxf(o.w, 0.f);
                                    }
                                    *reinterpret_cast<float4*>(dst) = o;
                                } else {
                                    const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        if (col + e < p.N) {
                                            float o = e4[e];
                                            if (beta != 0.f) o += beta * dst[e];
                                            if (relu) o = fmaxf(o, 0.f);
                                            dst[e] = o;
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
            }
            if constexpr (kConv == 0) {
                // this warp's part of the tile is in C: the forwarders may copy it to the peers
                if (p.n_dest > 1) {
                    __threadfence();  // the tile's stores have reached L2, where the forwarders read them
                    __syncwarp();
                    if (lane == 0) smem_add_release(smem_u32(&fwd_count_s), 1u);
                }
            }
        }
        // The next kernel of the stream may start its set-up under this one's exit.
        grid_launch_dependents();
    }

    tc_fence_before_sync();
    if constexpr (kPair) {
        // Neither CTA may release TMEM or exit while the other can still be the target of a
        // pair product, a completion signal or a remote arrive.
        __syncwarp();
        cluster_sync();
        if (warp == 1) {
            __syncwarp();
            tmem_dealloc_pair(tmem, Cfg::kTmemCols);
        }
    } else {
        __syncthreads();
        if (warp == 1) {
            __syncwarp();
            tmem_dealloc(tmem, Cfg::kTmemCols);
        }
    }
}

// Adds the split-K partials (split x batch x M x N, one matrix after the other) into C and applies
// the epilogue.  `lanes` (a power of two up to 32) threads share one element: lane j adds parts
// j, j + lanes, ... in ascending order, then a fixed shuffle tree adds the lanes — the same order
// on every run.  Few elements with many parts (a weight gradient contracted over a whole batch)
// would otherwise leave one thread walking hundreds of parts a whole matrix apart.
__global__ void splitk_reduce_kernel(const GemmParams p, const float* __restrict__ partial,
                                     float* __restrict__ C, int split, long long batch, long long M,
                                     long long N, long long ldc, long long strideC, float alpha,
                                     float beta, int lanes) {
    grid_dependency_wait();  // the partials come from the kernel before this one
    const long long total = batch * M * N;
    const int lane = threadIdx.x & 31;
    const int sub = lane & (lanes - 1);
    const int per_warp = 32 / lanes;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long i0 = warp * per_warp; i0 < total; i0 += warps * per_warp) {
        const long long i = i0 + lane / lanes;
        float s = 0.f;
        if (i < total)
            for (int k = sub; k < split; k += lanes) s += partial[(long long)k * total + i];
        for (int off = lanes >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (i < total && sub == 0) {
            const long long b = i / (M * N);
            const long long r = (i - b * M * N) / N;
            const long long c = i - b * M * N - r * N;
            float* out = C + b * strideC + r * ldc + c;
            *out = finish_output(p, alpha * s, beta != 0.f ? *out : 0.f, static_cast<int>(r),
                                 static_cast<int>(c));
        }
    }
}

// Adds the compact split-K partials of the tail-wave tiles into C (ascending split order):
// block x handles tile x / 8, rows [x % 8 * tile_rows / 8, ...).
__global__ void tail_reduce_kernel(const GemmParams p, int tile_rows, int bn) {
    grid_dependency_wait();  // the partials come from the kernel before this one
    const int tl = blockIdx.x >> 3;
    const int slab = blockIdx.x & 7;
    GemmParams q = p;
    q.split_k = 1;
    q.fd_split = 0;  // the multiplier of a division by one
    const Work wk = decode_work(q, tl);  // tile_offset is applied inside
    const int rows_per = tile_rows / 8;
    const int chunks = bn / 4;
    const long long tile_elems = (long long)tile_rows * bn;
    for (int i = threadIdx.x; i < rows_per * chunks; i += blockDim.x) {
        const int r = slab * rows_per + i / chunks;
        const int c4 = (i % chunks) * 4;
        const int row = wk.mt * tile_rows + r;
        const int col = wk.nt * bn + c4;
        if (row >= p.M || col >= p.N) continue;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < p.split_k; ++sp) {
            const float4 v = *reinterpret_cast<const float4*>(
                p.partial + ((long long)sp * p.tail_tiles + tl) * tile_elems + (long long)r * bn + c4);
            s.x += v.x;
            s.y += v.y;
            s.z += v.z;
            s.w += v.w;
        }
        float* out = p.dest[0] + (long long)wk.b * p.strideC + (long long)row * p.ldc + col;
        const float e4[4] = {s.x, s.y, s.z, s.w};
        for (int e = 0; e < 4; ++e) {
            if (col + e < p.N) {
                out[e] = finish_output(p, p.alpha * e4[e], p.beta != 0.f ? out[e] : 0.f, row, col + e);
            }
        }
    }
}

// K == 0: the product is empty, C = beta * C.
// Sums the weight gradient's split partials (rows x ld_part each, ascending split order within a
// lane, then a fixed shuffle tree): columns [0, kcols) go to dweight, column kcols — the product with
// the ones column — to dbias.  One warp per element: the partials of one element are `split`
// floats a whole matrix apart.
__global__ void conv_dw_reduce_kernel(const float* __restrict__ partial, int split, int rows, int kcols,
                                      int ld_part, float* __restrict__ dweight, float* __restrict__ dbias,
                                      float beta) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    const long long total = (long long)rows * ld_part;
    for (long long i = warp; i < total; i += warps) {
        float s = 0.f;
        for (int k = lane; k < split; k += 32) s += partial[(long long)k * total + i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) {
            const int r = static_cast<int>(i / ld_part), c = static_cast<int>(i - (long long)r * ld_part);
            float* out = c < kcols ? dweight + (long long)r * kcols + c : dbias + r;
            *out = s + (beta != 0.f ? beta * *out : 0.f);
        }
    }
}

// Test aid for the bounded waits: one warp waits, with the given budget, on a barrier that nobody
// ever arrives at.  The wait runs out, records kStatSelfTest in *status and raises the abort flag —
// the same path a lost TMA copy or tensor-core completion would take in the product kernels — and
// the kernel returns normally.  Nothing here touches TMA or tensor memory.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long budget_ns, int* observed) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_s;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_s = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const bool got = wait_bar(smem_u32(&bar), 0, &abort_s, status, kStatSelfTest, budget_ns);
    __syncthreads();
    // observed[0]: threads whose wait returned "completed" (must be 0); observed[1]: the abort flag
    if (got) atomicAdd(observed, 1);
    if (threadIdx.x == 0) observed[1] = abort_s;
}

__global__ void scale_c_kernel(float* __restrict__ C, long long batch, long long M, long long N,
                               long long ldc, long long strideC, float beta) {
    const long long total = batch * M * N;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const long long b = i / (M * N);
        const long long r = (i - b * M * N) / N;
        const long long c = i - b * M * N - r * N;
        float* out = C + b * strideC + r * ldc + c;
        *out = (beta == 0.f) ? 0.f : beta * *out;
    }
}

}  // namespace b200
