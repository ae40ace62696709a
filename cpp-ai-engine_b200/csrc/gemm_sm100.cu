// Host side of the B200 GEMM library: argument checks, tile / loader / split-K selection,
// TMA tensor-map encoding, launches, and the extern "C" surface declared in
// include/b200_gemm.h.  No CPU fallback exists: a shape the kernels cannot run is an error.
#include "../../include/b200_gemm.h"
#include "attention_kernel.cuh"
#include "attention_bwd_kernel.cuh"
#include "gemm_kernel.cuh"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <utility>

namespace b200 {
namespace {

constexpr int kMaxDevices = 64;

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    int cc_major = 0;
    int* status = nullptr;  // device status word of the bounded waits
    // staging for the *_host entry point (grow-only)
    float* stage_a = nullptr;
    float* stage_b = nullptr;
    float* stage_c = nullptr;
    void* stage_ws = nullptr;
    size_t cap_a = 0, cap_b = 0, cap_c = 0, cap_ws = 0;
    // streams and events of the pipelined host path (created on first use)
    cudaStream_t s_h2d = nullptr, s_comp = nullptr, s_comp2 = nullptr, s_d2h = nullptr, s_d2h2 = nullptr;
    cudaEvent_t ev_a[16] = {}, ev_b[16] = {}, ev_c[256] = {};
    bool pipe_ready = false;
};

std::mutex g_mutex;
std::mutex g_host_mutex[kMaxDevices];  // one b200_matmul_f32_host call per device at a time
DeviceState g_dev[kMaxDevices];
std::atomic<uint64_t> g_launches{0};

struct Options {
    long tile_n = 0;
    long split_k = 0;
    long promote_every = 0;  // 0 = automatic: every k-block (3xTF32), every 8th (TF32)
    long force_ldg = 0;
    long pair_mode = 0;  // 0 automatic, 1 never, 2 whenever legal
    long host_pipeline = 1;  // b200_matmul_f32_host: overlap transfers with the math
    long tail_split = 1;     // split the tiles of a mostly-empty last wave along K
    long group_m = 0;        // tile rows per scheduling band; 0 = automatic
    long tf32_round = 1;     // TF32 mode: round operands to nearest (1) or let the tensor core truncate (0)
    long head_mode = 0;      // 3xTF32 head: 0 = rounded to nearest by the workers, 1 = the tensor core's truncation
    long pdl = 1;            // launch with programmatic stream serialization (set-up overlaps the previous kernel)
    long map_cache = 1;      // reuse encoded TMA tensor maps between calls
    long block_k = 0;        // values of k per pipeline stage: 0 = automatic, 32, or 64 (TMA loader, tiles up to 64 wide)
    long split_warps = 0;    // pair kernel: 8 = eight more warps that only split, the workers only drain
    long pair_workers = 8;   // worker warps per CTA of the pair kernel: 8, or 16 (measured 3-5 % slower)
};
// Process-wide knobs, read without synchronisation on every call: set them while no other thread
// is inside the library (they exist for benchmarking).
Options g_opt;

// k-blocks accumulated in TMEM before the partial sum is promoted to fp32 registers.  The
// fp32-accurate mode promotes every k-block (the tensor core truncates its accumulator, which would
// otherwise cost ~3e-5 at K = 2048); in TF32 mode the operands' own rounding (~1e-3 per product)
// dwarfs that, and longer chains are 20 % faster.
int promote_interval(int precision) {
    if (g_opt.promote_every >= 1) return static_cast<int>(g_opt.promote_every);
    return precision == B200_PRECISION_TF32 ? 8 : 1;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// Resolves the driver's tensor-map encoder at run time so the library itself does not link
// against libcuda and still loads on a machine without a driver.
int resolve_encoder() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return B200_EDEVICE;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return 0;
}

int device_state(DeviceState** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return B200_EDEVICE;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        int major = 0, sms = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
            return static_cast<int>(e);
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
            return static_cast<int>(e);
        if (major != 10) return B200_EDEVICE;  // tcgen05 / TMEM exist on sm_100 only
        if ((e = cudaMalloc(&st.status, sizeof(int))) != cudaSuccess) return static_cast<int>(e);
        if ((e = cudaMemset(st.status, 0, sizeof(int))) != cudaSuccess) return static_cast<int>(e);
        st.cc_major = major;
        st.sm_count = sms;
        st.ready = true;
    }
    *out = &st;
    return 0;
}

struct OperandMap {
    CUtensorMap map;
    uint32_t lbo, sbo, kstep, ksub, layout;
};

// Describes one operand tile to TMA (how to fetch it) and to the tensor core (how it lies in
// shared memory afterwards).
//   k_contig: k is the contiguous index of the stored matrix -> K-major tile: one box of
//             `rows` x BK, rows of BK*4 bytes, swizzle = row width (128 B or 64 B).
//   else      the m / n index is contiguous -> MN-major tile: boxes of 32 (m|n) x BK (k),
//             128-byte rows with 32-byte swizzle atoms, the only MN-major layout the tensor
//             core accepts for 32-bit operands.
int make_operand_map(OperandMap* om, const float* base, bool k_contig, int64_t rows_total,
                     int64_t K, int64_t ld, int64_t batch_stride, int64_t batch, int tile_rows,
                     int bk) {
    cuuint64_t dims[3];
    cuuint64_t strides[2];
    cuuint32_t box[3];
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    CUtensorMapSwizzle swz;
    const int64_t nbatch = batch_stride ? batch : 1;
    if (k_contig) {
        dims[0] = static_cast<cuuint64_t>(K);
        dims[1] = static_cast<cuuint64_t>(rows_total);
        // a row of the box is one swizzle row: at most 32 floats (128 bytes); a wider k-block is
        // fetched as several boxes side by side
        const int box_k = bk >= 32 ? 32 : bk;
        box[0] = box_k;
        box[1] = tile_rows;
        swz = (box_k == 32) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
        om->layout = (box_k == 32) ? kLayoutSw128 : kLayoutSw64;
        om->lbo = 16;
        om->sbo = 8u * box_k * 4u;    // eight rows
        om->kstep = 32;               // 8 floats along the row
        om->ksub = tile_rows * 128u;  // the next 32 values of k: the next sub-tile
    } else {
        dims[0] = static_cast<cuuint64_t>(rows_total);
        dims[1] = static_cast<cuuint64_t>(K);
        box[0] = 32;
        box[1] = bk;
        swz = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
        om->layout = 1;           // 128-byte swizzle with 32-byte atoms
        om->lbo = bk * 128u;      // next 32 m|n: next box
        om->sbo = 512;            // next 4 k: four 128-byte rows
        om->kstep = 1024;         // 8 k
        om->ksub = 4096;          // 32 k: the rows of a box simply continue
    }
    dims[2] = static_cast<cuuint64_t>(nbatch);
    box[2] = 1;
    strides[0] = static_cast<cuuint64_t>(ld) * 4u;
    const int64_t outer_rows = k_contig ? rows_total : K;
    const int64_t bs = batch_stride ? batch_stride : ld * outer_rows;
    strides[1] = static_cast<cuuint64_t>(bs) * 4u;
    if (strides[1] == 0) strides[1] = 16;
    CUresult r = g_encode(&om->map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                          const_cast<float*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : B200_EINVAL;
}

// A steady-state caller (a training step, a decode loop) issues the same products on the same
// buffers again and again, and cuTensorMapEncodeTiled costs about a microsecond per operand — a
// large part of what the host spends on an engine-sized product.  The encoded map depends only on
// the arguments below (never on the buffer's contents), so each thread keeps the last maps it
// encoded in a small direct-mapped table.
struct MapKey {
    const void* base;
    int64_t rows_total, K, ld, batch_stride, batch;
    int32_t k_contig, tile_rows, bk, dev;
};
struct MapSlot {
    MapKey key;
    OperandMap om;
    bool valid;
};
constexpr int kMapSlots = 128;

int cached_operand_map(OperandMap* om, const float* base, bool k_contig, int64_t rows_total, int64_t K,
                       int64_t ld, int64_t batch_stride, int64_t batch, int tile_rows, int bk) {
    if (!g_opt.map_cache)
        return make_operand_map(om, base, k_contig, rows_total, K, ld, batch_stride, batch, tile_rows, bk);
    thread_local MapSlot slots[kMapSlots] = {};
    MapKey key;
    std::memset(&key, 0, sizeof(key));  // padding bytes take part in the comparison
    int dev = 0;
    cudaGetDevice(&dev);
    key.base = base;
    key.rows_total = rows_total;
    key.K = K;
    key.ld = ld;
    key.batch_stride = batch_stride;
    key.batch = batch_stride ? batch : 1;
    key.k_contig = k_contig ? 1 : 0;
    key.tile_rows = tile_rows;
    key.bk = bk;
    key.dev = dev;
    uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
    h ^= (static_cast<uint64_t>(rows_total) * 0xC2B2AE3D27D4EB4Full) ^ (static_cast<uint64_t>(K) << 21) ^
         (static_cast<uint64_t>(ld) << 7) ^ static_cast<uint64_t>(tile_rows * 2 + key.k_contig);
    MapSlot& slot = slots[(h >> 32) % kMapSlots];
    if (slot.valid && std::memcmp(&slot.key, &key, sizeof(key)) == 0) {
        *om = slot.om;
        return 0;
    }
    int rc = make_operand_map(om, base, k_contig, rows_total, K, ld, batch_stride, batch, tile_rows, bk);
    if (rc) return rc;
    slot.key = key;
    slot.om = *om;
    slot.valid = true;
    return 0;
}

bool tma_legal(const float* base, int64_t ld, int64_t batch_stride, int64_t batch) {
    if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
    if (ld & 3) return false;
    if (batch > 1 && batch_stride != 0 && (batch_stride & 3)) return false;
    if (ld * 4 >= (1ll << 40) || batch_stride * 4 >= (1ll << 40)) return false;
    return true;
}

// One launch through cudaLaunchKernelEx: optional cluster of two CTAs, and (option "pdl") the
// programmatic-stream-serialization attribute, with which the kernel may become resident and run
// its set-up (barriers, tensor-memory allocation, descriptor prefetch) while the previous kernel of
// the stream drains; it executes griddepcontrol.wait before it touches global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                          int cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(static_cast<unsigned>(block), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = static_cast<unsigned>(cluster);
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (g_opt.pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return e;
}

// Opt-in to more than 48 KB of dynamic shared memory, once per kernel and device.
template <typename Kernel>
int ensure_smem_attr(Kernel kernel, std::atomic<bool>* done, uint32_t bytes) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return B200_EDEVICE;
    if (done[dev].load(std::memory_order_acquire)) return 0;
    std::lock_guard<std::mutex> lock(g_mutex);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(bytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    done[dev].store(true, std::memory_order_release);
    return 0;
}

template <int BN, int BK, bool kTma>
int launch_cfg(const GemmParams& params, const CUtensorMap& ma, const CUtensorMap& mb, int grid,
               cudaStream_t stream) {
    using Cfg = TileCfg<BN, BK>;
    GemmParams p = params;
    fill_schedule(p);
    static std::atomic<bool> attr_set[kMaxDevices] = {};
    if (int rc = ensure_smem_attr(gemm_tf32_kernel<BN, BK, kTma>, attr_set, Cfg::kSmemBytes)) return rc;
    return static_cast<int>(launch_kernel(gemm_tf32_kernel<BN, BK, kTma>, grid, kThreads, Cfg::kSmemBytes,
                                          stream, 1, p, ma, mb));
}

// CTA-pair kernel (tile 256 x 256): launched as clusters of two CTAs.  Two variants: eight worker
// warps per CTA (default) or sixteen (option "pair_workers"; twice the warps per scheduler, half the
// accumulators each — bit-identical results, measured 3-5 % slower at 4096^3 ... 16384^3: the
// workers' instruction latency is not what binds the kernel).
template <int WW, int SW = 0>
int max_pair_clusters_for(int dev) {
    static std::atomic<int> cached[kMaxDevices] = {};
    if (cached[dev].load(std::memory_order_acquire) > 0) return cached[dev].load(std::memory_order_relaxed);
    std::lock_guard<std::mutex> lock(g_mutex);
    using Cfg = TileCfg<256, 32, true, WW>;
    auto kernel = gemm_tf32_kernel<256, 32, true, true, 0, WW, SW>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(Cfg::kSmemBytes)) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(Cfg::kThreadsCfg + SW * 32, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cached[dev].store(n, std::memory_order_release);
    return n;
}
int max_pair_clusters(int dev) {
    if (g_opt.split_warps == 8) return max_pair_clusters_for<8, 8>(dev);
    return g_opt.pair_workers == 16 ? max_pair_clusters_for<16>(dev) : max_pair_clusters_for<8>(dev);
}

template <int WW, int SW = 0>
int launch_pair_for(const GemmParams& params, const CUtensorMap& ma, const CUtensorMap& mb, int clusters,
                    cudaStream_t stream) {
    using Cfg = TileCfg<256, 32, true, WW>;
    GemmParams p = params;
    fill_schedule(p);
    return static_cast<int>(launch_kernel(gemm_tf32_kernel<256, 32, true, true, 0, WW, SW>, 2 * clusters,
                                          Cfg::kThreadsCfg + SW * 32, Cfg::kSmemBytes, stream, 2, p, ma, mb));
}
int launch_pair(const GemmParams& params, const CUtensorMap& ma, const CUtensorMap& mb, int clusters,
                cudaStream_t stream) {
    if (g_opt.split_warps == 8) return launch_pair_for<8, 8>(params, ma, mb, clusters, stream);
    return g_opt.pair_workers == 16 ? launch_pair_for<16>(params, ma, mb, clusters, stream)
                                    : launch_pair_for<8>(params, ma, mb, clusters, stream);
}

// Convolution kernels: register-staged loader with the implicit im2col gather (MODE 1 forward,
// 2 weight gradient, 3 input gradient).
template <int BN, int MODE = 1>
int launch_conv_cfg(const GemmParams& params, int grid, cudaStream_t stream) {
    using Cfg = TileCfg<BN, 32>;
    GemmParams p = params;
    fill_schedule(p);
    static std::atomic<bool> attr_set[kMaxDevices] = {};
    auto kernel = gemm_tf32_kernel<BN, 32, false, false, MODE>;
    if (int rc = ensure_smem_attr(kernel, attr_set, Cfg::kSmemBytes)) return rc;
    CUtensorMap unused{};
    return static_cast<int>(launch_kernel(kernel, grid, kThreads, Cfg::kSmemBytes, stream, 1, p, unused, unused));
}

int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

template <int MODE>
int launch_conv(int bn, const GemmParams& p, int grid, cudaStream_t stream) {
    switch (bn) {
        case 32: return launch_conv_cfg<32, MODE>(p, grid, stream);
        case 64: return launch_conv_cfg<64, MODE>(p, grid, stream);
        case 128: return launch_conv_cfg<128, MODE>(p, grid, stream);
        default: return launch_conv_cfg<256, MODE>(p, grid, stream);
    }
}

// Narrowest tile that covers `cols` output columns while filling the SMs, as for any narrow product.
int conv_tile_n(const DeviceState& st, int64_t rows, int64_t cols) {
    int bn = 32;
    for (int cand : {256, 128, 64, 32}) {
        if (cand > 32 && cols <= cand / 2) continue;
        const int64_t tiles = ceil_div(rows, kBM) * static_cast<int64_t>(ceil_div(cols, cand));
        bn = cand;
        if (tiles >= st.sm_count) break;
    }
    return bn;
}

// The weight gradient contracts over the n * oh * ow output positions into a small
// (out_c x c*kh*kw) result: its k-blocks are shared out over the SMs (deterministic split-K).
struct ConvDwPlan {
    int bn, tiles_m, tiles_n, kblocks, split_k, kb_per_split;
    size_t bytes;  // split-K partials
};
ConvDwPlan conv_dw_plan(const DeviceState& st, int64_t positions, int64_t out_c, int64_t kcols) {
    ConvDwPlan pl{};
    pl.bn = conv_tile_n(st, out_c, kcols);
    pl.tiles_m = ceil_div(out_c, kBM);
    pl.tiles_n = ceil_div(kcols, pl.bn);
    pl.kblocks = ceil_div(positions, 32);
    const int tiles = pl.tiles_m * pl.tiles_n;
    int split = st.sm_count / (tiles > 0 ? tiles : 1);
    if (split > pl.kblocks / 2) split = pl.kblocks / 2;  // at least two k-blocks per part
    if (split < 1) split = 1;
    pl.kb_per_split = ceil_div(pl.kblocks, split);
    pl.split_k = ceil_div(pl.kblocks, pl.kb_per_split);
    pl.bytes = pl.split_k > 1 ? static_cast<size_t>(pl.split_k) * out_c * kcols * sizeof(float) : 0;
    return pl;
}

// dbias[o] = sum over (n, oh, ow) of dy[n][o][oh][ow] (+ beta * dbias[o]): one block per channel,
// fixed summation order.
__global__ void conv_bias_grad_kernel(const float* __restrict__ dy, float* __restrict__ dbias, int n, int out_c,
                                      int ohw, float beta) {
    __shared__ float part[256];
    const int o = blockIdx.x;
    float s = 0.f;
    const long long total = (long long)n * ohw;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) {
        const long long img = i / ohw, sp = i - img * ohw;
        s += __ldg(dy + (img * out_c + o) * ohw + sp);
    }
    part[threadIdx.x] = s;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if ((int)threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) dbias[o] = part[0] + (beta != 0.f ? beta * dbias[o] : 0.f);
}

int dispatch(int bn, int bk, bool tma, const GemmParams& p, const CUtensorMap& ma,
             const CUtensorMap& mb, int grid, cudaStream_t stream) {
#define B200_CASE(BN_)                                                                     \
    case BN_:                                                                              \
        if (!tma) return launch_cfg<BN_, 32, false>(p, ma, mb, grid, stream);              \
        return launch_cfg<BN_, 32, true>(p, ma, mb, grid, stream);
    if (bk == 64) {
        if (!tma) return B200_EINVAL;
        if (bn == 32) return launch_cfg<32, 64, true>(p, ma, mb, grid, stream);
        if (bn == 64) return launch_cfg<64, 64, true>(p, ma, mb, grid, stream);
        return B200_EINVAL;
    }
    switch (bn) {
        B200_CASE(32)
        B200_CASE(64)
        B200_CASE(128)
        B200_CASE(256)
        default:
            return B200_EINVAL;
    }
#undef B200_CASE
}


constexpr bool kAutoBlockK64 = false;  // automatic choice of 64-wide k-blocks (see make_plan)

struct Plan {
    int bn, bk, split_k, kb_per_split, kblocks, tiles_m, tiles_n;
    bool tma;
    bool pair;  // CTA-pair kernel: 256-row tiles
    // Tail wave: when the tile count leaves the last wave mostly empty, the tiles of that wave
    // are split along K (tail_split ways) in a second launch so that all SMs stay busy.
    int full_tiles, tail_tiles, tail_split, tail_kb_per_split;
    size_t tail_bytes;
};

Plan make_plan(const DeviceState& st, int64_t batch, int64_t M, int64_t N, int64_t K, bool tma_ok,
               size_t workspace_bytes) {
    Plan pl{};
    pl.tma = tma_ok && !g_opt.force_ldg;
    pl.bk = 32;
    pl.tiles_m = ceil_div(M, kBM);
    const int sms = st.sm_count > 0 ? st.sm_count : 148;
    int bn = 32;
    bool pair = false;
    int auto_parts = 0;  // K-split chosen together with the tile (0: tile forced by option)
    const int64_t kblocks = ceil_div(K, 32);
    const size_t out_bytes = static_cast<size_t>(batch) * M * N * sizeof(float);  // one partial matrix
    const bool pair_legal = pl.tma && pl.bk == 32 && M > kBM && g_opt.pair_mode != 1;
    if (g_opt.tile_n == 32 || g_opt.tile_n == 64 || g_opt.tile_n == 128 || g_opt.tile_n == 256) {
        bn = static_cast<int>(g_opt.tile_n);
        pair = pair_legal && bn == 256 && g_opt.pair_mode == 2;
    } else {
        // Time model, fitted to CUDA-graph replays of 256^3 ... 4096^3 and the engine's shapes on a
        // B200 (microseconds):
        //     T = launch + waves x (item(tile) + k-blocks per item x t(tile))  [+ reduction if K is split]
        // t is what one k-block of 32 costs a CTA (or CTA pair) — latency-bound near 1 us for the
        // narrow tiles, the tensor pipe for the wide ones — `item` the pipeline fill and the store
        // of one tile, and a K-split adds its second kernel: 1.7 us + 0.47 us per MB of partials
        // read and written.  For products of many waves this is the throughput ranking
        // (pair > 256 > 128 > 64 > 32 per column); for engine-sized ones it weighs a shorter
        // k-loop on more SMs against the reduction it costs.  Narrow products get narrow tiles
        // instead of padding (N = 8, 10, 16, 24 run 32 wide).
        const int cand[5] = {256, 256, 128, 64, 32};
        const bool cand_pair[5] = {true, false, false, false, false};
        const double t_kb[5] = {1.37, 1.63, 1.17, 1.06, 1.06};
        const double item_us[5] = {7.5, 6.7, 4.2, 2.5, 2.0};
        constexpr double kLaunchUs = 3.5;
        double best = -1.0;
        for (int i = 0; i < 5; ++i) {
            const int c = cand[i];
            if (cand_pair[i] && !pair_legal) continue;
            if (!cand_pair[i] && g_opt.pair_mode == 2 && pair_legal && N > 128) continue;
            if (c > 32 && N <= c / 2) continue;  // more than half the tile would be padding
            const int rows = cand_pair[i] ? 2 * kBM : kBM;
            const int units = cand_pair[i] ? (sms / 2 > 0 ? sms / 2 : 1) : sms;
            const int64_t tm = ceil_div(M, rows), tn = ceil_div(N, c);
            const int64_t tiles = batch * tm * tn;
            auto time_of = [&](int64_t parts) {
                const int64_t items = tiles * parts;
                const int64_t waves = (items + units - 1) / units;
                const int64_t kb_item = (kblocks + parts - 1) / parts;
                double t = kLaunchUs + static_cast<double>(waves) *
                                           (item_us[i] + static_cast<double>(kb_item) * t_kb[i]);
                if (parts > 1)
                    t += 1.7 + 0.47e-6 * static_cast<double>(parts + 1) * static_cast<double>(batch) *
                                   static_cast<double>(M) * static_cast<double>(N) * 4.0;
                return t;
            };
            int64_t parts = 1;
            double t = time_of(1);
            // deterministic split-K: few tiles, a k-loop worth cutting, room for the partials
            if (!cand_pair[i] && g_opt.split_k == 0 && tiles * 2 <= units && kblocks >= 8) {
                int64_t p2 = std::min<int64_t>(units / tiles, kblocks / 4);
                // a workspace too small for that many partial matrices still allows a shallower split
                p2 = std::min<int64_t>(p2, static_cast<int64_t>(std::min<size_t>(workspace_bytes / out_bytes, 1u << 20)));
                if (p2 < 1) p2 = 1;
                const int64_t per = (kblocks + p2 - 1) / p2;
                p2 = (kblocks + per - 1) / per;
                if (p2 > 1 && static_cast<size_t>(p2) * out_bytes <= workspace_bytes && time_of(p2) < t) {
                    parts = p2;
                    t = time_of(p2);
                }
            }
            if (best < 0.0 || t < best) {
                best = t;
                bn = c;
                pair = cand_pair[i];
                auto_parts = static_cast<int>(parts);
            }
        }
    }
    pl.bn = bn;
    // Large products run on CTA pairs (256 x 256 tiles, two SMs per tile).
    pl.pair = pair;
    if (pl.pair) pl.tiles_m = ceil_div(M, 2 * kBM);
    pl.tiles_n = ceil_div(N, bn);
    // Narrow tiles are latency-bound: their k-loop is a chain of barrier hand-overs per k-block, so
    // 64 values of k per stage (two swizzle rows side by side) halve the hand-overs.  TMA loader only.
    const bool bk64_legal = pl.tma && !pl.pair && bn <= 64;
    if (bk64_legal && (g_opt.block_k == 64 || (g_opt.block_k == 0 && kAutoBlockK64 && K >= 256))) pl.bk = 64;
    pl.kblocks = ceil_div(K, pl.bk);
    // Deterministic split-K for tall-skinny products (few output tiles, long K).
    pl.split_k = 1;
    pl.kb_per_split = pl.kblocks;
    const int64_t tiles = batch * pl.tiles_m * static_cast<int64_t>(pl.tiles_n);
    int want = 1;
    if (g_opt.split_k > 1 && !pl.pair) {
        want = static_cast<int>(g_opt.split_k);
    } else if (g_opt.split_k == 0 && auto_parts > 0) {
        want = auto_parts;
    } else if (g_opt.split_k == 0 && !pl.pair && tiles * 2 <= sms && pl.kblocks >= 8) {
        want = static_cast<int>(sms / tiles);
        if (want > pl.kblocks / 4) want = pl.kblocks / 4;
    }
    if (want > pl.kblocks) want = pl.kblocks;
    if (g_opt.split_k == 0 && want > 1) {  // automatic: as deep a split as the workspace holds
        const size_t fit = workspace_bytes / out_bytes;
        if (static_cast<size_t>(want) > fit) want = static_cast<int>(fit);
    }
    if (want > 1) {
        const int per = ceil_div(pl.kblocks, want);
        const int split = ceil_div(pl.kblocks, per);
        const size_t need = static_cast<size_t>(split) * batch * M * N * sizeof(float);
        if (split > 1 && workspace_bytes >= need) {
            pl.split_k = split;
            pl.kb_per_split = per;
        }
    }
    // Tail wave.  Example: 4096^3 is 256 pair tiles on 74 clusters = 3.46 waves; the last 34
    // tiles run two-way split as 68 half-length items, so the launch pair takes 3.5 wave-times
    // instead of 4.
    pl.full_tiles = static_cast<int>(tiles);
    pl.tail_tiles = 0;
    pl.tail_split = 1;
    pl.tail_kb_per_split = pl.kblocks;
    pl.tail_bytes = 0;
    if (pl.split_k == 1 && g_opt.tail_split != 0 && pl.kblocks >= 32 && pl.bn >= 128) {
        const int units = pl.pair ? (sms / 2 > 0 ? sms / 2 : 1) : sms;
        const int64_t full = (tiles / units) * units;
        const int64_t tail = tiles - full;
        if (full > 0 && tail > 0 && tail * 10 <= units * 6) {
            int split = static_cast<int>(units / tail);
            if (split > 4) split = 4;
            const int per = ceil_div(pl.kblocks, split);
            split = ceil_div(pl.kblocks, per);
            const size_t need = static_cast<size_t>(split) * tail * (pl.pair ? 2 * kBM : kBM) * pl.bn *
                                sizeof(float);
            if (split > 1 && workspace_bytes >= need) {
                pl.full_tiles = static_cast<int>(full);
                pl.tail_tiles = static_cast<int>(tail);
                pl.tail_split = split;
                pl.tail_kb_per_split = per;
                pl.tail_bytes = need;
            }
        }
    }
    return pl;
}

int gemm_impl(DeviceState& st, const float* A, const float* B, float* const* dest, int n_dest,
              int64_t batch, int64_t M, int64_t N, int64_t K, int transA, int transB, int64_t lda,
              int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB, int64_t strideC,
              float alpha, float beta, int precision, void* workspace, size_t workspace_bytes,
              cudaStream_t stream, const b200_epilogue* ep = nullptr) {
    if (ep != nullptr) {
        if (ep->addend != nullptr && ep->ld_addend < N) return B200_EINVAL;
        if (ep->relu != 0 && ep->relu != 1) return B200_EINVAL;
        if (K == 0 && (ep->bias || ep->addend || ep->relu)) return B200_EINVAL;  // nothing to fuse into
    }
    if (batch < 0 || M < 0 || N < 0 || K < 0) return B200_EINVAL;
    if (precision != B200_PRECISION_3XTF32 && precision != B200_PRECISION_TF32) return B200_EINVAL;
    if (n_dest < 1 || n_dest > kMaxDest || dest == nullptr) return B200_EINVAL;
    if (batch == 0 || M == 0 || N == 0) return B200_OK;
    for (int i = 0; i < n_dest; ++i)
        if (dest[i] == nullptr) return B200_EINVAL;
    if (M > 0x7fffffffll || N > 0x7fffffffll || K > 0x7fffffffll || batch > 0x7fffffffll)
        return B200_ERANGE;
    if (ldc < N || strideC < 0 || strideA < 0 || strideB < 0) return B200_EINVAL;
    if (batch > 1 && strideC < M * ldc && strideC != 0) {
        // matrices closer together than their own extent overlap — unless they sit side by side in the
        // rows of one buffer (the heads of a (S, heads * d) tensor: strideC >= N and batch * strideC <= ldc)
        if (!(strideC >= N && batch * strideC <= ldc)) return B200_EINVAL;
    }
    if (batch > 1 && strideC == 0) return B200_EINVAL;  // every batch would write the same C
    float* C = dest[0];
    if (K == 0) {
        for (int i = 0; i < n_dest; ++i) {
            scale_c_kernel<<<st.sm_count * 4, 256, 0, stream>>>(dest[i], batch, M, N, ldc, strideC,
                                                                beta);
            g_launches.fetch_add(1, std::memory_order_relaxed);
        }
        return static_cast<int>(cudaGetLastError());
    }
    if (A == nullptr || B == nullptr) return B200_EINVAL;
    if (lda < (transA ? M : K) || ldb < (transB ? K : N)) return B200_EINVAL;

    const bool tma_ok = tma_legal(A, lda, strideA, batch) && tma_legal(B, ldb, strideB, batch);
    const bool can_split = (n_dest == 1);
    Plan pl = make_plan(st, batch, M, N, K, tma_ok,
                        (can_split && workspace != nullptr &&
                         (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0)
                            ? workspace_bytes
                            : 0);
    if (n_dest != 1) {  // the tail launch reduces into one C
        pl.full_tiles = static_cast<int>(batch * pl.tiles_m * static_cast<int64_t>(pl.tiles_n));
        pl.tail_tiles = 0;
    }
    const int64_t total = pl.tail_tiles > 0
                              ? static_cast<int64_t>(pl.full_tiles)
                              : batch * pl.tiles_m * static_cast<int64_t>(pl.tiles_n) * pl.split_k;
    if (total > 0x7fffffffll) return B200_ERANGE;

    GemmParams p{};
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    p.batch = static_cast<int>(batch);
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.kblocks = pl.kblocks;
    p.split_k = pl.split_k;
    p.kb_per_split = pl.kb_per_split;
    // The tiles in flight at one time should cover a near-square patch of C: 74 pair tiles are
    // 8 x 9, 148 single tiles (128 x 256) are 16 x 9.
    p.group_m = g_opt.group_m > 0 ? static_cast<int>(g_opt.group_m) : (pl.pair ? 8 : 16);
    p.total_work = static_cast<int>(total);
    p.A = A;
    p.B = B;
    for (int i = 0; i < n_dest; ++i) p.dest[i] = dest[i];
    p.n_dest = n_dest;
    p.lda = lda;
    p.ldb = ldb;
    p.ldc = ldc;
    p.strideA = strideA;
    p.strideB = strideB;
    p.strideC = strideC;
    p.transA = transA ? 1 : 0;
    p.transB = transB ? 1 : 0;
    p.alpha = alpha;
    p.beta = beta;
    p.precision = precision;
    p.promote_every = promote_interval(precision);
    p.tf32_round = g_opt.tf32_round ? 1 : 0;
    p.trunc_hi = g_opt.head_mode == 1 ? 1 : 0;
    p.partial = static_cast<float*>(workspace);
    p.status = st.status;
    if (ep != nullptr) {
        p.bias = ep->bias;
        p.addend = ep->addend;
        p.ld_addend = ep->ld_addend;
        p.relu = ep->relu;
    }
    p.a_vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15u) == 0 && (lda & 3) == 0 &&
                  (strideA & 3) == 0)
                     ? 1
                     : 0;
    p.b_vec_ok = ((reinterpret_cast<uintptr_t>(B) & 15u) == 0 && (ldb & 3) == 0 &&
                  (strideB & 3) == 0)
                     ? 1
                     : 0;
    p.c_vec_ok = ((ldc & 3) == 0 && (strideC & 3) == 0) ? 1 : 0;
    for (int i = 0; i < n_dest; ++i)
        if (reinterpret_cast<uintptr_t>(dest[i]) & 15u) p.c_vec_ok = 0;

    OperandMap oa{}, ob{};
    const bool a_k_contig = !transA;  // A stored M x K
    const bool b_k_contig = transB;   // B stored N x K
    if (pl.tma) {
        int rc = resolve_encoder();
        if (rc) return rc;
        rc = cached_operand_map(&oa, A, a_k_contig, M, K, lda, strideA, batch, kBM, pl.bk);
        if (rc) return rc;
        rc = cached_operand_map(&ob, B, b_k_contig, N, K, ldb, strideB, batch,
                              pl.pair ? pl.bn / 2 : pl.bn, pl.bk);
        if (rc) return rc;
        p.a_lbo = oa.lbo;
        p.a_sbo = oa.sbo;
        p.a_kstep = oa.kstep;
        p.a_ksub = oa.ksub;
        p.a_layout = oa.layout;
        p.b_lbo = ob.lbo;
        p.b_sbo = ob.sbo;
        p.b_kstep = ob.kstep;
        p.b_ksub = ob.ksub;
        p.b_layout = ob.layout;
        p.idesc = make_idesc_tf32(pl.pair ? 2 * kBM : kBM, pl.bn, a_k_contig ? 0 : 1,
                                  b_k_contig ? 0 : 1);
    } else {
        // the register-staged loader always writes K-major 128-byte-swizzled tiles
        p.a_lbo = p.b_lbo = 16;
        p.a_sbo = p.b_sbo = 1024;
        p.a_kstep = p.b_kstep = 32;
        p.a_layout = p.b_layout = kLayoutSw128;
        p.idesc = make_idesc_tf32(kBM, pl.bn, 0, 0);
    }

    auto launch = [&](const GemmParams& q) -> int {
        if (pl.pair) {
            int dev = 0;
            cudaGetDevice(&dev);
            int clusters = max_pair_clusters(dev);
            if (clusters <= 0) return B200_EDEVICE;
            if (clusters > q.total_work) clusters = q.total_work;
            return launch_pair(q, oa.map, ob.map, clusters, stream);
        }
        const int grid = q.total_work < st.sm_count ? q.total_work : st.sm_count;
        return dispatch(pl.bn, pl.bk, pl.tma, q, oa.map, ob.map, grid, stream);
    };
    int rc = launch(p);
    if (rc) return rc;
    if (pl.tail_tiles > 0) {
        GemmParams q = p;
        q.tile_offset = pl.full_tiles;
        q.tail_tiles = pl.tail_tiles;
        q.split_k = pl.tail_split;
        q.kb_per_split = pl.tail_kb_per_split;
        q.total_work = pl.tail_tiles * pl.tail_split;
        rc = launch(q);
        if (rc) return rc;
        fill_schedule(q);
        rc = static_cast<int>(launch_kernel(tail_reduce_kernel, pl.tail_tiles * 8, 256, 0, stream, 1, q,
                                            pl.pair ? 2 * kBM : kBM, pl.bn));
        if (rc) return rc;
    }
    if (pl.split_k > 1) {
        const int64_t elems = batch * M * N;
        // about two blocks of 256 threads per SM: more lanes than that only add blocks (a 96 x 384
        // result in 16 parts took 8.8 us with 8 lanes per element, 5 us with 2)
        const int64_t max_threads = static_cast<int64_t>(st.sm_count) * 2 * 256;
        int lanes = 1;  // threads per element: as many as the parts and the GPU allow
        while (lanes < 32 && lanes * 2 <= pl.split_k && elems * lanes * 2 <= max_threads) lanes *= 2;
        int blocks = static_cast<int>((elems * lanes + 255) / 256);
        if (blocks > st.sm_count * 8) blocks = st.sm_count * 8;
        rc = static_cast<int>(launch_kernel(splitk_reduce_kernel, blocks, 256, 0, stream, 1, p,
                                            static_cast<const float*>(workspace), C, pl.split_k,
                                            static_cast<long long>(batch), static_cast<long long>(M),
                                            static_cast<long long>(N), static_cast<long long>(ldc),
                                            static_cast<long long>(strideC), alpha, beta, lanes));
    }
    return rc;
}

// ------------------------------------------------------------------------------------------
// Allocation-free entry point: scratch and status live in the library's own device image.
// ------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB per GPU that loads the library

// Split-K partial sums of b200_gemm_f32_static_scratch.  Shared by every call on the device
// and never cleared: the GEMM kernel overwrites every partial the reduction later reads.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
// Bits of bounded waits that ran out in launches of that entry point (starts at zero).
static __device__ int g_static_status;

struct StaticState {
    bool ready = false;
    void* scratch = nullptr;  // device address of g_static_scratch on this device
    DeviceState st;           // sm_count + status pointer, no owned allocations
};
StaticState g_static[kMaxDevices];

// In host code the two symbols above are host-side stand-ins, not device addresses: the
// address a kernel may use has to be asked for, once per device, with that device current.
int static_state(StaticState** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return B200_EDEVICE;
    std::lock_guard<std::mutex> lock(g_mutex);
    StaticState& ss = g_static[dev];
    if (!ss.ready) {
        int major = 0, sms = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
            return static_cast<int>(e);
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
            return static_cast<int>(e);
        if (major != 10) return B200_EDEVICE;
        void* scratch = nullptr;
        void* status = nullptr;
        if ((e = cudaGetSymbolAddress(&scratch, g_static_scratch)) != cudaSuccess)
            return static_cast<int>(e);
        if ((e = cudaGetSymbolAddress(&status, g_static_status)) != cudaSuccess)
            return static_cast<int>(e);
        ss.scratch = scratch;
        ss.st.status = static_cast<int*>(status);
        ss.st.cc_major = major;
        ss.st.sm_count = sms;
        ss.st.ready = true;
        ss.ready = true;
    }
    *out = &ss;
    return 0;
}

int grow(void** ptr, size_t* cap, size_t need) {
    if (need <= *cap) return 0;
    if (*ptr) cudaFree(*ptr);
    *ptr = nullptr;
    *cap = 0;
    cudaError_t e = cudaMalloc(ptr, need);
    if (e != cudaSuccess) return static_cast<int>(e);
    *cap = need;
    return 0;
}


// One large product from host buffers as a 2-D wavefront: row panels of A and column panels of B
// are uploaded alternately (A_0, B_0, A_1, B_1, ...).  When B_k lands, the column strip
// C(0..k, k) = A_0..k x B_k is multiplied as ONE product; when A_k lands, the row strip
// C(k, 0..k-1) = A_k x B_0..k-1; each strip is downloaded as soon as it is done.  Uploads, kernels
// and downloads run on streams of their own, so the bus works in both directions under the math.  Thin
// panels keep the work that only the last pair of panels unlocks small while each strip is still
// one large launch.  What can be multiplied grows with the square of what has been uploaded, so the
// SMs idle ~10 ms early on and the math trails the uploads (2 GiB in 41 ms at 52 GB/s) at the end:
// a 16384^3 product takes ~55 ms, close to T_math + T_upload^2 / (4 T_math), the best this order of
// uploads allows.  Overlap needs page-locked host buffers; with pageable ones the copies serialise
// but the result is the same.
int host_wavefront(DeviceState& st, const float* a, const float* b, float* out, int64_t M, int64_t K,
                   int64_t N) {
    cudaError_t e;
    if (!st.pipe_ready) {
        if ((e = cudaStreamCreateWithFlags(&st.s_h2d, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&st.s_comp, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&st.s_comp2, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&st.s_d2h, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&st.s_d2h2, cudaStreamNonBlocking)) != cudaSuccess) return e;
        for (auto& ev : st.ev_a)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        for (auto& ev : st.ev_b)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        for (auto& ev : st.ev_c)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        st.pipe_ready = true;
    }
    // panels of whole 256-row / 256-column tiles, at most 16 per side, none thinner than 1024
    // 12 panels per side measured best at 16384^3 (55.6 ms; 8: 57.8, 16: 58.2, 4: 62.7): thinner
    // strips fill the GPU worse, wider ones leave more work behind the last upload
    const int64_t parts = g_opt.host_pipeline > 1 ? std::min<int64_t>(g_opt.host_pipeline, 16) : 12;
    const int64_t thinnest = parts > 8 ? 1024 : 2048;
    auto panel = [&](int64_t dim) {
        int64_t p = (dim + parts - 1) / parts;
        p = ((p + 255) / 256) * 256;
        return p < thinnest ? thinnest : p;
    };
    const int64_t bm = panel(M), bn = panel(N);
    const int pm = static_cast<int>((M + bm - 1) / bm), pn = static_cast<int>((N + bn - 1) / bn);
    float* dA = st.stage_a;
    float* dB = st.stage_b;
    float* dC = st.stage_c;

    auto upload_a = [&](int i) -> cudaError_t {
        const int64_t r0 = i * bm, rows = std::min<int64_t>(bm, M - r0);
        cudaError_t err = cudaMemcpyAsync(dA + r0 * K, a + r0 * K, static_cast<size_t>(rows) * K * 4,
                                          cudaMemcpyHostToDevice, st.s_h2d);
        return err != cudaSuccess ? err : cudaEventRecord(st.ev_a[i], st.s_h2d);
    };
    auto upload_b = [&](int j) -> cudaError_t {
        const int64_t c0 = j * bn, cols = std::min<int64_t>(bn, N - c0);
        cudaError_t err = cudaMemcpy2DAsync(dB + c0, static_cast<size_t>(N) * 4, b + c0,
                                            static_cast<size_t>(N) * 4, static_cast<size_t>(cols) * 4,
                                            static_cast<size_t>(K), cudaMemcpyHostToDevice, st.s_h2d);
        return err != cudaSuccess ? err : cudaEventRecord(st.ev_b[j], st.s_h2d);
    };
    // C[r0 : r0 + rows, c0 : c0 + cols], once the uploads recorded in `ready` have landed.  The strips
    // are independent products (disjoint parts of C, no scratch), so they alternate between two
    // pairs of a compute and a download stream: a strip's persistent CTAs that find no tile left in
    // its last wave exit and the next strip's CTAs start on those SMs instead of waiting for the whole
    // launch to end, and a strip's download queues behind its own stream's strips only.
    int strips = 0;
    auto strip = [&](int64_t r0, int64_t rows, int64_t c0, int64_t cols, cudaEvent_t ready) -> int {
        if (rows <= 0 || cols <= 0) return 0;
        cudaError_t err;
        cudaStream_t comp = (strips & 1) ? st.s_comp2 : st.s_comp;
        cudaStream_t down = (strips & 1) ? st.s_d2h2 : st.s_d2h;
        if ((err = cudaStreamWaitEvent(comp, ready, 0)) != cudaSuccess) return err;
        float* dest[1] = {dC + r0 * N + c0};
        int rc = gemm_impl(st, dA + r0 * K, dB + c0, dest, 1, 1, rows, cols, K, 0, 0, K, N, N, 0, 0,
                           rows * N, 1.0f, 0.0f, B200_PRECISION_3XTF32, nullptr, 0, comp);
        if (rc) return rc;
        cudaEvent_t done = st.ev_c[strips++];
        if ((err = cudaEventRecord(done, comp)) != cudaSuccess) return err;
        if ((err = cudaStreamWaitEvent(down, done, 0)) != cudaSuccess) return err;
        err = cudaMemcpy2DAsync(out + r0 * N + c0, static_cast<size_t>(N) * 4, dC + r0 * N + c0,
                                static_cast<size_t>(N) * 4, static_cast<size_t>(cols) * 4,
                                static_cast<size_t>(rows), cudaMemcpyDeviceToHost, down);
        return err;
    };

    // The upload stream is in order, so waiting for the newest panel covers all earlier ones.
    const int steps = std::max(pm, pn);
    for (int k = 0; k < steps; ++k) {
        if (k < pm && (e = upload_a(k)) != cudaSuccess) return e;
        if (k < pn && (e = upload_b(k)) != cudaSuccess) return e;
        const int rows_have = std::min(k + 1, pm), cols_before = std::min(k, pn);
        if (k < pn) {  // column strip: every row panel uploaded so far x B_k
            const int64_t c0 = k * bn;
            int rc = strip(0, std::min<int64_t>(rows_have * bm, M), c0, std::min<int64_t>(bn, N - c0), st.ev_b[k]);
            if (rc) return rc;
        }
        if (k < pm) {  // row strip: A_k x every column panel before B_k
            const int64_t r0 = k * bm;
            int rc = strip(r0, std::min<int64_t>(bm, M - r0), 0, std::min<int64_t>(cols_before * bn, N),
                           k < pn ? st.ev_b[k] : st.ev_a[k]);
            if (rc) return rc;
        }
    }
    if ((e = cudaStreamSynchronize(st.s_h2d)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(st.s_comp)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(st.s_comp2)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(st.s_d2h)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(st.s_d2h2)) != cudaSuccess) return e;
    return B200_OK;
}

}  // namespace
}  // namespace b200

namespace b200 {
// For the sharding layer (shard_sm100.cu): the current device's status word and the launch counter.
int* device_status_word(int* rc) {
    DeviceState* st = nullptr;
    *rc = device_state(&st);
    return *rc ? nullptr : st->status;
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace b200

using namespace b200;

extern "C" {

int b200_gemm_f32(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
                  int64_t K, int transA, int transB, int64_t lda, int64_t ldb, int64_t ldc,
                  int64_t strideA, int64_t strideB, int64_t strideC, float alpha, float beta,
                  int precision, void* workspace, size_t workspace_bytes, void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    float* dest[1] = {C};
    if (C == nullptr) return B200_EINVAL;
    if (batch == 1 && strideC == 0) strideC = M * ldc;
    return gemm_impl(*st, A, B, dest, 1, batch, M, N, K, transA, transB, lda, ldb, ldc, strideA,
                     strideB, strideC, alpha, beta, precision, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream));
}

int b200_gemm_f32_fused(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
                        int64_t K, int transA, int transB, int64_t lda, int64_t ldb, int64_t ldc,
                        int64_t strideA, int64_t strideB, int64_t strideC, float alpha, float beta,
                        int precision, const b200_epilogue* epilogue, void* workspace,
                        size_t workspace_bytes, void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    float* dest[1] = {C};
    if (C == nullptr) return B200_EINVAL;
    if (batch == 1 && strideC == 0) strideC = M * ldc;
    return gemm_impl(*st, A, B, dest, 1, batch, M, N, K, transA, transB, lda, ldb, ldc, strideA,
                     strideB, strideC, alpha, beta, precision, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), epilogue);
}

size_t b200_gemm_f32_workspace(int64_t batch, int64_t M, int64_t N, int64_t K) {
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
    DeviceState tmp;
    DeviceState* st = nullptr;
    if (device_state(&st) != 0) {
        tmp.sm_count = 148;
        st = &tmp;
    }
    Plan pl = make_plan(*st, batch, M, N, K, true, static_cast<size_t>(-1));
    if (pl.split_k <= 1) return pl.tail_bytes;
    return static_cast<size_t>(pl.split_k) * batch * M * N * sizeof(float);
}

int b200_gemm_f32_plan(int64_t batch, int64_t M, int64_t N, int64_t K, size_t workspace_bytes,
                       b200_plan_info* out) {
    if (out == nullptr || batch <= 0 || M <= 0 || N <= 0 || K <= 0) return B200_EINVAL;
    DeviceState tmp;
    DeviceState* st = nullptr;
    if (device_state(&st) != 0) {
        tmp.sm_count = 148;
        st = &tmp;
    }
    const Plan pl = make_plan(*st, batch, M, N, K, true, workspace_bytes);
    out->tile_n = pl.bn;
    out->pair = pl.pair ? 1 : 0;
    out->split_k = pl.split_k;
    out->tail_tiles = pl.tail_tiles;
    out->tail_split = pl.tail_tiles > 0 ? pl.tail_split : 1;
    out->kernels = 1 + (pl.split_k > 1 ? 1 : 0) + (pl.tail_tiles > 0 ? 2 : 0);
    out->workspace_used = pl.split_k > 1 ? static_cast<size_t>(pl.split_k) * batch * M * N * sizeof(float)
                                         : pl.tail_bytes;
    return B200_OK;
}

int b200_matmul_f32(const float* a, const float* b, float* out, size_t batch, size_t rows,
                    size_t inner_dim, size_t cols, int a_batched, int b_batched, float beta,
                    void* workspace, size_t workspace_bytes, void* stream) {
    const int64_t M = static_cast<int64_t>(rows), K = static_cast<int64_t>(inner_dim),
                  N = static_cast<int64_t>(cols), nb = static_cast<int64_t>(batch);
    return b200_gemm_f32(a, b, out, nb, M, N, K, 0, 0, K, N, N, a_batched ? M * K : 0,
                         b_batched ? K * N : 0, M * N, 1.0f, beta, B200_PRECISION_3XTF32, workspace,
                         workspace_bytes, stream);
}

int b200_matmul_f32_host(const float* a, const float* b, float* out, size_t batch, size_t rows,
                         size_t inner_dim, size_t cols, int a_batched, int b_batched, float beta) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (a == nullptr || b == nullptr || out == nullptr) return B200_EINVAL;
    const size_t na = (a_batched ? batch : 1) * rows * inner_dim * sizeof(float);
    const size_t nb = (b_batched ? batch : 1) * inner_dim * cols * sizeof(float);
    const size_t nc = batch * rows * cols * sizeof(float);
    if (nc == 0) return B200_OK;
    const size_t nws = b200_gemm_f32_workspace(static_cast<int64_t>(batch), static_cast<int64_t>(rows),
                                               static_cast<int64_t>(cols),
                                               static_cast<int64_t>(inner_dim));
    // The staging buffers, streams and events are per device and shared by every caller: a second
    // thread calling on the same device waits here until the first call has returned.
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> host_lock(g_host_mutex[dev]);
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if ((rc = grow(reinterpret_cast<void**>(&st->stage_a), &st->cap_a, na ? na : 16))) return rc;
        if ((rc = grow(reinterpret_cast<void**>(&st->stage_b), &st->cap_b, nb ? nb : 16))) return rc;
        if ((rc = grow(reinterpret_cast<void**>(&st->stage_c), &st->cap_c, nc))) return rc;
        if (nws && (rc = grow(&st->stage_ws, &st->cap_ws, nws))) return rc;
    }
    // Large single products overlap their transfers with the math, block by block.
    if (batch == 1 && beta == 0.0f && rows >= 4096 && cols >= 4096 && inner_dim >= 512 &&
        (cols % 4) == 0 && (inner_dim % 4) == 0 && g_opt.host_pipeline != 0) {
        rc = host_wavefront(*st, a, b, out, static_cast<int64_t>(rows), static_cast<int64_t>(inner_dim),
                            static_cast<int64_t>(cols));
        if (rc != B200_OK && st->pipe_ready) {
            // leave no copy from or to the caller's buffers in flight behind an error return
            cudaStreamSynchronize(st->s_h2d);
            cudaStreamSynchronize(st->s_comp);
            cudaStreamSynchronize(st->s_comp2);
            cudaStreamSynchronize(st->s_d2h);
            cudaStreamSynchronize(st->s_d2h2);
        }
        return rc;
    }
    cudaStream_t stream = nullptr;
    cudaError_t e;
    if (na && (e = cudaMemcpyAsync(st->stage_a, a, na, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
        return static_cast<int>(e);
    if (nb && (e = cudaMemcpyAsync(st->stage_b, b, nb, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
        return static_cast<int>(e);
    if (beta != 0.0f &&
        (e = cudaMemcpyAsync(st->stage_c, out, nc, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
        return static_cast<int>(e);
    rc = b200_matmul_f32(st->stage_a, st->stage_b, st->stage_c, batch, rows, inner_dim, cols,
                         a_batched, b_batched, beta, nws ? st->stage_ws : nullptr, nws, stream);
    if (rc) return rc;
    if ((e = cudaMemcpyAsync(out, st->stage_c, nc, cudaMemcpyDeviceToHost, stream)) != cudaSuccess)
        return static_cast<int>(e);
    if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return static_cast<int>(e);
    return B200_OK;
}

int b200_conv2d_forward_f32(const float* x, const float* weight, const float* bias, float* y,
                            int64_t n, int64_t c, int64_t h, int64_t w, int64_t out_c, int64_t kh,
                            int64_t kw, int64_t stride, int64_t pad, int relu, int precision,
                            void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (n < 0 || c <= 0 || out_c <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0) return B200_EINVAL;
    if (precision != B200_PRECISION_3XTF32 && precision != B200_PRECISION_TF32) return B200_EINVAL;
    if (h + 2 * pad < kh || w + 2 * pad < kw) return B200_EINVAL;  // empty output
    const int64_t oh = (h + 2 * pad - kh) / stride + 1, ow = (w + 2 * pad - kw) / stride + 1;
    const int64_t M = n * oh * ow, K = c * kh * kw, N = out_c;
    if (M == 0) return B200_OK;
    if (x == nullptr || weight == nullptr || y == nullptr) return B200_EINVAL;
    if (M > 0x7fffffffll || K > 0x7fffffffll || n * c * h * w > 0x7fffffffffffll) return B200_ERANGE;
    const int bn = conv_tile_n(*st, M, N);
    GemmParams p{};
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    p.batch = 1;
    p.tiles_m = ceil_div(M, kBM);
    p.tiles_n = ceil_div(N, bn);
    p.kblocks = ceil_div(K, 32);
    p.split_k = 1;
    p.kb_per_split = p.kblocks;
    p.group_m = 16;
    p.total_work = p.tiles_m * p.tiles_n;
    p.A = x;
    p.B = weight;  // (out_c, K) row-major: the transposed-B form, no transpose is built
    p.dest[0] = y;
    p.n_dest = 1;
    p.ldb = K;
    p.ldc = N;
    p.transB = 1;
    p.alpha = 1.0f;
    p.precision = precision;
    p.promote_every = promote_interval(precision);
    p.status = st->status;
    p.bias = bias;
    p.relu = relu ? 1 : 0;
    p.b_vec_ok = ((reinterpret_cast<uintptr_t>(weight) & 15u) == 0 && (K & 3) == 0) ? 1 : 0;
    p.a_lbo = p.b_lbo = 16;
    p.a_sbo = p.b_sbo = 1024;
    p.a_kstep = p.b_kstep = 32;
    p.a_layout = p.b_layout = kLayoutSw128;
    p.idesc = make_idesc_tf32(kBM, bn, 0, 0);
    p.cv_c = static_cast<int>(c);
    p.cv_h = static_cast<int>(h);
    p.cv_w = static_cast<int>(w);
    p.cv_kh = static_cast<int>(kh);
    p.cv_kw = static_cast<int>(kw);
    p.cv_stride = static_cast<int>(stride);
    p.cv_pad = static_cast<int>(pad);
    p.cv_oh = static_cast<int>(oh);
    p.cv_ow = static_cast<int>(ow);
    p.cv_oc = static_cast<int>(out_c);
    p.cv_store_hw = static_cast<int>(oh * ow);
    p.cv_ones_col = -1;
    p.cv_table = (K <= kConvTableMax && kh < 16384 && kw < 16384 && h + 2 * pad < 16384 && w + 2 * pad < 16384 &&
                  c * h * w < 0x7fffffffll)
                     ? 1
                     : 0;
    const int grid = p.total_work < st->sm_count ? p.total_work : st->sm_count;
    return launch_conv<1>(bn, p, grid, static_cast<cudaStream_t>(stream));
}

size_t b200_conv2d_backward_workspace(int64_t n, int64_t c, int64_t h, int64_t w, int64_t out_c, int64_t kh,
                                      int64_t kw, int64_t stride, int64_t pad) {
    if (n <= 0 || c <= 0 || out_c <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0) return 0;
    if (h + 2 * pad < kh || w + 2 * pad < kw) return 0;
    DeviceState tmp;
    DeviceState* st = nullptr;
    if (device_state(&st) != 0) {
        tmp.sm_count = 148;
        st = &tmp;
    }
    const int64_t oh = (h + 2 * pad - kh) / stride + 1, ow = (w + 2 * pad - kw) / stride + 1;
    return conv_dw_plan(*st, n * oh * ow, out_c, c * kh * kw + 1).bytes;  // + the bias column
}

int b200_conv2d_backward_f32(const float* x, const float* weight, const float* dy, float* dx, float* dweight,
                             float* dbias, int64_t n, int64_t c, int64_t h, int64_t w, int64_t out_c,
                             int64_t kh, int64_t kw, int64_t stride, int64_t pad, float beta, int precision,
                             void* workspace, size_t workspace_bytes, void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (n < 0 || c <= 0 || out_c <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0) return B200_EINVAL;
    if (precision != B200_PRECISION_3XTF32 && precision != B200_PRECISION_TF32) return B200_EINVAL;
    if (h + 2 * pad < kh || w + 2 * pad < kw) return B200_EINVAL;  // empty output
    const int64_t oh = (h + 2 * pad - kh) / stride + 1, ow = (w + 2 * pad - kw) / stride + 1;
    const int64_t positions = n * oh * ow, kcols = c * kh * kw, pixels = n * h * w;
    if (dy == nullptr && positions > 0) return B200_EINVAL;
    if ((dweight != nullptr && x == nullptr) || (dx != nullptr && weight == nullptr)) return B200_EINVAL;
    if (positions > 0x7fffffffll || kcols > 0x7fffffffll || pixels > 0x7fffffffll ||
        out_c * kh * kw > 0x7fffffffll)
        return B200_ERANGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    GemmParams base{};
    base.batch = 1;
    base.n_dest = 1;
    base.group_m = 16;
    base.alpha = 1.0f;
    base.beta = beta;
    base.precision = precision;
    base.promote_every = promote_interval(precision);
    base.status = st->status;
    base.a_lbo = base.b_lbo = 16;
    base.a_sbo = base.b_sbo = 1024;
    base.a_kstep = base.b_kstep = 32;
    base.a_layout = base.b_layout = kLayoutSw128;
    base.cv_c = static_cast<int>(c);
    base.cv_h = static_cast<int>(h);
    base.cv_w = static_cast<int>(w);
    base.cv_kh = static_cast<int>(kh);
    base.cv_kw = static_cast<int>(kw);
    base.cv_stride = static_cast<int>(stride);
    base.cv_pad = static_cast<int>(pad);
    base.cv_oh = static_cast<int>(oh);
    base.cv_ow = static_cast<int>(ow);
    base.cv_oc = static_cast<int>(out_c);
    base.cv_ones_col = -1;

    // The bias sums ride along with the weight gradient as one more column (dOut^T x ones) whenever
    // that product is split; otherwise they have a small kernel of their own.
    bool bias_done = dbias == nullptr;
    if (dweight != nullptr && positions > 0) {
        const int64_t ncols = kcols + (dbias != nullptr ? 1 : 0);
        ConvDwPlan pl = conv_dw_plan(*st, positions, out_c, ncols);
        const bool ws_ok = workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0 &&
                           workspace_bytes >= pl.bytes;
        if (pl.split_k > 1 && ws_ok) {
            GemmParams p = base;
            p.M = static_cast<int>(out_c);
            p.N = static_cast<int>(ncols);
            p.K = static_cast<int>(positions);
            p.tiles_m = pl.tiles_m;
            p.tiles_n = pl.tiles_n;
            p.kblocks = pl.kblocks;
            p.split_k = pl.split_k;
            p.kb_per_split = pl.kb_per_split;
            p.total_work = pl.tiles_m * pl.tiles_n * pl.split_k;
            p.A = dy;
            p.B = x;
            p.dest[0] = dweight;  // not written by a split launch
            p.ldc = ncols;
            p.partial = static_cast<float*>(workspace);
            p.a_vec_ok = ((reinterpret_cast<uintptr_t>(dy) & 15u) == 0 && ((oh * ow) & 3) == 0) ? 1 : 0;
            p.cv_ones_col = dbias != nullptr ? static_cast<int>(kcols) : -1;
            p.idesc = make_idesc_tf32(kBM, pl.bn, 0, 0);
            const int grid = p.total_work < st->sm_count ? p.total_work : st->sm_count;
            if ((rc = launch_conv<2>(pl.bn, p, grid, s))) return rc;
            const int64_t elems = out_c * ncols;
            int blocks = static_cast<int>((elems + 7) / 8);  // 8 warps per block, one element per warp
            if (blocks > st->sm_count * 8) blocks = st->sm_count * 8;
            conv_dw_reduce_kernel<<<blocks, 256, 0, s>>>(static_cast<const float*>(workspace), pl.split_k,
                                                         static_cast<int>(out_c), static_cast<int>(kcols),
                                                         static_cast<int>(ncols), dweight, dbias, beta);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            if ((rc = static_cast<int>(cudaGetLastError()))) return rc;
            bias_done = true;
        } else {  // a single part per tile, stored directly
            ConvDwPlan one = conv_dw_plan(*st, positions, out_c, kcols);
            GemmParams p = base;
            p.M = static_cast<int>(out_c);
            p.N = static_cast<int>(kcols);
            p.K = static_cast<int>(positions);
            p.tiles_m = one.tiles_m;
            p.tiles_n = one.tiles_n;
            p.kblocks = one.kblocks;
            p.split_k = 1;
            p.kb_per_split = one.kblocks;
            p.total_work = one.tiles_m * one.tiles_n;
            p.A = dy;
            p.B = x;
            p.dest[0] = dweight;
            p.ldc = kcols;
            p.a_vec_ok = ((reinterpret_cast<uintptr_t>(dy) & 15u) == 0 && ((oh * ow) & 3) == 0) ? 1 : 0;
            p.c_vec_ok = ((reinterpret_cast<uintptr_t>(dweight) & 15u) == 0 && (kcols & 3) == 0) ? 1 : 0;
            p.cv_ones_col = -1;
            p.idesc = make_idesc_tf32(kBM, one.bn, 0, 0);
            const int grid = p.total_work < st->sm_count ? p.total_work : st->sm_count;
            if ((rc = launch_conv<2>(one.bn, p, grid, s))) return rc;
        }
    } else if (dweight != nullptr && positions == 0) {
        scale_c_kernel<<<st->sm_count * 4, 256, 0, s>>>(dweight, 1, out_c, kcols, kcols, 0, beta);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if ((rc = static_cast<int>(cudaGetLastError()))) return rc;
    }
    if (!bias_done) {
        conv_bias_grad_kernel<<<static_cast<int>(out_c), 256, 0, s>>>(dy, dbias, static_cast<int>(n),
                                                                      static_cast<int>(out_c),
                                                                      static_cast<int>(oh * ow), beta);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if ((rc = static_cast<int>(cudaGetLastError()))) return rc;
    }
    if (dx != nullptr && pixels > 0) {
        GemmParams p = base;
        p.M = static_cast<int>(pixels);
        p.N = static_cast<int>(c);
        p.K = static_cast<int>(out_c * kh * kw);
        const int bn = conv_tile_n(*st, pixels, c);
        p.tiles_m = ceil_div(pixels, kBM);
        p.tiles_n = ceil_div(c, bn);
        p.kblocks = ceil_div(static_cast<int64_t>(p.K), 32);
        p.split_k = 1;
        p.kb_per_split = p.kblocks;
        p.total_work = p.tiles_m * p.tiles_n;
        p.A = dy;
        p.B = weight;
        p.dest[0] = dx;
        p.ldc = c;
        p.cv_store_hw = static_cast<int>(h * w);
        p.cv_table = (stride == 1 && p.K <= kConvTableMax && kh < 16384 && kw < 16384 && h + 2 * pad < 16384 &&
                      w + 2 * pad < 16384 && out_c * oh * ow < 0x7fffffffll)
                         ? 1
                         : 0;
        p.idesc = make_idesc_tf32(kBM, bn, 0, 0);
        const int grid = p.total_work < st->sm_count ? p.total_work : st->sm_count;
        if ((rc = launch_conv<3>(bn, p, grid, s))) return rc;
    }
    return B200_OK;
}

}  // extern "C"

namespace {
template <int CH>
cudaError_t launch_attention(const b200::AttnParams& p, int grid, uint32_t smem, cudaStream_t stream) {
    static uint32_t attr_bytes[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > attr_bytes[dev]) {
        cudaError_t e = cudaFuncSetAttribute(b200::attention_fwd_kernel<CH>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attr_bytes[dev] = smem;
    }
    b200::attention_fwd_kernel<CH><<<grid, b200::kAttnThreads, smem, stream>>>(p);
    return cudaGetLastError();
}
template <int CH>
cudaError_t launch_attention_bwd(const b200::AttnBwdParams& p, int grid, uint32_t smem, cudaStream_t stream) {
    static uint32_t attr_bytes[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > attr_bytes[dev]) {
        cudaError_t e = cudaFuncSetAttribute(b200::attention_bwd_kernel<CH>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attr_bytes[dev] = smem;
    }
    b200::attention_bwd_kernel<CH><<<grid, b200::kAttnThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

// Shared-memory layout of the attention backward kernel; returns the bytes to request, or 0 if
// the tiles do not fit one CTA.
uint32_t attention_bwd_layout(b200::AttnBwdParams& p) {
    const auto up = [](int v, int m) { return (v + m - 1) / m * m; };
    p.sq_pad = up(p.s_q, 32);
    p.sk_pad = up(p.s_k, 32);
    p.dk_pad = up(p.d_k, 32);
    p.dv_pad = up(p.d_v, 32);
    p.dk_n = up(p.d_k, 16);
    p.dv_n = up(p.d_v, 16);
    p.rows_q = up(p.s_q, 8);
    p.rows_k = up(p.s_k, 8);
    p.sz_qa = 128u * p.dk_pad * 4u;
    p.sz_doa = 128u * p.dv_pad * 4u;
    p.sz_kb = static_cast<uint32_t>(p.sk_pad) * p.dk_pad * 4u;
    p.sz_vb = static_cast<uint32_t>(p.sk_pad) * p.dv_pad * 4u;
    p.sz_wt = static_cast<uint32_t>(p.rows_k) * p.sq_pad * 4u;
    p.sz_ds = static_cast<uint32_t>(p.rows_q) * p.sk_pad * 4u;
    p.sz_dst = p.sz_wt;
    p.sz_dot = static_cast<uint32_t>(p.dv_n) * p.sq_pad * 4u;
    p.sz_kt = static_cast<uint32_t>(p.dk_n) * p.sk_pad * 4u;
    p.sz_qt = static_cast<uint32_t>(p.dk_n) * p.sq_pad * 4u;
    uint32_t a = 0;  // the first two products
    p.off_qa = a, a += 2 * p.sz_qa;
    p.off_doa = a, a += 2 * p.sz_doa;
    p.off_kb = a, a += 2 * p.sz_kb;
    p.off_vb = a, a += 2 * p.sz_vb;
    uint32_t b = 0;  // the last three, over the same bytes
    p.off_wt = b, b += 2 * p.sz_wt;
    p.off_ds = b, b += 2 * p.sz_ds;
    p.off_dst = b, b += 2 * p.sz_dst;
    p.off_dot = b, b += 2 * p.sz_dot;
    p.off_kt = b, b += 2 * p.sz_kt;
    p.off_qt = b, b += 2 * p.sz_qt;
    // 16 KB of slack: an A tile with fewer than 128 rows is read past its end; 1 KB to align
    const uint32_t total = std::max(a, b) + 16384u + 1024u;
    return total <= 227u * 1024u ? total : 0u;
}
}  // namespace

namespace b200 {
// For the any-size attention layer (attention_any.cu): does the fused backward kernel take this head?
bool attention_backward_fits_one_cta(int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v) {
    if (s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return false;
    if (s_q > 128 || s_k > kAttnMaxSk || d_k > kAttnMaxD || d_v > kAttnMaxD) return false;
    AttnBwdParams p{};
    p.s_q = static_cast<int>(s_q);
    p.s_k = static_cast<int>(s_k);
    p.d_k = static_cast<int>(d_k);
    p.d_v = static_cast<int>(d_v);
    return attention_bwd_layout(p) != 0;
}
}  // namespace b200

extern "C" {

int b200_attention_f32_strided(const float* q, const float* k, const float* v, const float* mask,
                               float* out, float* weights, int64_t batch, int64_t heads, int64_t s_q,
                               int64_t s_k, int64_t d_k, int64_t d_v, const int64_t q_strides[3],
                               const int64_t k_strides[3], const int64_t v_strides[3],
                               const int64_t out_strides[3], float scale, int precision, void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (batch < 0 || heads <= 0 || s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return B200_EINVAL;
    if (precision != B200_PRECISION_3XTF32 && precision != B200_PRECISION_TF32) return B200_EINVAL;
    if (q_strides == nullptr || k_strides == nullptr || v_strides == nullptr || out_strides == nullptr)
        return B200_EINVAL;
    if (q_strides[2] < d_k || k_strides[2] < d_k || v_strides[2] < d_v || out_strides[2] < d_v) return B200_EINVAL;
    for (int i = 0; i < 2; ++i)
        if (q_strides[i] < 0 || k_strides[i] < 0 || v_strides[i] < 0 || out_strides[i] < 0) return B200_EINVAL;
    if (s_q > 128 || s_k > kAttnMaxSk || d_k > kAttnMaxD || d_v > kAttnMaxD) return B200_ERANGE;
    if (batch == 0) return B200_OK;
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return B200_EINVAL;
    if (batch > 0x7fffffffll / heads) return B200_ERANGE;
    AttnParams p{};
    p.q = q;
    p.k = k;
    p.v = v;
    p.mask = mask;
    p.out = out;
    p.weights = weights;
    p.q_bs = q_strides[0], p.q_hs = q_strides[1], p.q_ld = q_strides[2];
    p.k_bs = k_strides[0], p.k_hs = k_strides[1], p.k_ld = k_strides[2];
    p.v_bs = v_strides[0], p.v_hs = v_strides[1], p.v_ld = v_strides[2];
    p.o_bs = out_strides[0], p.o_hs = out_strides[1], p.o_ld = out_strides[2];
    p.batch = static_cast<int>(batch * heads);
    p.heads = static_cast<int>(heads);
    p.s_q = static_cast<int>(s_q);
    p.s_k = static_cast<int>(s_k);
    p.d_k = static_cast<int>(d_k);
    p.d_v = static_cast<int>(d_v);
    p.sk_pad = static_cast<int>((s_k + 31) / 32 * 32);
    p.dk_pad = static_cast<int>((d_k + 31) / 32 * 32);
    p.dv_pad = static_cast<int>((d_v + 15) / 16 * 16);
    p.scale = scale;
    p.precision = precision;
    p.status = st->status;
    const uint32_t q_bytes = 128u * p.dk_pad * 4u, k_bytes = static_cast<uint32_t>(p.sk_pad) * p.dk_pad * 4u;
    const uint32_t p_bytes = 128u * p.sk_pad * 4u, v_bytes = static_cast<uint32_t>(p.dv_pad) * p.sk_pad * 4u;
    const uint32_t region1 = std::max(2 * (q_bytes + k_bytes), 2 * p_bytes);
    const uint32_t smem = region1 + 2 * v_bytes + 1024;
    const int grid = static_cast<int>(std::min<int64_t>(p.batch, st->sm_count));
    cudaError_t e = cudaSuccess;
    switch (p.sk_pad / 32) {
        case 1: e = launch_attention<1>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
        case 2: e = launch_attention<2>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
        case 3: e = launch_attention<3>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
        default: e = launch_attention<4>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
    }
    if (e != cudaSuccess) return static_cast<int>(e);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_OK;
}

int b200_attention_f32(const float* q, const float* k, const float* v, const float* mask, float* out,
                       float* weights, int64_t batch, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
                       float scale, int precision, void* stream) {
    if (s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return B200_EINVAL;
    const int64_t qs[3] = {s_q * d_k, 0, d_k}, ks[3] = {s_k * d_k, 0, d_k};
    const int64_t vs[3] = {s_k * d_v, 0, d_v}, os[3] = {s_q * d_v, 0, d_v};
    return b200_attention_f32_strided(q, k, v, mask, out, weights, batch, 1, s_q, s_k, d_k, d_v, qs, ks, vs, os,
                                      scale, precision, stream);
}

int b200_attention_backward_f32_strided(const float* q, const float* k, const float* v, const float* mask,
                                        const float* dout, float* dq, float* dk, float* dv, int64_t batch,
                                        int64_t heads, int64_t s_q, int64_t s_k, int64_t d_k, int64_t d_v,
                                        const int64_t q_strides[3], const int64_t k_strides[3],
                                        const int64_t v_strides[3], const int64_t out_strides[3], float scale,
                                        float beta, int precision, void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (batch < 0 || heads <= 0 || s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return B200_EINVAL;
    if (precision != B200_PRECISION_3XTF32 && precision != B200_PRECISION_TF32) return B200_EINVAL;
    if (q_strides == nullptr || k_strides == nullptr || v_strides == nullptr || out_strides == nullptr)
        return B200_EINVAL;
    if (q_strides[2] < d_k || k_strides[2] < d_k || v_strides[2] < d_v || out_strides[2] < d_v) return B200_EINVAL;
    for (int i = 0; i < 2; ++i)
        if (q_strides[i] < 0 || k_strides[i] < 0 || v_strides[i] < 0 || out_strides[i] < 0) return B200_EINVAL;
    if (s_q > 128 || s_k > kAttnMaxSk || d_k > kAttnMaxD || d_v > kAttnMaxD) return B200_ERANGE;
    if (batch == 0) return B200_OK;
    if (q == nullptr || k == nullptr || v == nullptr || dout == nullptr) return B200_EINVAL;
    if (batch > 0x7fffffffll / heads) return B200_ERANGE;
    AttnBwdParams p{};
    p.q = q;
    p.k = k;
    p.v = v;
    p.mask = mask;
    p.dout = dout;
    p.dq = dq;
    p.dk = dk;
    p.dv = dv;
    p.q_bs = q_strides[0], p.q_hs = q_strides[1], p.q_ld = q_strides[2];
    p.k_bs = k_strides[0], p.k_hs = k_strides[1], p.k_ld = k_strides[2];
    p.v_bs = v_strides[0], p.v_hs = v_strides[1], p.v_ld = v_strides[2];
    p.o_bs = out_strides[0], p.o_hs = out_strides[1], p.o_ld = out_strides[2];
    p.batch = static_cast<int>(batch * heads);
    p.heads = static_cast<int>(heads);
    p.s_q = static_cast<int>(s_q);
    p.s_k = static_cast<int>(s_k);
    p.d_k = static_cast<int>(d_k);
    p.d_v = static_cast<int>(d_v);
    p.scale = scale;
    p.beta = beta;
    p.precision = precision;
    p.status = st->status;
    const uint32_t smem = attention_bwd_layout(p);
    if (smem == 0) return B200_ERANGE;  // the tiles of this shape do not fit one CTA
    const int grid = static_cast<int>(std::min<int64_t>(p.batch, st->sm_count));
    cudaError_t e = cudaSuccess;
    switch (p.sk_pad / 32) {
        case 1: e = launch_attention_bwd<1>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
        case 2: e = launch_attention_bwd<2>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
        case 3: e = launch_attention_bwd<3>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
        default: e = launch_attention_bwd<4>(p, grid, smem, static_cast<cudaStream_t>(stream)); break;
    }
    if (e != cudaSuccess) return static_cast<int>(e);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return B200_OK;
}

int b200_attention_backward_f32(const float* q, const float* k, const float* v, const float* mask,
                                const float* dout, float* dq, float* dk, float* dv, int64_t batch, int64_t s_q,
                                int64_t s_k, int64_t d_k, int64_t d_v, float scale, float beta, int precision,
                                void* stream) {
    if (s_q <= 0 || s_k <= 0 || d_k <= 0 || d_v <= 0) return B200_EINVAL;
    const int64_t qs[3] = {s_q * d_k, 0, d_k}, ks[3] = {s_k * d_k, 0, d_k};
    const int64_t vs[3] = {s_k * d_v, 0, d_v}, os[3] = {s_q * d_v, 0, d_v};
    return b200_attention_backward_f32_strided(q, k, v, mask, dout, dq, dk, dv, batch, 1, s_q, s_k, d_k, d_v, qs, ks,
                                               vs, os, scale, beta, precision, stream);
}

int b200_gemm_f32_colshard(const float* A, const float* B, float* const* dest, int n_dest,
                           int64_t M, int64_t N, int64_t K, int64_t col0, int64_t cols, int64_t lda,
                           int64_t ldb, int64_t ldc, int precision, void* stream) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (dest == nullptr || n_dest < 1 || n_dest > kMaxDest) return B200_EINVAL;
    if (col0 < 0 || cols < 0 || col0 + cols > N || ldb < N || ldc < N) return B200_EINVAL;
    float* shifted[kMaxDest];
    for (int i = 0; i < n_dest; ++i) {
        if (dest[i] == nullptr) return B200_EINVAL;
        shifted[i] = dest[i] + col0;
    }
    return gemm_impl(*st, A, B ? B + col0 : nullptr, shifted, n_dest, 1, M, cols, K, 0, 0, lda, ldb,
                     ldc, 0, 0, M * ldc, 1.0f, 0.0f, precision, nullptr, 0,
                     static_cast<cudaStream_t>(stream));
}

int b200_gemm_f32_static_scratch(const float* A, const float* B, float* C, int64_t batch, int64_t M,
                                 int64_t N, int64_t K, int transA, int transB, int64_t lda,
                                 int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB,
                                 int64_t strideC, float alpha, float beta, int precision,
                                 int* device_status, void* stream) {
    StaticState* ss = nullptr;
    int rc = static_state(&ss);
    if (rc) return rc;
    if (C == nullptr) return B200_EINVAL;
    if (batch < 0 || M < 0 || N < 0 || K < 0) return B200_EINVAL;
    if (batch == 1 && strideC == 0) strideC = M * ldc;
    // The plan is the one b200_gemm_f32 makes when it is handed 4 MiB of workspace: the automatic
    // K-split is as deep as the fixed scratch holds (possibly not split at all), and a last wave
    // whose K-split partials do not fit runs unsplit.  Only a split that the caller FORCED through
    // the "split_k" option and that does not fit is refused: there is no honest way to run it.
    if (batch > 0 && M > 0 && N > 0 && K > 0 && g_opt.split_k > 1) {
        const int64_t kblocks = (K + 31) / 32;
        const int64_t want = std::min<int64_t>(g_opt.split_k, kblocks);
        const int64_t per = (kblocks + want - 1) / want;
        const int64_t split = (kblocks + per - 1) / per;
        const size_t one = static_cast<size_t>(batch) * M * N * sizeof(float);
        if (split > 1 && one > kStaticScratchBytes / static_cast<size_t>(split)) return B200_ENOSPACE;
    }
    DeviceState st = ss->st;  // plain copy: holds no allocation
    if (device_status != nullptr) st.status = device_status;
    float* dest[1] = {C};
    return gemm_impl(st, A, B, dest, 1, batch, M, N, K, transA, transB, lda, ldb, ldc, strideA,
                     strideB, strideC, alpha, beta, precision, ss->scratch, kStaticScratchBytes,
                     static_cast<cudaStream_t>(stream));
}

int b200_gemm_status(void) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    int word = 0;
    if ((e = cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
        return static_cast<int>(e);
    if (word != 0) cudaMemset(st->status, 0, sizeof(int));
    // the word inside the library's device image that b200_gemm_f32_static_scratch reports to when
    // its caller passed no status pointer (its address is known once that entry point has run here)
    int dev = 0;
    cudaGetDevice(&dev);
    int* static_word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (dev >= 0 && dev < kMaxDevices && g_static[dev].ready) static_word = g_static[dev].st.status;
    }
    if (static_word != nullptr) {
        int w2 = 0;
        if ((e = cudaMemcpy(&w2, static_word, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
            return static_cast<int>(e);
        if (w2 != 0) cudaMemset(static_word, 0, sizeof(int));
        word |= w2;
    }
    return word != 0 ? B200_ETIMEDOUT : B200_OK;
}

int b200_gemm_selftest_timeout(unsigned budget_us, int* observed_host) {
    DeviceState* st = nullptr;
    int rc = device_state(&st);
    if (rc) return rc;
    if (budget_us == 0 || budget_us > 100000) return B200_EINVAL;  // at most 0.1 s
    int* observed = nullptr;
    cudaError_t e = cudaMalloc(&observed, 2 * sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaMemset(observed, 0, 2 * sizeof(int));
    wait_timeout_selftest_kernel<<<1, 32>>>(st->status, static_cast<unsigned long long>(budget_us) * 1000ull,
                                            observed);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    int host[2] = {0, 0};
    if (e == cudaSuccess) e = cudaMemcpy(host, observed, sizeof(host), cudaMemcpyDeviceToHost);
    cudaFree(observed);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (observed_host != nullptr) {
        observed_host[0] = host[0];
        observed_host[1] = host[1];
    }
    return B200_OK;
}

uint64_t b200_gemm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200_gemm_set_option(const char* name, long value) {
    if (name == nullptr) return B200_EINVAL;
    if (!std::strcmp(name, "tile_n")) {
        if (value != 0 && value != 32 && value != 64 && value != 128 && value != 256)
            return B200_EINVAL;
        g_opt.tile_n = value;
    } else if (!std::strcmp(name, "split_k")) {
        if (value < 0) return B200_EINVAL;
        g_opt.split_k = value;
    } else if (!std::strcmp(name, "promote_every")) {
        if (value < 0) return B200_EINVAL;
        g_opt.promote_every = value;
    } else if (!std::strcmp(name, "force_ldg")) {
        g_opt.force_ldg = value ? 1 : 0;
    } else if (!std::strcmp(name, "group_m")) {
        if (value < 0 || value > 4096) return B200_EINVAL;
        g_opt.group_m = value;
    } else if (!std::strcmp(name, "tail_split")) {
        g_opt.tail_split = value ? 1 : 0;
    } else if (!std::strcmp(name, "host_pipeline")) {
        if (value < 0 || value > 16) return B200_EINVAL;
        g_opt.host_pipeline = value;
    } else if (!std::strcmp(name, "tf32_round")) {
        g_opt.tf32_round = value ? 1 : 0;
    } else if (!std::strcmp(name, "pair_mode")) {
        if (value < 0 || value > 2) return B200_EINVAL;
        g_opt.pair_mode = value;
    } else if (!std::strcmp(name, "head_mode")) {
        if (value < 0 || value > 1) return B200_EINVAL;
        g_opt.head_mode = value;
    } else if (!std::strcmp(name, "block_k")) {
        if (value != 0 && value != 32 && value != 64) return B200_EINVAL;
        g_opt.block_k = value;
    } else if (!std::strcmp(name, "split_warps")) {
        if (value != 0 && value != 8) return B200_EINVAL;
        g_opt.split_warps = value;
    } else if (!std::strcmp(name, "pair_workers")) {
        if (value != 8 && value != 16) return B200_EINVAL;
        g_opt.pair_workers = value;
    } else if (!std::strcmp(name, "pdl")) {
        g_opt.pdl = value ? 1 : 0;
    } else if (!std::strcmp(name, "map_cache")) {
        g_opt.map_cache = value ? 1 : 0;
    } else {
        return B200_EINVAL;
    }
    return B200_OK;
}

const char* b200_gemm_strerror(int code) {
    switch (code) {
        case B200_OK: return "success";
        case B200_EINVAL: return "invalid argument (shape, stride, flag or null pointer)";
        case B200_ERANGE: return "dimension out of the range the kernels index";
        case B200_ENOSPACE: return "scratch too small for this shape (the fixed 4 MiB of b200_gemm_f32_static_scratch)";
        case B200_EDEVICE: return "no sm_100 device, or the driver lacks cuTensorMapEncodeTiled";
        case B200_ETIMEDOUT: return "a bounded device-side wait ran out";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}

}  // extern "C"
