// Column-sharded products over the GPUs of one node behind the C ABI (include/b200_gemm.h):
// the communicator handle, the cross-GPU barrier that brackets the fused gather, the NCCL gather,
// and the host-buffer pipeline of the sharded product.  The reference has nothing here to mirror
// (single device, src/cuda/runtime.cu:83).
//
// One rank per GPU: a process per GPU, or one thread per GPU inside one process.  Never two ranks
// on one GPU — the barrier kernels of different ranks wait for one another.
#include "../../include/b200_gemm.h"
#include "shard_layout.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>

namespace b200 {
int* device_status_word(int* rc);  // gemm_sm100.cu: the current device's status word of the bounded waits
void count_launch();               // gemm_sm100.cu: b200_gemm_launch_count bookkeeping
}  // namespace b200

namespace {

constexpr int kMaxRanks = 8;
constexpr int kStatBarrier = 64;  // status bit: a cross-GPU barrier wait ran out
constexpr unsigned long long kBarrierBudgetNs = 2000000000ull;  // 2 s, like every other device wait
constexpr int kMaxChunks = B200_SHARD_MAX_CHUNKS;
constexpr int kMaxColumnParts = 2;  // host-buffer pipeline: B's columns are uploaded in this many pieces

// ------------------------------------------------------------------------------------------
// NCCL, resolved at run time: the library has no link-time dependency on it.  If the process
// already holds a libnccl.so.2 (a Python process that imported torch; a C++ program linked against
// NCCL) that copy is used, so that communicators created by the caller and the calls made here
// belong to the same NCCL.
// ------------------------------------------------------------------------------------------
struct NcclApi {
    int (*all_gather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*error_string)(int) = nullptr;
    bool tried = false, ok = false;
};
NcclApi g_nccl;
std::mutex g_nccl_mutex;
constexpr int kNcclFloat32 = 7;  // ncclFloat32 of nccl.h

bool load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.tried) return g_nccl.ok;
    g_nccl.tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) return false;
    g_nccl.all_gather = reinterpret_cast<decltype(g_nccl.all_gather)>(dlsym(h, "ncclAllGather"));
    g_nccl.error_string = reinterpret_cast<decltype(g_nccl.error_string)>(dlsym(h, "ncclGetErrorString"));
    g_nccl.ok = g_nccl.all_gather != nullptr;
    return g_nccl.ok;
}

// ------------------------------------------------------------------------------------------
// cross-GPU barrier
// ------------------------------------------------------------------------------------------
struct BarrierArgs {
    uint32_t* flags[kMaxRanks];  // flags[r]: rank r's block of `world` words, mapped into this process
    int rank, world;
    uint32_t epoch;
    int* status;
};

// Thread t tells rank t "rank `rank` has reached barrier `epoch`" (a system-scope release store into
// word `rank` of rank t's block: everything this GPU wrote before — the tiles the product kernel
// stored into the peers' C among it — is visible to a GPU that sees the flag), then waits until word
// t of this rank's own block says the same of rank t.  Epochs only grow, so a fast peer that is
// already one barrier ahead does no harm.  The wait is bounded: after two seconds it records
// kStatBarrier in *status and returns.
__global__ void shard_barrier_kernel(const BarrierArgs a) {
    const int t = static_cast<int>(threadIdx.x);
    if (t >= a.world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags[t] + a.rank), "r"(a.epoch) : "memory");
    const uint32_t* mine = a.flags[a.rank] + t;
    unsigned long long start = 0;
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int32_t>(v - a.epoch) >= 0) break;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (start == 0) start = now;
        if (now - start > kBarrierBudgetNs) {
            atomicOr(a.status, kStatBarrier);
            break;
        }
        __nanosleep(200);
    }
}

}  // namespace

struct b200_shard_comm {
    int rank = 0, world = 1;
    int device = 0;
    // fused mode: every rank's C (M x N, leading dimension ldc) and flag block, as mapped here
    bool have_peers = false;
    float* c_bufs[kMaxRanks] = {};
    uint32_t* flags[kMaxRanks] = {};
    uint32_t epoch = 0;
    // NCCL mode
    void* nccl = nullptr;
    float* gathered = nullptr;  // [world][M][width] staging of the packed column blocks
    size_t cap_gathered = 0;
    // host-buffer pipeline (created on first use)
    bool pipe_ready = false;
    cudaStream_t s_h2d = nullptr, s_comm = nullptr, s_comp = nullptr, s_d2h = nullptr;
    cudaEvent_t ev_b[kMaxColumnParts] = {}, ev_a[kMaxChunks] = {}, ev_g[kMaxChunks] = {};
    cudaEvent_t ev_c[kMaxChunks * kMaxColumnParts] = {};
    float* d_a = nullptr;  // gathered A, [chunk][rank][chunk_rows][K]
    float* d_b = nullptr;  // this rank's columns of B, K x cols
    float* d_c = nullptr;  // this rank's columns of C, [chunk][rank][chunk_rows][cols]
    void* d_ws = nullptr;
    size_t cap_a = 0, cap_b = 0, cap_c = 0, cap_ws = 0;
};

namespace {

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

int launch_barrier(b200_shard_comm* c, cudaStream_t stream) {
    int rc = 0;
    int* status = b200::device_status_word(&rc);
    if (rc) return rc;
    BarrierArgs a{};
    for (int r = 0; r < c->world; ++r) a.flags[r] = c->flags[r];
    a.rank = c->rank;
    a.world = c->world;
    a.epoch = ++c->epoch;
    a.status = status;
    shard_barrier_kernel<<<1, 32, 0, stream>>>(a);
    b200::count_launch();
    return static_cast<int>(cudaGetLastError());
}

int check_device(const b200_shard_comm* c) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    return dev == c->device ? 0 : B200_EINVAL;  // a communicator belongs to the device it was made on
}

}  // namespace

extern "C" {

int b200_shard_comm_create(b200_shard_comm** out, int rank, int world) {
    if (out == nullptr || world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return B200_EINVAL;
    int rc = 0;
    (void)b200::device_status_word(&rc);  // also rejects a device that is not sm_100
    if (rc) return rc;
    b200_shard_comm* c = new (std::nothrow) b200_shard_comm();
    if (c == nullptr) return B200_ENOSPACE;
    c->rank = rank;
    c->world = world;
    cudaGetDevice(&c->device);
    *out = c;
    return B200_OK;
}

int b200_shard_comm_set_peers(b200_shard_comm* c, float* const* c_bufs, uint32_t* const* flags) {
    if (c == nullptr || c_bufs == nullptr || flags == nullptr) return B200_EINVAL;
    for (int r = 0; r < c->world; ++r) {
        if (c_bufs[r] == nullptr || flags[r] == nullptr) return B200_EINVAL;
        if (reinterpret_cast<uintptr_t>(flags[r]) & 3u) return B200_EINVAL;
    }
    for (int r = 0; r < c->world; ++r) {
        c->c_bufs[r] = c_bufs[r];
        c->flags[r] = flags[r];
    }
    c->have_peers = true;
    return B200_OK;
}

int b200_shard_comm_set_nccl(b200_shard_comm* c, void* nccl_comm) {
    if (c == nullptr || nccl_comm == nullptr) return B200_EINVAL;
    if (!load_nccl()) return B200_EDEVICE;
    c->nccl = nccl_comm;
    return B200_OK;
}

int b200_shard_comm_destroy(b200_shard_comm* c) {
    if (c == nullptr) return B200_OK;
    int dev = -1;
    cudaGetDevice(&dev);
    if (dev != c->device) cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    if (c->gathered) cudaFree(c->gathered);
    if (c->d_a) cudaFree(c->d_a);
    if (c->d_b) cudaFree(c->d_b);
    if (c->d_c) cudaFree(c->d_c);
    if (c->d_ws) cudaFree(c->d_ws);
    if (c->pipe_ready) {
        cudaStreamDestroy(c->s_h2d);
        cudaStreamDestroy(c->s_comm);
        cudaStreamDestroy(c->s_comp);
        cudaStreamDestroy(c->s_d2h);
        for (auto& ev : c->ev_b) cudaEventDestroy(ev);
        for (auto& ev : c->ev_a) cudaEventDestroy(ev);
        for (auto& ev : c->ev_g) cudaEventDestroy(ev);
        for (auto& ev : c->ev_c) cudaEventDestroy(ev);
    }
    if (dev >= 0 && dev != c->device) cudaSetDevice(dev);
    delete c;
    return B200_OK;
}

void b200_shard_columns(int64_t N, int world, int rank, int64_t* col0, int64_t* cols) {
    b200_shard::columns(N, world, rank, col0, cols);
}

int b200_gemm_f32_sharded(b200_shard_comm* c, int mode, const float* A, const float* B, float* C, int64_t M,
                          int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int precision,
                          void* stream_) {
    if (c == nullptr || C == nullptr) return B200_EINVAL;
    if (mode != B200_SHARD_FUSED && mode != B200_SHARD_NCCL) return B200_EINVAL;
    if (M < 0 || N < 0 || K < 0 || ldc < N || ldb < N) return B200_EINVAL;
    if (int rc = check_device(c)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int64_t col0 = 0, cols = 0;
    b200_shard::columns(N, c->world, c->rank, &col0, &cols);
    if (M == 0 || N == 0) return B200_OK;

    if (mode == B200_SHARD_FUSED) {
        if (c->world > 1 && !c->have_peers) return B200_EINVAL;
        if (c->world > 1 && c->c_bufs[c->rank] != C) return B200_EINVAL;  // C must be the registered buffer
        // Entry barrier: no rank stores into a peer's C before every rank has finished, in stream
        // order, whatever it had queued that still reads the previous result.
        if (c->world > 1)
            if (int rc = launch_barrier(c, stream)) return rc;
        if (cols > 0) {
            // own C first, then the peers in ring order: the ranks do not all push to one GPU at once
            float* dest[kMaxRanks];
            dest[0] = C;
            int n = 1;
            for (int i = 1; i < c->world; ++i) dest[n++] = c->c_bufs[(c->rank + i) % c->world];
            int rc = b200_gemm_f32_colshard(A, B, dest, n, M, N, K, col0, cols, lda, ldb, ldc, precision, stream);
            if (rc) return rc;
        }
        // Exit barrier: when it has passed on this GPU, every peer's product kernel (and with it
        // every store into this GPU's C) had completed before that peer raised its flag.
        if (c->world > 1)
            if (int rc = launch_barrier(c, stream)) return rc;
        return B200_OK;
    }

    // NCCL: the own columns are computed straight into this rank's slot of a packed
    // [world][M][width] staging buffer, gathered in place, and every block is copied to its columns.
    if (c->world == 1) {
        float* dest[1] = {C};
        return b200_gemm_f32_colshard(A, B, dest, 1, M, N, K, 0, N, lda, ldb, ldc, precision, stream);
    }
    if (c->nccl == nullptr) return B200_EINVAL;
    int64_t width = 0;
    for (int r = 0; r < c->world; ++r) {
        int64_t r0, rc_;
        b200_shard::columns(N, c->world, r, &r0, &rc_);
        width = std::max(width, rc_);
    }
    const size_t block = static_cast<size_t>(M) * width;
    if (int rc = grow(reinterpret_cast<void**>(&c->gathered), &c->cap_gathered, block * c->world * sizeof(float)))
        return rc;
    float* mine = c->gathered + block * c->rank;
    if (cols > 0) {
        // b200_gemm_f32 on the column block, written packed (leading dimension = width)
        int rc = b200_gemm_f32(A, B + col0, mine, 1, M, cols, K, 0, 0, lda, ldb, width, 0, 0, M * width, 1.0f, 0.0f,
                               precision, nullptr, 0, stream);
        if (rc) return rc;
    }
    int nrc = g_nccl.all_gather(mine, c->gathered, block, kNcclFloat32, c->nccl, stream);
    if (nrc != 0) return B200_EDEVICE;
    for (int r = 0; r < c->world; ++r) {
        int64_t r0, rc_;
        b200_shard::columns(N, c->world, r, &r0, &rc_);
        if (rc_ == 0) continue;
        cudaError_t e = cudaMemcpy2DAsync(C + r0, static_cast<size_t>(ldc) * 4, c->gathered + block * r,
                                          static_cast<size_t>(width) * 4, static_cast<size_t>(rc_) * 4,
                                          static_cast<size_t>(M), cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return B200_OK;
}

int b200_shard_host_plan(int64_t M, int world, int chunks, b200_shard_host_layout* out) {
    return b200_shard::host_plan(M, world, chunks, out) ? B200_OK : B200_EINVAL;
}

int b200_matmul_f32_host_sharded(b200_shard_comm* c, const float* a_rows, const float* b_cols, float* c_cols,
                                 int64_t M, int64_t N, int64_t K, int chunks) {
    if (c == nullptr || a_rows == nullptr || b_cols == nullptr || c_cols == nullptr) return B200_EINVAL;
    if (M <= 0 || N <= 0 || K <= 0) return B200_EINVAL;
    if (int rc = check_device(c)) return rc;
    if (c->world > 1 && c->nccl == nullptr) return B200_EINVAL;
    b200_shard_host_layout lay{};
    if (!b200_shard::host_plan(M, c->world, chunks, &lay)) return B200_EINVAL;
    int64_t col0 = 0, cols = 0;
    b200_shard::columns(N, c->world, c->rank, &col0, &cols);
    const int P = lay.chunks;
    const int64_t cr = lay.chunk_rows, strip_rows = cr * c->world;
    cudaError_t e;
    if (!c->pipe_ready) {
        if ((e = cudaStreamCreateWithFlags(&c->s_h2d, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&c->s_comm, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&c->s_comp, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&c->s_d2h, cudaStreamNonBlocking)) != cudaSuccess) return e;
        for (auto& ev : c->ev_b)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        for (auto& ev : c->ev_a)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        for (auto& ev : c->ev_g)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        for (auto& ev : c->ev_c)
            if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return e;
        c->pipe_ready = true;
    }
    // B's columns go up in two halves when a half is still wide enough for efficient strips (2048
    // columns): the first strip needs only the first half, so the math starts after half of B and one
    // chunk of A instead of after all of B (16384^3 on two GPUs: 33.8 -> 31.2 ms; no difference on four).
    const int H = (cols >= 4096 && cols % 64 == 0) ? kMaxColumnParts : 1;
    const int64_t part = cols / H;
    const size_t ws_bytes = cols > 0 ? b200_gemm_f32_workspace(1, strip_rows, part, K) : 0;
    if (int rc = grow(reinterpret_cast<void**>(&c->d_a), &c->cap_a, static_cast<size_t>(M) * K * 4)) return rc;
    if (int rc = grow(reinterpret_cast<void**>(&c->d_b), &c->cap_b, static_cast<size_t>(K) * std::max<int64_t>(cols, 1) * 4))
        return rc;
    if (int rc = grow(reinterpret_cast<void**>(&c->d_c), &c->cap_c, static_cast<size_t>(M) * std::max<int64_t>(cols, 1) * 4))
        return rc;
    if (ws_bytes)
        if (int rc = grow(&c->d_ws, &c->cap_ws, ws_bytes)) return rc;

    int rc = B200_OK;
    auto fail = [&](int code) {
        // leave no copy from or to the caller's buffers in flight behind an error return
        cudaStreamSynchronize(c->s_h2d);
        cudaStreamSynchronize(c->s_comm);
        cudaStreamSynchronize(c->s_comp);
        cudaStreamSynchronize(c->s_d2h);
        return code;
    };
    auto upload_b = [&](int h) -> cudaError_t {
        if (cols > 0) {
            cudaError_t err = cudaMemcpy2DAsync(c->d_b + h * part, static_cast<size_t>(cols) * 4, b_cols + h * part,
                                                static_cast<size_t>(cols) * 4, static_cast<size_t>(part) * 4,
                                                static_cast<size_t>(K), cudaMemcpyHostToDevice, c->s_h2d);
            if (err != cudaSuccess) return err;
        }
        return cudaEventRecord(c->ev_b[h], c->s_h2d);
    };
    // this rank's rows of chunk ch -> its slot of the chunk's gathered block; then every rank's rows
    // of the chunk, over NVLink, into local memory before any kernel reads them
    auto upload_and_gather_a = [&](int ch) -> int {
        float* strip_a = c->d_a + static_cast<size_t>(ch) * strip_rows * K;
        float* slot = strip_a + static_cast<size_t>(c->rank) * cr * K;
        cudaError_t err = cudaMemcpyAsync(slot, a_rows + static_cast<size_t>(ch) * cr * K, static_cast<size_t>(cr) * K * 4,
                                          cudaMemcpyHostToDevice, c->s_h2d);
        if (err != cudaSuccess) return err;
        if ((err = cudaEventRecord(c->ev_a[ch], c->s_h2d)) != cudaSuccess) return err;
        if ((err = cudaStreamWaitEvent(c->s_comm, c->ev_a[ch], 0)) != cudaSuccess) return err;
        if (c->world > 1) {
            if (g_nccl.all_gather(slot, strip_a, static_cast<size_t>(cr) * K, kNcclFloat32, c->nccl, c->s_comm) != 0)
                return B200_EDEVICE;
        }
        return cudaEventRecord(c->ev_g[ch], c->s_comm);
    };
    // the strip's rows x column part h of this rank's columns, as one product, and its way home
    auto strip = [&](int ch, int h) -> int {
        if (cols == 0) return 0;
        cudaError_t err;
        if ((err = cudaStreamWaitEvent(c->s_comp, c->ev_g[ch], 0)) != cudaSuccess) return err;
        if ((err = cudaStreamWaitEvent(c->s_comp, c->ev_b[h], 0)) != cudaSuccess) return err;
        const float* strip_a = c->d_a + static_cast<size_t>(ch) * strip_rows * K;
        float* strip_c = c->d_c + static_cast<size_t>(ch) * strip_rows * cols + h * part;
        int r = b200_gemm_f32(strip_a, c->d_b + h * part, strip_c, 1, strip_rows, part, K, 0, 0, K, cols, cols, 0, 0,
                              strip_rows * cols, 1.0f, 0.0f, B200_PRECISION_3XTF32, ws_bytes ? c->d_ws : nullptr,
                              ws_bytes, c->s_comp);
        if (r) return r;
        cudaEvent_t done = c->ev_c[ch * kMaxColumnParts + h];
        if ((err = cudaEventRecord(done, c->s_comp)) != cudaSuccess) return err;
        if ((err = cudaStreamWaitEvent(c->s_d2h, done, 0)) != cudaSuccess) return err;
        for (int rk = 0; rk < c->world; ++rk) {
            // rows of rank rk in this chunk: global rows [rk * rows_per_rank + ch * cr, + cr)
            const int64_t g0 = rk * lay.rows_per_rank + static_cast<int64_t>(ch) * cr;
            err = cudaMemcpy2DAsync(c_cols + static_cast<size_t>(g0) * cols + h * part, static_cast<size_t>(cols) * 4,
                                    strip_c + static_cast<size_t>(rk) * cr * cols, static_cast<size_t>(cols) * 4,
                                    static_cast<size_t>(part) * 4, static_cast<size_t>(cr), cudaMemcpyDeviceToHost,
                                    c->s_d2h);
            if (err != cudaSuccess) return err;
        }
        return 0;
    };
    // upload order: B part 0, A chunk 0, the other parts of B, the other chunks of A
    if ((e = upload_b(0)) != cudaSuccess) return fail(e);
    if ((rc = upload_and_gather_a(0)) != 0) return fail(rc);
    for (int h = 1; h < H; ++h)
        if ((e = upload_b(h)) != cudaSuccess) return fail(e);
    for (int h = 0; h < H; ++h)
        if ((rc = strip(0, h)) != 0) return fail(rc);
    for (int ch = 1; ch < P; ++ch) {
        if ((rc = upload_and_gather_a(ch)) != 0) return fail(rc);
        for (int h = 0; h < H; ++h)
            if ((rc = strip(ch, h)) != 0) return fail(rc);
    }
    if ((e = cudaStreamSynchronize(c->s_h2d)) != cudaSuccess) return fail(e);
    if ((e = cudaStreamSynchronize(c->s_comm)) != cudaSuccess) return fail(e);
    if ((e = cudaStreamSynchronize(c->s_comp)) != cudaSuccess) return fail(e);
    if ((e = cudaStreamSynchronize(c->s_d2h)) != cudaSuccess) return fail(e);
    return B200_OK;
}

}  // extern "C"
