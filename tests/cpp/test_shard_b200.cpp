// A C++ caller of the sharded product (include/b200_gemm.h: b200_shard_comm_*, b200_gemm_f32_sharded,
// b200_matmul_f32_host_sharded) on the GPUs of one box: one process, one thread per GPU.
//   fused mode   the peers' C buffers and flag blocks are plain device pointers of the other GPUs
//                (peer access enabled), the product kernel stores every tile into all of them
//   NCCL mode    a communicator from ncclCommInitAll, one ncclAllGather of packed column blocks
//   host mode    every rank uploads 1/world of A's rows and its columns of B, rows gathered over NVLink
// Every rank's result is compared, bit for bit, with the unsharded product of GPU 0 and, on sampled
// rows, with the CPU oracle (test infrastructure).  The reference has no multi-GPU path to mirror
// (src/cuda/runtime.cu:83).
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "../../include/b200_gemm.h"
#include "../../oracle/matmul_oracle.h"

namespace {

int g_checks = 0, g_failures = 0;
std::mutex g_print;
void check(bool ok, const std::string& what) {
    std::lock_guard<std::mutex> lock(g_print);
    ++g_checks;
    if (!ok) ++g_failures;
    std::printf("%s %s\n", ok ? "  [ ok ]" : "  [FAIL]", what.c_str());
}

#define CUDA_OK(x)                                                                        \
    do {                                                                                  \
        cudaError_t e_ = (x);                                                             \
        if (e_ != cudaSuccess) {                                                          \
            std::printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            std::exit(2);                                                                 \
        }                                                                                 \
    } while (0)

// a reusable barrier for the rank threads (host side)
struct HostBarrier {
    std::mutex m;
    std::condition_variable cv;
    int count = 0, generation = 0, n;
    explicit HostBarrier(int n_) : n(n_) {}
    void wait() {
        std::unique_lock<std::mutex> lock(m);
        const int gen = generation;
        if (++count == n) {
            count = 0;
            ++generation;
            cv.notify_all();
        } else {
            cv.wait(lock, [&] { return gen != generation; });
        }
    }
};

double scaled_error(const float* got, const float* want, size_t n) {
    double worst = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const double w = want[i];
        worst = std::fmax(worst, std::fabs(got[i] - w) / std::fmax(1.0, std::fabs(w)));
    }
    return worst;
}

// ncclCommInitAll / ncclCommDestroy from the system's NCCL, found at run time like the library does
using InitAllFn = int (*)(void**, int, const int*);
using DestroyFn = int (*)(void*);

}  // namespace

int main() {
    int ngpu = 0;
    CUDA_OK(cudaGetDeviceCount(&ngpu));
    if (ngpu < 2) {
        std::printf("SKIPPED: needs two GPUs, found %d\n", ngpu);
        return 0;
    }
    const int world = 2;
    const int64_t M = 1024, N = 2048, K = 512;
    std::vector<float> a(M * K), b(K * N);
    std::mt19937 gen(1);
    std::normal_distribution<float> dist(0.0f, 1.0f / std::sqrt(static_cast<float>(K)));
    for (auto& v : a) v = dist(gen);
    for (auto& v : b) v = dist(gen);

    for (int r = 0; r < world; ++r) {
        CUDA_OK(cudaSetDevice(r));
        for (int p = 0; p < world; ++p) {
            if (p == r) continue;
            int can = 0;
            CUDA_OK(cudaDeviceCanAccessPeer(&can, r, p));
            if (!can) {
                std::printf("SKIPPED: GPU %d cannot access GPU %d\n", r, p);
                return 0;
            }
            cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) CUDA_OK(e);
            cudaGetLastError();
        }
    }

    // per-rank device buffers, visible to every thread (one address space)
    std::vector<float*> dA(world), dB(world), dC(world);
    std::vector<uint32_t*> dFlags(world);
    for (int r = 0; r < world; ++r) {
        CUDA_OK(cudaSetDevice(r));
        CUDA_OK(cudaMalloc(&dA[r], M * K * 4));
        CUDA_OK(cudaMalloc(&dB[r], K * N * 4));
        CUDA_OK(cudaMalloc(&dC[r], M * N * 4));
        CUDA_OK(cudaMalloc(&dFlags[r], 64 * 4));
        CUDA_OK(cudaMemcpy(dA[r], a.data(), M * K * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(dB[r], b.data(), K * N * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemset(dFlags[r], 0, 64 * 4));
        CUDA_OK(cudaDeviceSynchronize());
    }
    // the unsharded product on GPU 0
    std::vector<float> whole(M * N);
    {
        CUDA_OK(cudaSetDevice(0));
        float* t = nullptr;
        CUDA_OK(cudaMalloc(&t, M * N * 4));
        int rc = b200_gemm_f32(dA[0], dB[0], t, 1, M, N, K, 0, 0, K, N, N, 0, 0, M * N, 1.0f, 0.0f,
                               B200_PRECISION_3XTF32, nullptr, 0, nullptr);
        check(rc == 0, "unsharded product launches");
        CUDA_OK(cudaMemcpy(whole.data(), t, M * N * 4, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaFree(t));
        std::vector<float> cpu(64 * N);
        oracle_matmul_f32(a.data(), b.data(), cpu.data(), 1, 64, static_cast<size_t>(K), static_cast<size_t>(N), 1, 1, 0);
        check(scaled_error(whole.data(), cpu.data(), 64 * N) <= 1e-5, "unsharded product vs the CPU oracle (64 rows)");
    }

    // NCCL communicators for the two devices (system NCCL, resolved like the library resolves it)
    void* nccl[2] = {nullptr, nullptr};
    DestroyFn nccl_destroy = nullptr;
    {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h != nullptr) {
            auto init_all = reinterpret_cast<InitAllFn>(dlsym(h, "ncclCommInitAll"));
            nccl_destroy = reinterpret_cast<DestroyFn>(dlsym(h, "ncclCommDestroy"));
            const int devs[2] = {0, 1};
            if (init_all == nullptr || init_all(nccl, 2, devs) != 0) nccl[0] = nccl[1] = nullptr;
        }
        check(nccl[0] != nullptr, "NCCL communicators for two GPUs (ncclCommInitAll)");
    }

    HostBarrier hb(world);
    std::vector<std::vector<float>> fused(world), gathered(world), host_cols(world);
    std::vector<int> rcs(world * 8, -999);
    auto rank_main = [&](int r) {
        CUDA_OK(cudaSetDevice(r));
        b200_shard_comm* comm = nullptr;
        rcs[r * 8 + 0] = b200_shard_comm_create(&comm, r, world);
        rcs[r * 8 + 1] = b200_shard_comm_set_peers(comm, dC.data(), dFlags.data());
        hb.wait();
        // ---- fused: twice in a row (the second call overwrites a C the first one filled)
        CUDA_OK(cudaMemset(dC[r], 0xff, M * N * 4));
        CUDA_OK(cudaDeviceSynchronize());
        hb.wait();
        int rc = 0;
        for (int it = 0; it < 2 && rc == 0; ++it)
            rc = b200_gemm_f32_sharded(comm, B200_SHARD_FUSED, dA[r], dB[r], dC[r], M, N, K, K, N, N,
                                       B200_PRECISION_3XTF32, nullptr);
        rcs[r * 8 + 2] = rc;
        CUDA_OK(cudaDeviceSynchronize());
        rcs[r * 8 + 3] = b200_gemm_status();
        fused[r].resize(M * N);
        CUDA_OK(cudaMemcpy(fused[r].data(), dC[r], M * N * 4, cudaMemcpyDeviceToHost));
        hb.wait();
        // ---- NCCL gather
        if (nccl[r] != nullptr) {
            rcs[r * 8 + 4] = b200_shard_comm_set_nccl(comm, nccl[r]);
            CUDA_OK(cudaMemset(dC[r], 0xff, M * N * 4));
            CUDA_OK(cudaDeviceSynchronize());
            hb.wait();
            rc = b200_gemm_f32_sharded(comm, B200_SHARD_NCCL, dA[r], dB[r], dC[r], M, N, K, K, N, N,
                                       B200_PRECISION_3XTF32, nullptr);
            rcs[r * 8 + 5] = rc;
            CUDA_OK(cudaDeviceSynchronize());
            gathered[r].resize(M * N);
            CUDA_OK(cudaMemcpy(gathered[r].data(), dC[r], M * N * 4, cudaMemcpyDeviceToHost));
            hb.wait();
            // ---- host buffers: this rank's rows of A, its columns of B, its columns of C
            int64_t col0 = 0, cols = 0;
            b200_shard_columns(N, world, r, &col0, &cols);
            const int64_t per = M / world;
            float *ha = nullptr, *hbuf = nullptr, *hc = nullptr;
            CUDA_OK(cudaMallocHost(&ha, per * K * 4));
            CUDA_OK(cudaMallocHost(&hbuf, K * cols * 4));
            CUDA_OK(cudaMallocHost(&hc, M * cols * 4));
            std::memcpy(ha, a.data() + r * per * K, per * K * 4);
            for (int64_t k = 0; k < K; ++k) std::memcpy(hbuf + k * cols, b.data() + k * N + col0, cols * 4);
            std::memset(hc, 0xff, M * cols * 4);
            hb.wait();
            rc = b200_matmul_f32_host_sharded(comm, ha, hbuf, hc, M, N, K, 0);
            rcs[r * 8 + 6] = rc;
            host_cols[r].assign(hc, hc + M * cols);
            CUDA_OK(cudaFreeHost(ha));
            CUDA_OK(cudaFreeHost(hbuf));
            CUDA_OK(cudaFreeHost(hc));
            hb.wait();
        }
        rcs[r * 8 + 7] = b200_shard_comm_destroy(comm);
    };
    std::vector<std::thread> threads;
    for (int r = 0; r < world; ++r) threads.emplace_back(rank_main, r);
    for (auto& t : threads) t.join();

    for (int r = 0; r < world; ++r) {
        const std::string who = "rank " + std::to_string(r) + ": ";
        check(rcs[r * 8 + 0] == 0 && rcs[r * 8 + 1] == 0, who + "communicator created, peers registered");
        check(rcs[r * 8 + 2] == 0 && rcs[r * 8 + 3] == 0, who + "fused sharded product ran, no device wait ran out");
        check(std::memcmp(fused[r].data(), whole.data(), M * N * 4) == 0,
              who + "fused: all of C, bit-identical to the unsharded product");
        if (nccl[r] != nullptr) {
            check(rcs[r * 8 + 4] == 0 && rcs[r * 8 + 5] == 0, who + "NCCL sharded product ran");
            check(std::memcmp(gathered[r].data(), whole.data(), M * N * 4) == 0,
                  who + "NCCL: all of C, bit-identical to the unsharded product");
            int64_t col0 = 0, cols = 0;
            b200_shard_columns(N, world, r, &col0, &cols);
            // a strip is a product of its own: its K may be split where the whole product's is not, so
            // the columns agree to rounding; a misplaced row or chunk would be off by the size of the values
            bool same = rcs[r * 8 + 6] == 0 && host_cols[r].size() == static_cast<size_t>(M * cols);
            double worst = 0.0;
            for (int64_t i = 0; same && i < M; ++i)
                worst = std::fmax(worst, scaled_error(host_cols[r].data() + i * cols, whole.data() + i * N + col0,
                                                      static_cast<size_t>(cols)));
            check(same && worst <= 2e-6, who + "host buffers: own columns of C match the unsharded product");
        }
        check(rcs[r * 8 + 7] == 0, who + "communicator destroyed");
    }
    if (nccl_destroy != nullptr)
        for (int r = 0; r < world; ++r)
            if (nccl[r] != nullptr) nccl_destroy(nccl[r]);
    std::printf("\n%s (%d checks, %d failures)\n", g_failures == 0 ? "ALL TESTS PASSED" : "FAILED", g_checks, g_failures);
    return g_failures == 0 ? 0 : 1;
}
