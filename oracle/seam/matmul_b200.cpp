// src/cuda/matmul_b200.cpp — what a maintainer of cpp-ai-engine adds IN PLACE OF
// src/cuda/kernels_matmul.cu to run every matrix product of the engine on libb200gemm.so.
//
// It defines the two symbols that unit defines: the seam engine::cuda::ops::matmul
// (include/engine/detail/cuda_ops.hpp:46-47; body src/cuda/kernels_matmul.cu:761-898) and
// shared::collect_matmul_probes (src/cuda/kernels_matmul.cu:904), and uses only the engine's own
// Storage accessors (include/engine/detail/storage.hpp:99-117) and the helpers its CUDA units
// already share (src/cuda/kernels_common.cuh: launched_ok, scratch_buffer).
//
// This file is compiled against the UNMODIFIED reference by `make -C oracle ref_cuda` (test
// infrastructure: the result runs the reference's own CPU/GPU parity tests over the new kernels);
// it is not part of the library.
#include "b200_gemm.h"

#include "engine/cuda.hpp"
#include "engine/detail/cuda_ops.hpp"
#include "engine/detail/storage.hpp"

#include <stdexcept>
#include <string>
#include <vector>

namespace engine {
namespace cuda {
namespace ops {

namespace shared {
// Declared in src/cuda/kernels_common.cuh, defined in src/cuda/kernels.cu.  (That header also
// declares a __global__ kernel, so a plain C++ unit re-states the three declarations it needs.)
bool launched_ok(const char* what, Storage& out);
float* scratch_buffer(size_t floats);
struct Probe {
    const char* name;
    const void* fn;
    int block_threads;
};
// The occupancy report (src/cuda/kernels.cu:1448-1498) asks the matmul unit for its kernels;
// the library's kernels are not visible to cudaFuncGetAttributes from here, so it lists none.
void collect_matmul_probes(std::vector<Probe>&) {}
}  // namespace shared

bool matmul(const Storage& a, const Storage& b, Storage& out, size_t batch, size_t rows,
            size_t inner_dim, size_t cols, bool a_batched, bool b_batched, float beta) {
    // The engine's own switch and its empty-product rule stay (src/cuda/kernels_matmul.cu:763-764):
    // with the backend disabled the caller asked for the CPU loop.  Nothing else is declined: no
    // size threshold, no kernel that cannot take beta, no grid limit on the batch.
    if (!enabled()) return false;
    if (batch == 0 || rows == 0 || inner_dim == 0 || cols == 0) return false;
    if (out.size() != batch * rows * cols) return false;

    const float* pa = a.device();                          // uploads if the device copy is stale
    const float* pb = b.device();
    float* pc = (beta == 0.0f) ? out.device_write()         // never uploaded, fully overwritten
                               : out.device_mut();          // uploaded first, then accumulated into
    // split-K partials live in the engine's own growable scratch (src/cuda/kernels.cu:593-604)
    const size_t ws_bytes = b200_gemm_f32_workspace(static_cast<int64_t>(batch), static_cast<int64_t>(rows),
                                                    static_cast<int64_t>(cols), static_cast<int64_t>(inner_dim));
    float* ws = ws_bytes ? shared::scratch_buffer((ws_bytes + 3) / 4) : nullptr;
    // MatmulKernel::TensorCore / TensorCoreFp16 are the engine's opt-in reduced-precision selectors
    // (include/engine/cuda.hpp:153-177): they map to the single-product TF32 mode.  Everything
    // else, Auto included, is the fp32-accurate default.
    const MatmulKernel sel = matmul_kernel();
    const int precision = (sel == MatmulKernel::TensorCore || sel == MatmulKernel::TensorCoreFp16)
                              ? B200_PRECISION_TF32
                              : B200_PRECISION_3XTF32;
    const int64_t M = static_cast<int64_t>(rows), K = static_cast<int64_t>(inner_dim), N = static_cast<int64_t>(cols);
    const int rc = b200_gemm_f32(pa, pb, pc, static_cast<int64_t>(batch), M, N, K, 0, 0, K, N, N,
                                 a_batched ? M * K : 0, b_batched ? K * N : 0, M * N, 1.0f, beta, precision,
                                 ws, ws ? ws_bytes : 0, /*stream=*/nullptr);
    if (rc != 0) {
        if (beta == 0.0f) out.revert_device_write();        // as the reference does on a failed launch
        throw std::runtime_error(std::string("b200 matmul: ") + b200_gemm_strerror(rc));
    }
    return shared::launched_ok("matmul_b200", out);         // the engine's launch accounting
}

}  // namespace ops
}  // namespace cuda
}  // namespace engine
