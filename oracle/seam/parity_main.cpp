// TEST INFRASTRUCTURE.  Runs two suites of the reference's own test program — its CPU/GPU parity
// tests (tests/test_cuda_parity.cpp) and the index replay (tests/test_cuda_indexing.cpp) — against
// a build of the unmodified reference whose matmul unit is oracle/seam/matmul_b200.cpp.  The other
// suites need the fixture directory of the reference's source tree and have nothing to do with the
// device seam; they are left out.  Same closing lines as tests/test_main.cpp.
#include "test_support.hpp"

int main() {
    std::cout << "====================================================\n";
    std::cout << "  cpp-ai-engine CUDA suites over libb200gemm.so      \n";
    std::cout << "====================================================\n";
    run_cuda_indexing_tests();
    run_cuda_parity_tests();
    std::cout << "\n====================================================\n";
    if (testing::g_failures == 0) {
        std::cout << "  ALL TESTS PASSED (" << testing::g_checks << " checks)\n";
    } else {
        std::cout << "  " << testing::g_failures << " OF " << testing::g_checks << " CHECKS FAILED\n";
    }
    std::cout << "====================================================\n";
    return testing::g_failures == 0 ? 0 : 1;
}
