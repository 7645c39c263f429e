// Runs the reference's own unit tests (src/runtests.cpp, compiled unmodified with -DUSE_CUDA and
// -Dmain=reference_runtests_main) against this library's wrappers: the six CPU known-answer tests
// and the nine CUDA-vs-CPU operator tests (src/runtests.cpp:883-900).  The two "smoke" tests at
// src/runtests.cpp:904-905 are left out: under USE_CUDA they hand uninitialised device pointers to
// the kernels (transformerWeights::d_* is never set there), which is undefined behaviour on any GPU
// build including the reference's.
#include <cstdio>

int test_matmul_square();
int test_matmul_rectangular();
int test_RMSNorm();
int test_rope();
int test_softmax();
int test_swiglu();
int test_cuda_gemv();
int test_cuda_gemv_f16();
int test_cuda_rmsnorm();
int test_cuda_rope();
int test_cuda_swiglu();
int test_cuda_softmax_multihead();
int test_cuda_scale_multihead();
int test_cuda_residual_add();
int test_cuda_aggregation();

int main() {
    printf("--- Lighter++ unit tests against liblpp_b200 ---\n");
    int failures = 0;
    failures += test_matmul_square();
    failures += test_matmul_rectangular();
    failures += test_RMSNorm();
    failures += test_rope();
    failures += test_softmax();
    failures += test_swiglu();
    failures += test_cuda_gemv();
    failures += test_cuda_gemv_f16();
    failures += test_cuda_rmsnorm();
    failures += test_cuda_rope();
    failures += test_cuda_swiglu();
    failures += test_cuda_softmax_multihead();
    failures += test_cuda_scale_multihead();
    failures += test_cuda_residual_add();
    failures += test_cuda_aggregation();
    printf(failures == 0 ? "ALL TESTS PASSED\n" : "%d TESTS FAILED\n", failures);
    return failures;
}
