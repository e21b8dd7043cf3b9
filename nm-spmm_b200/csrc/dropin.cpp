// The reference's C++ entry points (include/NM-SpMM.h of the reference, lines
// 10-24) as thin wrappers over the C-ABI.  Error behaviour mirrors the reference:
// the functions return void; an unsupported sparsity family prints the reference's
// "Not support!" line and launches nothing (src/kernel_64x128_8x8.cu:264-265,
// 584-585); other failures are reported on stderr.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "NM-SpMM.h"
#include "nmspmm_b200.h"

namespace {

bool near(float a, float b) { return std::fabs(a - b) < 1e-6f; }

// The reference's signatures carry no choice of arithmetic.  A program linked against this
// library without source changes selects the tensor-core path by setting the environment
// variable NMSPMM_PATH=tf32 before its first launcher call (anything else: exact FP32).
int dropin_path()
{
    static const int path = [] {
        const char* v = std::getenv("NMSPMM_PATH");
        return (v && (std::strcmp(v, "tf32") == 0 || std::strcmp(v, "TF32") == 0)) ? NMSPMM_PATH_TF32 : NMSPMM_PATH_FP32;
    }();
    return path;
}

void report(const char* who, int rc)
{
    if (rc != NMSPMM_OK)
        std::fprintf(stderr, "%s: %s (cuda error %d)\n", who, nmspmm_status_string(rc), nmspmm_last_cuda_error());
}

void launch_low(const char* who, int layout_ns, float* A, float* B, int* D, float* C, int M, int N, int K, int W,
                float sparsity, int SPLIT_K)
{
    (void)W;
    int n_keep;
    if (near(sparsity, 0.75f) || near(sparsity, 0.875f)) {
        std::printf("Not support! Please use high sparsity version for sparsity %.3f\n", sparsity);
        return;
    } else if (near(sparsity, 0.5f)) {
        n_keep = 16;
    } else if (near(sparsity, 0.625f)) {
        n_keep = 12;
    } else if (near(sparsity, 0.0f)) {
        n_keep = 32;
    } else {
        return;                                  // the reference launches nothing for other values
    }
    nmspmm_gemm_desc d = { M, N, K, n_keep, NMSPMM_FORMAT_LOW, layout_ns, dropin_path(), SPLIT_K > 1 ? SPLIT_K : 0, 0 };
    report(who, nmspmm_gemm_with_cached_workspace(&d, A, B, D, nullptr, C, nullptr));
}

void launch_high(const char* who, int layout_ns, float* A, float* B, int* D, int* column_info, float* C, int M, int N,
                 int K, int W, float sparsity, int SPLIT_K)
{
    (void)W;
    int n_keep;
    if (near(sparsity, 0.5f) || near(sparsity, 0.625f)) {
        std::printf("Not support! Please use low sparsity version for sparsity %.2f\n", sparsity);
        return;
    } else if (near(sparsity, 0.75f)) {
        n_keep = 8;
    } else if (near(sparsity, 0.875f)) {
        n_keep = 4;
    } else {
        return;
    }
    nmspmm_gemm_desc d = { M, N, K, n_keep, NMSPMM_FORMAT_HIGH, layout_ns, dropin_path(), SPLIT_K > 1 ? SPLIT_K : 0, 0 };
    report(who, nmspmm_gemm_with_cached_workspace(&d, A, B, D, column_info, C, nullptr));
}

}  // namespace

void PreProcessing_low_sparsity(int* DT, int W, int Q, int Ns)
{
    report("PreProcessing_low_sparsity", nmspmm_preprocess_low_host(DT, W, Q, Ns));
}

void PreProcessing_high_sparsity(int* column_info, int pruning_M, int pruning_N, int* DT, int W, int Q, int N, int Ns)
{
    report("PreProcessing_high_sparsity", nmspmm_preprocess_high_host(column_info, pruning_M, pruning_N, DT, W, Q, N, Ns));
}

void transIndex(int* DT, int W, int N, int Q, int& pruning_N, int& pruning_M)
{
    report("transIndex", nmspmm_trans_index_host(DT, W, N, Q, &pruning_N, &pruning_M));
}

#define NMSPMM_DROPIN(NAME, NS)                                                                                         \
    void nmGEMM_##NAME##_matrices_low_sparsity(float* A, float* B, int* D, float* C, int M, int N, int K, int W,        \
                                               float sparsity, int SPLIT_K)                                             \
    {                                                                                                                   \
        launch_low("nmGEMM_" #NAME "_matrices_low_sparsity", NS, A, B, D, C, M, N, K, W, sparsity, SPLIT_K);            \
    }                                                                                                                   \
    void nmGEMM_##NAME##_matrices_high_sparsity(float* A, float* B, int* D, int* column_info, float* C, int M, int N,   \
                                                int K, int W, float sparsity, int SPLIT_K)                              \
    {                                                                                                                   \
        launch_high("nmGEMM_" #NAME "_matrices_high_sparsity", NS, A, B, D, column_info, C, M, N, K, W, sparsity,       \
                    SPLIT_K);                                                                                           \
    }

NMSPMM_DROPIN(huge, 128)
NMSPMM_DROPIN(large, 64)
NMSPMM_DROPIN(medium, 64)
NMSPMM_DROPIN(small, 32)
