// Timing sweeps of the reference's two benchmark suites, written against the public
// interface include/NM-SpMM.h only, so that the same source links either to the reference's
// own kernels (recompiled for sm_100a) or to this repository's library.  Measurement
// infrastructure: not part of the product, not a parity check (no result is compared).
//
// Default mode -- the 5 x 20 grid of benchmark/kernel_performance/run_test/nmspmm/
// run_nmspmm.sh:16-18 of the reference (M in {256 .. 4096}, twenty (N, K) pairs of LLM linear
// layers), for one sparsity.  As in that script, a shape's figure is the best
// dense-equivalent TFLOP/s (2 M N K / t, tests/test_nmspmm.cu:139) over the four entry points
// that accept the shape and SPLIT_K in {1, 2, 4, 8}.
//
// Table mode (first argument "table") -- benchmark/different_kernel/run_nmspmm.sh:16-37: six
// square-ish shapes, one line per (shape, entry point) with the dense-equivalent TFLOP/s of
// each SPLIT_K in {1, 2, 4, 8}.
//
// Inputs are seeded pseudo-random operands in the reference's formats (values do not matter
// for the timing; indices are valid sorted N:M indices).
//
// usage: sweep <sparsity> [iterations] [m ...]       (one line per shape on stdout)
//        sweep table <sparsity> [iterations]         (one line per shape and entry point)
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "NM-SpMM.h"

#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));    \
            exit(1);                                                                      \
        }                                                                                 \
    } while (0)

static uint64_t mix(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

typedef void (*LowFn)(float*, float*, int*, float*, int, int, int, int, float, int);
typedef void (*HighFn)(float*, float*, int*, int*, float*, int, int, int, int, float, int);
struct Entry { const char* name; int ms, ns, layout; LowFn low; HighFn high; };

int main(int argc, char** argv)
{
    const bool table = argc > 1 && std::string(argv[1]) == "table";
    if (table) { --argc; ++argv; }
    if (argc < 2) {
        fprintf(stderr, "usage: %s [table] <sparsity> [iterations] [m ...]\n", argv[0]);
        return 2;
    }
    const float sparsity = static_cast<float>(atof(argv[1]));
    const int iters = argc > 2 ? atoi(argv[2]) : 10;
    std::vector<int> Ms;
    for (int i = 3; i < argc; ++i) Ms.push_back(atoi(argv[i]));
    if (Ms.empty()) Ms = { 256, 512, 1024, 2048, 4096 };
    const int tM[6] = { 512, 512, 512, 1024, 2048, 4096 }, tN[6] = { 512, 1024, 2048, 2048, 4096, 4096 },
              tK[6] = { 512, 1024, 2048, 2048, 4096, 4096 };
    if (table) Ms.assign(1, 0);
    const int Ns[20] = { 2048, 6144, 2048, 5632, 4096, 12288, 4096, 11008, 5120, 15360, 5120, 13824, 6656, 19968, 6656, 17920, 8192, 24576, 8192, 22016 };
    const int Ks[20] = { 2048, 2048, 5632, 2048, 4096, 4096, 11008, 4096, 5120, 5120, 13824, 5120, 6656, 6656, 17920, 6656, 8192, 8192, 22016, 8192 };
    const Entry entries[4] = {
        { "small", 32, 32, 32, nmGEMM_small_matrices_low_sparsity, nmGEMM_small_matrices_high_sparsity },
        { "medium", 32, 64, 64, nmGEMM_medium_matrices_low_sparsity, nmGEMM_medium_matrices_high_sparsity },
        { "large", 64, 64, 64, nmGEMM_large_matrices_low_sparsity, nmGEMM_large_matrices_high_sparsity },
        { "huge", 64, 128, 128, nmGEMM_huge_matrices_low_sparsity, nmGEMM_huge_matrices_high_sparsity },
    };
    const int n_keep = static_cast<int>(std::lround(32 * (1.0 - sparsity)));
    const bool high = sparsity > 0.7f;                    // 75 % and 87.5 % go through the high-sparsity entry points
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    printf("# sparsity %.3f, n_keep %d, %d timed launches per configuration\n", sparsity, n_keep, iters);
    for (int M0 : Ms) {
        for (int s = 0; s < (table ? 6 : 20); ++s) {
            const int M = table ? tM[s] : M0, N = table ? tN[s] : Ns[s], K = table ? tK[s] : Ks[s];
            const int W = K / 32 * n_keep, Q = N / VEC_LEN;
            // operands in the reference's formats
            std::vector<float> hA(static_cast<size_t>(M) * K), hB(static_cast<size_t>(W) * N);
            for (size_t i = 0; i < hA.size(); ++i) hA[i] = static_cast<float>(mix(i) >> 40) * (1.0f / 16777216.0f);
            for (size_t i = 0; i < hB.size(); ++i) hB[i] = static_cast<float>(mix(i + (1ull << 40)) >> 40) * (1.0f / 16777216.0f);
            std::vector<int> raw(static_cast<size_t>(W) * Q);
            for (int win = 0; win < K / 32; ++win)
                for (int q = 0; q < Q; ++q) {
                    int perm[32];
                    for (int i = 0; i < 32; ++i) perm[i] = i;
                    for (int i = 0; i < n_keep; ++i) {               // partial Fisher-Yates, then sort the kept ones
                        const int j = i + static_cast<int>(mix((static_cast<uint64_t>(win) * Q + q) * 64 + i + (2ull << 40)) % (32 - i));
                        std::swap(perm[i], perm[j]);
                    }
                    std::sort(perm, perm + n_keep);
                    for (int i = 0; i < n_keep; ++i) raw[(static_cast<size_t>(win) * n_keep + i) * Q + q] = perm[i];
                }
            float *dA, *dB, *dC;
            CK(cudaMalloc(&dA, hA.size() * 4));
            CK(cudaMalloc(&dB, hB.size() * 4));
            CK(cudaMalloc(&dC, static_cast<size_t>(M) * N * 4));
            CK(cudaMemcpy(dA, hA.data(), hA.size() * 4, cudaMemcpyHostToDevice));
            CK(cudaMemcpy(dB, hB.data(), hB.size() * 4, cudaMemcpyHostToDevice));
            double best = 0.0;
            const char* best_entry = "-";
            int best_split = 0;
            for (int layout : { 32, 64, 128 }) {
                if (N % layout != 0) continue;
                // pack the indices for this layout through the public preprocessing functions
                std::vector<int> D = raw;
                int pn = n_keep, pm = 32;
                std::vector<int> cinfo;
                if (high) {
                    transIndex(D.data(), W, N, Q, pn, pm);
                    cinfo.assign((static_cast<size_t>(W / pn) * (N / layout) + 1) * pm, -1);
                    PreProcessing_high_sparsity(cinfo.data(), pm, pn, D.data(), W, Q, N, layout);
                } else {
                    PreProcessing_low_sparsity(D.data(), W, Q, layout);
                }
                int *dD, *dCI = nullptr;
                CK(cudaMalloc(&dD, D.size() * 4));
                CK(cudaMemcpy(dD, D.data(), D.size() * 4, cudaMemcpyHostToDevice));
                if (high) {
                    CK(cudaMalloc(&dCI, cinfo.size() * 4));
                    CK(cudaMemcpy(dCI, cinfo.data(), cinfo.size() * 4, cudaMemcpyHostToDevice));
                }
                for (const Entry& en : entries) {
                    if (en.layout != layout || M % en.ms != 0 || N % en.ns != 0) continue;
                    if (table) printf("%d %d %d %s", M, N, K, en.name);
                    for (int split : { 1, 2, 4, 8 }) {
                        auto launch = [&]() {       // like the reference's own timing loop: C is not cleared between launches
                            if (high) en.high(dA, dB, dD, dCI, dC, M, N, K, W, sparsity, split);
                            else en.low(dA, dB, dD, dC, M, N, K, W, sparsity, split);
                        };
                        for (int i = 0; i < 2; ++i) launch();
                        CK(cudaDeviceSynchronize());
                        CK(cudaEventRecord(e0));
                        for (int i = 0; i < iters; ++i) launch();
                        CK(cudaEventRecord(e1));
                        CK(cudaEventSynchronize(e1));
                        float ms = 0.f;
                        CK(cudaEventElapsedTime(&ms, e0, e1));
                        const double tf = 2.0 * M * N * K / (ms / iters * 1e-3) / 1e12;
                        if (tf > best) { best = tf; best_entry = en.name; best_split = split; }
                        if (table) printf(" %.3f", tf);
                    }
                    if (table) printf("\n");
                }
                CK(cudaFree(dD));
                if (dCI) CK(cudaFree(dCI));
            }
            CK(cudaGetLastError());
            if (table) printf("%d %d %d best %.3f %s %d\n", M, N, K, best, best_entry, best_split);
            else printf("%d %d %d %.3f %s %d\n", M, N, K, best, best_entry, best_split);
            fflush(stdout);
            CK(cudaFree(dA));
            CK(cudaFree(dB));
            CK(cudaFree(dC));
        }
    }
    return 0;
}
