// Drop-in C++ interface: the eleven free functions of M-H482/NM-SpMM's public
// header (include/NM-SpMM.h:8-24 of the reference), same names, argument order and
// meaning, implemented by this repository's sm_100a library.  A program written
// against the reference header compiles and links against libnmspmm_b200.so
// unchanged (the reference's own test driver is built that way by oracle/Makefile).
//
// Differences a caller can observe, all deliberate:
//   * the three preprocessing functions still take HOST pointers and work in place,
//     but the packing itself runs on the GPU (bit-identical output);
//   * the launchers overwrite C with A.B for every SPLIT_K (the reference adds
//     split-K partials onto C with atomics, src/kernel_64x128_8x8.cu:235-242, so it
//     needs a zeroed C and is order-dependent); SPLIT_K <= 1 lets the library choose;
//   * a launcher whose SPLIT_K resolves above 1 allocates scratch once per host
//     thread (the reference signatures carry no workspace argument);
//   * the CTA tile is chosen by the library, the entry point only selects the index
//     layout (Ns = 128 / 64 / 64 / 32 for huge / large / medium / small);
//   * the arithmetic is exact FP32 unless the environment variable NMSPMM_PATH=tf32 is set
//     before the first launcher call: then the launchers use the TF32 tensor-core path
//     (about 2e-3 relative error instead of 1e-6; the signatures have no argument for it).
// The C-ABI underneath is include/nmspmm_b200.h.
#ifndef NMSpMM_H
#define NMSpMM_H

#include <cuda.h>
#include <cuda_runtime.h>
#include <iostream>

#define VEC_LEN (32)

// ---- index packing (host pointers, in place) --------------------------------------
// [W][Q] -> [Q/Qs][W][Qs], Qs = Ns / VEC_LEN.
void PreProcessing_low_sparsity(int* DT, int W, int Q, int Ns);
// Per (Ns block, window): ascending list of used columns into column_info (-1 padded),
// indices replaced by their rank in it, then the same re-tiling.
void PreProcessing_high_sparsity(int* column_info, int pruning_M, int pruning_N, int* DT, int W, int Q, int N, int Ns);
// Merges pairs of pruning windows; doubles the caller's pruning_N and pruning_M.
void transIndex(int* DT, int W, int N, int Q, int& pruning_N, int& pruning_M);

// ---- launchers (device pointers; asynchronous on the default stream) -----------------
// sparsity in {0, 0.5, 0.625} -> *_low_sparsity, {0.75, 0.875} -> *_high_sparsity.
// D (and column_info) must have been packed for the entry point's Ns.
void nmGEMM_huge_matrices_low_sparsity(float* A, float* B, int* D, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);
void nmGEMM_huge_matrices_high_sparsity(float* A, float* B, int* D, int* column_info, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);

void nmGEMM_large_matrices_low_sparsity(float* A, float* B, int* D, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);
void nmGEMM_large_matrices_high_sparsity(float* A, float* B, int* D, int* column_info, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);

void nmGEMM_medium_matrices_low_sparsity(float* A, float* B, int* D, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);
void nmGEMM_medium_matrices_high_sparsity(float* A, float* B, int* D, int* column_info, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);

void nmGEMM_small_matrices_low_sparsity(float* A, float* B, int* D, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);
void nmGEMM_small_matrices_high_sparsity(float* A, float* B, int* D, int* column_info, float* C, int M, int N, int K, int W, float sparsity, int SPLIT_K);

#endif  // NMSpMM_H
