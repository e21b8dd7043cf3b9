// C-ABI handles onto the UNMODIFIED reference sources, compiled where they lie
// (see oracle/Makefile: REF points at the reference checkout).  TEST
// INFRASTRUCTURE ONLY: used to pin oracle/nm_oracle.c, to generate the golden
// fixtures under tests/golden/, and as the timed CPU baseline ("reference"
// kind).  Nothing here is linked into the shipped library, and this file holds
// no reference code: it only includes the reference's headers and forwards.
#include "NM-SpMM.h"   // reference include/NM-SpMM.h (VEC_LEN + prototypes)
#include "utils.h"     // reference include/utils.h   (nmGEMM_on_cpu, allclose)

extern "C" {

void ref_trans_index(int* DT, int W, int N, int Q, int* pruning_N, int* pruning_M)
{
    transIndex(DT, W, N, Q, *pruning_N, *pruning_M);
}

void ref_preprocess_high(int* column_info, int pruning_M, int pruning_N, int* DT, int W, int Q, int N, int Ns)
{
    PreProcessing_high_sparsity(column_info, pruning_M, pruning_N, DT, W, Q, N, Ns);
}

void ref_preprocess_low(int* DT, int W, int Q, int Ns)
{
    PreProcessing_low_sparsity(DT, W, Q, Ns);
}

// C += A*B with the reference's host multiply (OpenMP over rows of A).
void ref_nm_gemm_cpu(float* A, float* B, int* D, float* C, int M, int N, int K, int W)
{
    nmGEMM_on_cpu(A, B, D, C, M, N, K, W);
}

int ref_allclose(float* a, float* b, int n) { return allclose(a, b, n) ? 1 : 0; }

int ref_num_threads(void) { return omp_get_max_threads(); }
void ref_set_num_threads(int n) { omp_set_num_threads(n); }

}  // extern "C"
