/*
 * CPU restatement of the NM-SpMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the parity checker for the CUDA library: tests, the smoke check
 * and the benchmark's CPU-baseline leg call it; the shipped library never does.
 * It restates, in plain C, what the reference computes on the host:
 *
 *   oracle_trans_index      follows src/preprocessing.cu:3-15
 *   oracle_preprocess_high  follows src/preprocessing.cu:17-78
 *   oracle_preprocess_low   follows src/preprocessing.cu:80-100
 *   oracle_nm_gemm_f32      follows include/utils.h:82-95  (nmGEMM_on_cpu)
 *   oracle_nm_gemm_f64      same sum, accumulated in double (tolerance anchor
 *                           for the TF32 tensor-core path; no reference twin)
 *   oracle_nm_gemm_packed   same sum, but consuming the GPU-side operands
 *                           (row-major BT, re-tiled D, column_info) exactly as
 *                           the reference kernels index them
 *                           (src/kernel_64x128_8x8.cu:75-77,163-166,373,389)
 *
 * Parity is pinned: tests/test_oracle_golden.py checks every function against
 * fixtures produced by the reference's own code (tests/golden/make_golden.py)
 * and against the worked preprocessing example.
 *
 * Operand formats (include/utils.h:10-66 of the reference):
 *   A   col-major,  A[i + k*M]
 *   B   col-major compressed,  B[w + j*W]          (oracle side)
 *   BT  row-major compressed,  BT[w*N + j]         (GPU side)
 *   D   col-major, global k,   D[w + a*W], a = j/V (oracle side)
 *   DT  row-major, window-local k, DT[w*Q + a]     (GPU side, before packing)
 *   C   row-major,  C[i*N + j]
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_VEC_LEN 32

/* Merge pairs of 32-wide pruning windows into 64-wide ones: every odd window's
 * local indices move up by pruning_M.  The caller's N:M doubles. */
void oracle_trans_index(int* DT, int W, int N, int Q, int* pruning_N, int* pruning_M)
{
    const int pn = *pruning_N, pm = *pruning_M;
    (void)N;
    for (int a = 0; a < Q; ++a)
        for (int k = pn; k < W; k += 2 * pn)
            for (int u = 0; u < pn; ++u)
                DT[(size_t)(k + u) * Q + a] += pm;
    *pruning_M = pm * 2;
    *pruning_N = pn * 2;
}

/* [W][Q] -> [Q/Qs][W][Qs]; values untouched. */
static void retile(int* DT, int W, int Q, int Qs)
{
    int* buf = (int*)malloc(sizeof(int) * (size_t)W * Q);
    for (int j = 0; j < Q; j += Qs) {
        int* p = buf + (size_t)j * W;
        for (int row = 0; row < W; ++row)
            for (int col = 0; col < Qs; ++col)
                *p++ = DT[(size_t)row * Q + j + col];
    }
    memcpy(DT, buf, sizeof(int) * (size_t)W * Q);
    free(buf);
}

void oracle_preprocess_low(int* DT, int W, int Q, int Ns)
{
    retile(DT, W, Q, Ns / ORACLE_VEC_LEN);
}

/* For every (block of Qs vectors, window of pruning_N rows): list the used
 * local columns in ascending order (-1 padded to pruning_M), replace each index
 * by its rank in that list, then re-tile like the low path.  The extra
 * window the caller allocates past the last block is never written. */
void oracle_preprocess_high(int* column_info, int pruning_M, int pruning_N,
                            int* DT, int W, int Q, int N, int Ns)
{
    const int Qs = Ns / ORACLE_VEC_LEN;
    int* ci = column_info;
    int* used = (int*)malloc(sizeof(int) * pruning_M);
    int* rank = (int*)malloc(sizeof(int) * pruning_M);
    (void)N;
    for (int j = 0; j < Q; j += Qs) {
        for (int i = 0; i < W; i += pruning_N) {
            for (int x = 0; x < pruning_M; ++x) { ci[x] = -1; used[x] = 0; }
            for (int x = 0; x < pruning_N; ++x)
                for (int y = 0; y < Qs; ++y)
                    used[DT[(size_t)(i + x) * Q + j + y]] = 1;
            int n = 0;
            for (int x = 0; x < pruning_M; ++x)
                if (used[x]) { ci[n] = x; rank[x] = n; ++n; }
            for (int x = 0; x < pruning_N; ++x)
                for (int y = 0; y < Qs; ++y) {
                    int* e = &DT[(size_t)(i + x) * Q + j + y];
                    *e = rank[*e];
                }
            ci += pruning_M;
        }
    }
    free(used);
    free(rank);
    retile(DT, W, Q, Qs);
}

/* C += A*B over the compressed format, float accumulation in the reference's
 * order (k outer, j inner, one row of C at a time).  rows [i0, i1) only, so
 * that a bounded sample of a large problem can be timed. */
void oracle_nm_gemm_f32(const float* A, const float* B, const int* D, float* C,
                        int M, int N, int K, int W, int i0, int i1)
{
    (void)K;
#pragma omp parallel for schedule(static)
    for (int i = i0; i < i1; ++i)
        for (int k = 0; k < W; ++k)
            for (int j = 0; j < N; ++j) {
                int a = j / ORACLE_VEC_LEN;
                C[(size_t)i * N + j] += A[i + (size_t)D[k + (size_t)a * W] * M] * B[k + (size_t)j * W];
            }
}

/* Same sum with double products and double accumulation; C64 is overwritten. */
void oracle_nm_gemm_f64(const float* A, const float* B, const int* D, double* C64,
                        int M, int N, int K, int W, int i0, int i1)
{
    (void)K;
#pragma omp parallel for schedule(static)
    for (int i = i0; i < i1; ++i) {
        double* row = C64 + (size_t)i * N;
        for (int j = 0; j < N; ++j) row[j] = 0.0;
        for (int k = 0; k < W; ++k)
            for (int j = 0; j < N; ++j) {
                int a = j / ORACLE_VEC_LEN;
                row[j] += (double)A[i + (size_t)D[k + (size_t)a * W] * M] * (double)B[k + (size_t)j * W];
            }
    }
}

/* The product as the GPU kernels see their operands: BT row-major, D re-tiled to
 * [N/Ns][W][Qs].  Low path (column_info == NULL): windows of 32 k, ws = kept
 * rows per window, D holds the window-local k.  High path: windows of 64 k,
 * ws = kept rows per merged window, D holds a rank into
 * column_info[block][window][0..64).  C is overwritten. */
void oracle_nm_gemm_packed(const float* A, const float* BT, const int* D, const int* column_info,
                           float* C, int M, int N, int K, int W, int ws, int Ns)
{
    const int Qs = Ns / ORACLE_VEC_LEN;
    const int ks = column_info ? 64 : 32;
    const int nwin = W / ws;
    (void)K;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i) {
        float* row = C + (size_t)i * N;
        for (int j = 0; j < N; ++j) row[j] = 0.0f;
        for (int w = 0; w < W; ++w) {
            const int win = w / ws;
            for (int j = 0; j < N; ++j) {
                const int q = j / ORACLE_VEC_LEN, blk = q / Qs;
                int local = D[(size_t)blk * W * Qs + (size_t)w * Qs + q % Qs];
                if (column_info)
                    local = column_info[((size_t)blk * nwin + win) * ks + local];
                row[j] += A[i + ((size_t)win * ks + local) * M] * BT[(size_t)w * N + j];
            }
        }
    }
}

/* Threads the OpenMP loops above will use (1 when built without OpenMP). */
#ifdef _OPENMP
#include <omp.h>
int oracle_num_threads(void) { return omp_get_max_threads(); }
void oracle_set_num_threads(int n) { omp_set_num_threads(n); }
#else
int oracle_num_threads(void) { return 1; }
void oracle_set_num_threads(int n) { (void)n; }
#endif
