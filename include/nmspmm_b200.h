/*
 * nmspmm_b200 -- C-ABI of the sm_100a vector-wise N:M sparse GEMM library.
 *
 * C(M x N) = A(M x K) . B(K x N); B keeps `n_keep` rows out of every window of
 * 32 consecutive k, and 32 adjacent columns of B (one "vector") share the list
 * of kept rows.  Operand formats are the reference's (include/utils.h:10-66 of
 * M-H482/NM-SpMM):
 *
 *   A            col-major, A[i + k*M]                      float
 *   B            row-major compressed values, B[w*N + j]    float, W = K/32*n_keep rows
 *   DT           row-major [W][Q] window-local k (0..31)    int,   Q = N/32
 *   D            DT after packing: [N/Ns][W][Ns/32]         int
 *   column_info  high-sparsity path only: per (Ns block, 64-k window) the
 *                ascending list of used local columns, -1 padded to 64
 *   C            row-major, C[i*N + j]                      float
 *
 * Every function returns an nmspmm_status.  Pointers named *_dev are device
 * pointers, *_host are host pointers; all must be 16-byte aligned.  `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  Nothing here
 * allocates device memory except the functions that say so.
 *
 * The C++ entry points with the reference's exact names and signatures
 * (include/NM-SpMM.h of this repository) are thin wrappers over these.
 */
#ifndef NMSPMM_B200_H
#define NMSPMM_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nmspmm_status {
    NMSPMM_OK = 0,
    NMSPMM_INVALID_ARGUMENT = 1,   /* null / misaligned pointer, shape not divisible as required */
    NMSPMM_UNSUPPORTED = 2,        /* N:M ratio or layout outside the supported families */
    NMSPMM_CUDA_ERROR = 3,         /* a CUDA runtime call failed; see nmspmm_last_cuda_error() */
    NMSPMM_WORKSPACE_TOO_SMALL = 4,
    NMSPMM_DEVICE_TIMEOUT = 5      /* a bounded device-side wait gave up (status word set by the kernel) */
} nmspmm_status;

/* Arithmetic of the gathered mini-GEMM. */
typedef enum nmspmm_path {
    NMSPMM_PATH_FP32 = 0,          /* exact FP32 FFMA, register tiled */
    NMSPMM_PATH_TF32 = 1           /* TF32 products, FP32 accumulation: tcgen05 kind::tf32 with accumulators in TMEM;
                                      for M <= 64 warp-level mma.sync tiles of 16 / 32 / 64 rows */
} nmspmm_path;

/* Index format of D (selected in the reference by which entry point is called). */
typedef enum nmspmm_format {
    NMSPMM_FORMAT_LOW = 0,         /* D holds window-local k (window = 32); no column_info.
                                      Replaces PreProcessing_low_sparsity + *_low_sparsity launchers. */
    NMSPMM_FORMAT_HIGH = 1         /* D holds ranks into column_info (window = 64).
                                      Replaces transIndex + PreProcessing_high_sparsity + *_high_sparsity. */
} nmspmm_format;

const char* nmspmm_status_string(int status);
/* Last CUDA error code (cudaError_t as int) seen by this thread inside the library. */
int nmspmm_last_cuda_error(void);
/* Library version, 0xMMmmpp. */
int nmspmm_version(void);

/* ------------------------------------------------------------------ index packing
 * Device-pointer forms: one hand-written kernel each, bit-exact with the reference's
 * host loops.  They are out of place (DT_dev is read, D_dev is written; the two must
 * not overlap) so that the packing can be timed alone. */

/* Replaces transIndex (src/preprocessing.cu:3-15): rows of every odd 32-window get
 * +pruning_M, in place.  The caller doubles its own pruning_N / pruning_M afterwards. */
int nmspmm_trans_index_device(int* DT_dev, int W, int Q, int pruning_N, int pruning_M, void* stream);

/* Replaces PreProcessing_low_sparsity (src/preprocessing.cu:80-100): [W][Q] -> [Q/Qs][W][Qs]. */
int nmspmm_preprocess_low_device(const int* DT_dev, int* D_dev, int W, int Q, int Ns, void* stream);

/* Replaces PreProcessing_high_sparsity (src/preprocessing.cu:17-78).  DT_dev holds
 * merged-window indices (0..pruning_M-1, i.e. after trans_index); pruning_M <= 64.
 * Writes D_dev (ranks, re-tiled) and (N/Ns)*(W/pruning_N)*pruning_M ints of
 * column_info_dev.  With fuse_trans_index != 0, DT_dev holds the raw 0..31 indices,
 * pruning_N / pruning_M are the un-doubled values and the merge of window pairs is
 * done on the fly (DT_dev is not modified).  column_info_tail_ints further ints
 * after the last list are set to -1 (pass pruning_M for the reference driver's
 * extra window, 0 to leave them alone). */
int nmspmm_preprocess_high_device(const int* DT_dev, int* D_dev, int* column_info_dev,
                                  int pruning_M, int pruning_N, int W, int Q, int Ns,
                                  int fuse_trans_index, int column_info_tail_ints, void* stream);

/* Vector-wise N:M magnitude pruning of a dense weight on the GPU (no counterpart in the
 * reference, whose test driver draws random indices on the host, include/utils.h:46-64; this
 * produces the same formats from real weights without a round trip through the host).
 * dense_dev is row-major [K][N].  In every 32-row window and for every vector of vec_len (32
 * or 64) columns the n_keep rows with the largest sum of squares over the vector's columns are
 * kept (ties to the lower row), in ascending order: BT_dev [K/32*n_keep][N] receives their
 * values, DT_dev [K/32*n_keep][N/32] their window-local indices (one per 32 columns; with
 * vec_len 64 adjacent pairs are equal) -- the inputs of nmspmm_preprocess_*_device. */
int nmspmm_prune_device(const float* dense_dev, float* BT_dev, int* DT_dev,
                        int K, int N, int n_keep, int vec_len, void* stream);

/* Host-pointer forms with the reference's in-place semantics (H2D + kernel + D2H;
 * they allocate and free temporary device buffers).  The extra column_info window
 * is left untouched, like the reference. */
int nmspmm_trans_index_host(int* DT_host, int W, int N, int Q, int* pruning_N, int* pruning_M);
int nmspmm_preprocess_low_host(int* DT_host, int W, int Q, int Ns);
int nmspmm_preprocess_high_host(int* column_info_host, int pruning_M, int pruning_N,
                                int* DT_host, int W, int Q, int N, int Ns);

/* ------------------------------------------------------------------ the multiply */

/* CTA tiles compiled into the library (rows x columns of C).  The exact path has all of 1..7;
 * the TF32 path 128 x 128 and 128 x 256, the latter in two forms: the tensor core gathers the
 * kept rows of A (every format and ratio), or B is expanded with zeros and the A window is
 * multiplied whole (32-k formats with 16, 12 or 8 kept rows).  NMSPMM_TILE_128x256 leaves the
 * form to the library.  On the TF32 path ids 4 / 3 / 2 are streaming tiles of 16 / 32 / 64 rows on
 * warp-level MMA for M <= 16 / 32 / 64 (K in slices; 8:32 and 4:32 on the 64-k format, 16:32 and
 * 8:32 on the 32-k format), which the library takes by itself for such M. */
enum nmspmm_tile_id {
    NMSPMM_TILE_AUTO = 0,
    NMSPMM_TILE_128x128 = 1,
    NMSPMM_TILE_64x128 = 2,
    NMSPMM_TILE_32x128 = 3,
    NMSPMM_TILE_16x128 = 4,
    NMSPMM_TILE_128x256 = 5,
    NMSPMM_TILE_16x256 = 6,
    NMSPMM_TILE_32x256 = 7,
    NMSPMM_TILE_128x256_GATHER = 8,   /* TF32 path only */
    NMSPMM_TILE_128x256_EXPAND = 9    /* TF32 path only */
};

typedef struct nmspmm_gemm_desc {
    int M, N, K;
    int n_keep;        /* kept rows per 32-window: 32, 16, 12 (LOW) / 8, 4 (HIGH); LOW also takes 8 */
    int format;        /* nmspmm_format */
    int layout_ns;     /* Ns the index buffers were packed for: 32, 64 or 128 */
    int path;          /* nmspmm_path */
    int split_k;       /* >=1: that many K slices per tile; 0: the library balances k windows over the SMs */
    int tile;          /* 0: chosen by the library; otherwise one of enum nmspmm_tile_id: for testing and tuning */
    int vec_len;       /* 0 or 32: every 32 columns have their own index list (VEC_LEN of the reference,
                          include/NM-SpMM.h:8).  64: the caller promises that the lists of columns 64 v .. 64 v + 31
                          and 64 v + 32 .. 64 v + 63 are equal (a 64-wide vector stored in the reference's format as
                          two equal 32-wide ones; N % 64 == 0).  The TF32 path then gathers once per 64 columns
                          and reads only the even list; the FP32 path computes the same either way. */
} nmspmm_gemm_desc;

/* Bytes of scratch the multiply needs for this description (0 when every unit range is a
 * whole tile).  The scratch starts with a block of per-tile arrival counters,
 * NMSPMM_COUNTER_BYTES for every description of up to 16384 tiles, followed by slots for tile
 * pieces.  The counter block must be zero before the first use (cudaMemset once, e.g. of the
 * whole buffer); every multiply leaves it zero, and no multiply writes anything else there,
 * so one buffer can serve descriptions of different shapes, paths and splits one after the
 * other on a stream.  Two multiplies that overlap on the GPU need two buffers.  After
 * NMSPMM_DEVICE_TIMEOUT has been reported the library clears the block itself ahead of every
 * multiply (a CTA that gave up did not arrive at its counter). */
#define NMSPMM_COUNTER_BYTES (64u << 10)
size_t nmspmm_gemm_workspace_bytes(const nmspmm_gemm_desc* desc);

/* Replaces the eight nmGEMM_*_matrices_{low,high}_sparsity launchers
 * (src/kernel_*.cu).  C is overwritten with A.B for every split_k.  The pieces of a tile
 * are always summed in k order, so the result does not change from run to run: with up to
 * four pieces per tile the last piece to arrive adds them inside the multiply; with more
 * (deep K, few tiles) and for every split on the TF32 path the pieces stay in scratch and a
 * second, small kernel adds them on the same stream.  Asynchronous on `stream`: NMSPMM_OK
 * means the launch was queued.  A device-side bounded wait that gives up (see
 * nmspmm_device_status) is not reported here; poll nmspmm_device_status at a point where the
 * caller synchronises anyway.  column_info_dev is NULL for NMSPMM_FORMAT_LOW. */
int nmspmm_gemm(const nmspmm_gemm_desc* desc,
                const float* A_dev, const float* B_dev, const int* D_dev, const int* column_info_dev,
                float* C_dev, void* workspace_dev, size_t workspace_bytes, void* stream);

/* The multiply for activations stored row-major, A[i*K + k] (no counterpart in the reference,
 * whose A is col-major, include/utils.h:34-38; a linear layer's input is not).  A first kernel
 * on `stream` writes the col-major copy (its k rows padded to a multiple of 4 floats, so M
 * may be any positive number here) into the workspace, the multiply follows.
 * C is row-major M x N as everywhere.  The workspace holds what nmspmm_gemm needs (first, so
 * that the counter block keeps its place when the same workspace serves different M) and then
 * that copy: ask nmspmm_gemm_row_major_workspace_bytes. */
size_t nmspmm_gemm_row_major_workspace_bytes(const nmspmm_gemm_desc* desc);
int nmspmm_gemm_row_major(const nmspmm_gemm_desc* desc,
                          const float* A_rows_dev, const float* B_dev, const int* D_dev, const int* column_info_dev,
                          float* C_dev, void* workspace_dev, size_t workspace_bytes, void* stream);

/* The same with the activations and the result in 16-bit storage (IEEE half or bfloat16; no
 * counterpart in the reference, which is FP32 throughout, include/NM-SpMM.h:10-31).  x is
 * M x K row-major, y M x N row-major, both of `dtype`; B stays FP32 (weights kept in 16 bits
 * are widened once, nmspmm_widen_device, before they are compressed).  Every half and
 * bfloat16 value is a TF32 value, so on NMSPMM_PATH_TF32 the products of widened operands
 * are exact and only the FP32 sums and the final rounding of y (to nearest even) separate the
 * result from the real one; NMSPMM_PATH_FP32 is exact in the same sense.  One kernel widens
 * and transposes x, the multiply follows, one kernel rounds y; the workspace holds what the
 * multiply needs and the two FP32 copies. */
enum nmspmm_dtype { NMSPMM_DTYPE_F32 = 0, NMSPMM_DTYPE_F16 = 1, NMSPMM_DTYPE_BF16 = 2 };
size_t nmspmm_gemm_row_major_16_workspace_bytes(const nmspmm_gemm_desc* desc);
int nmspmm_gemm_row_major_16(const nmspmm_gemm_desc* desc, int dtype,
                             const void* x_rows_dev, const float* B_dev, const int* D_dev, const int* column_info_dev,
                             void* y_dev, void* workspace_dev, size_t workspace_bytes, void* stream);
/* n values (n % 4 == 0) of `dtype` at src_dev (8-byte aligned) -> FP32 at dst_dev (16-byte aligned). */
int nmspmm_widen_device(int dtype, const void* src_dev, float* dst_dev, size_t n, void* stream);

/* The multiply of one rank of a column-sharded B fused with the all-gather of C (no
 * counterpart in the reference, which runs on one GPU).  The rank's problem is
 * desc (N = the columns of its slab); every finished tile is stored, inside the multiply
 * kernel, into n_out (1..8) row-major buffers of row stride ldc floats at column offset col0:
 * the rank's own full-width C and the peer-mapped full-width C of every other rank (pointers
 * that this process may store through: CUDA IPC, VMM or symmetric-memory mappings; plain
 * st.global over NVLink, no multicast).  The stores ride along with the arithmetic instead
 * of following it as a collective.  The call orders nothing between ranks: the caller makes
 * sure every rank's C is free to be overwritten before the launch and that all ranks'
 * launches have completed before any C is read (two barriers).  ldc >= col0 + N; ldc and
 * col0 multiples of 4. */
int nmspmm_gemm_gather(const nmspmm_gemm_desc* desc,
                       const float* A_dev, const float* B_dev, const int* D_dev, const int* column_info_dev,
                       float* const* C_all, int n_out, long long ldc, int col0,
                       void* workspace_dev, size_t workspace_bytes, void* stream);

/* Same, with scratch that the library allocates on first use and keeps per host thread
 * (cudaMalloc inside the first call that needs it).  For callers bound to the
 * reference's launcher signatures, which carry no workspace argument. */
int nmspmm_gemm_with_cached_workspace(const nmspmm_gemm_desc* desc,
                                      const float* A_dev, const float* B_dev, const int* D_dev,
                                      const int* column_info_dev, float* C_dev, void* stream);

/* The multiply for callers that must not allocate.  (No counterpart in the reference:
 * its launchers need no scratch because they add split-K partials onto C with atomics.)
 *
 * Some hosts of this library cannot call cudaMalloc where the multiply runs: code that
 * executes inside another framework's allocator discipline, a latency-critical
 * section where an allocation would synchronise the device, or a process whose memory
 * budget was handed out in full at start-up.  For them the scratch that nmspmm_gemm
 * takes from the caller sits in a fixed array inside the library image:
 * NMSPMM_STATIC_SCRATCH_BYTES bytes of device memory on every GPU that loads the library,
 * held until the process exits.  The call is nmspmm_gemm with that array as workspace; it
 * calls no cudaMalloc, cudaFree or other allocating routine.
 *
 *  - With split_k = 0 the library first tries its automatic schedule; where that wants more
 *    than the array holds (it sizes its ranges for the machine: two slots per resident CTA)
 *    it falls back to the largest number of equal K slices per tile whose slots fit, down
 *    to whole tiles, which need no scratch.  The result is the same sum in a different
 *    order; it can be slower than nmspmm_gemm with caller scratch on skinny or deep-K shapes.
 *  - An explicit split_k whose slots exceed NMSPMM_STATIC_SCRATCH_BYTES is rejected with
 *    NMSPMM_WORKSPACE_TOO_SMALL and a message on stderr (nothing is launched).
 *  - The first call on a device looks the array's address up (cudaGetSymbolAddress, with
 *    that device current) and keeps it; make that first call before any stream capture.
 *  - Every call uses the same array and it keeps the previous call's contents.  The
 *    arrival counters at its head are cleared on `stream` ahead of the kernel; the slots
 *    are written before they are read.  Two calls that overlap on the GPU (different
 *    streams, or different host threads) race on it: serialise them. */
#define NMSPMM_STATIC_SCRATCH_BYTES (16u << 20)
int nmspmm_gemm_static_scratch(const nmspmm_gemm_desc* desc,
                               const float* A_dev, const float* B_dev, const int* D_dev,
                               const int* column_info_dev, float* C_dev, void* stream);

/* Reads the device status word that kernels raise when a bounded wait gives up
 * (synchronises the device).  Returns NMSPMM_OK or NMSPMM_DEVICE_TIMEOUT; the raw
 * word goes to *status_out when non-NULL; clear != 0 resets it. */
int nmspmm_device_status(int* status_out, int clear);

/* What the library resolved for a description (filled by nmspmm_gemm_plan). */
typedef struct nmspmm_gemm_plan_info {
    int tile;          /* nmspmm_tile_id */
    int tile_m, tile_n;
    int split_k;       /* explicit: K slices per tile; automatic: ranges per tile of the balanced tail, rounded up */
    int tiles_x, tiles_y;
    int n_virtual;     /* contiguous unit ranges the work is cut into (= CTAs launched) */
    int grid;          /* CTAs launched */
    int stream_k;      /* 1: automatic schedule (whole tiles + balanced tail); 0: explicit split */
    int n_dp;          /* automatic: leading tiles computed whole by one CTA each */
    int threads;
    int smem_bytes;
    int stages;
} nmspmm_gemm_plan_info;
int nmspmm_gemm_plan(const nmspmm_gemm_desc* desc, nmspmm_gemm_plan_info* out);

/* End-to-end form on HOST buffers: copies A, B, the raw DT [W][Q] and nothing else
 * to the device, packs the indices there, multiplies and copies C back.  Device
 * buffers are kept in a per-thread arena that grows on demand (this function
 * allocates).  Work is ordered after what `stream` holds at the call (NULL = a private
 * stream of the arena) and the function returns after all of it has drained.  From
 * M = 2048 up, A goes in and C comes out in row blocks on two copy streams of the arena
 * while other blocks are multiplied, so the transfers of both directions overlap the
 * arithmetic; the pageable-or-pinned state of the host buffers decides whether the
 * copies are truly asynchronous.  This is what a caller of the
 * reference's test driver does around its launcher (tests/test_nmspmm.cu:72-101). */
int nmspmm_gemm_host(const nmspmm_gemm_desc* desc,
                     const float* A_host, const float* B_host, const int* DT_host, float* C_host,
                     void* stream);
/* Frees the arena of nmspmm_gemm_host and the wrappers' cached scratch. */
int nmspmm_release_cached(void);

/* Sustained FP32 FMA rate of this GPU in TFLOP/s (2 flops per FMA), measured with a
 * register-only kernel on `stream` (synchronous; allocates 4 bytes).  packed = 0 uses
 * scalar FFMA, packed = 1 the two-lane packed FMA of sm_100.  The FP32 roofline
 * denominator is the larger of the two. */
int nmspmm_measure_ffma_peak(double* tflops_out, int packed, void* stream);

/* ------------------------------------------------------------------ tuned plans
 * The reference picks, per shape, the best of its four tilings x SPLIT_K in {1,2,4,8} by an
 * exhaustive sweep outside the library (benchmark/kernel_performance/run_test/nmspmm/
 * run_nmspmm.sh:16-38).  Here the result of such a sweep (nm-spmm_b200/tuner.py) lives in a
 * table the planner consults: a description with tile = 0 and split_k = 0 that matches an entry
 * on (M, N, K, n_keep, format, path, vec_len) gets the entry's tile and split_k (0 = the
 * library's automatic schedule on that tile) instead of the built-in heuristics.  The table
 * is read once per process from the text file named by the environment variable
 * NMSPMM_TUNED_PLANS (set but empty: none), else from tuned_plans.txt beside the library;
 * one entry per line, "M N K n_keep format path vec_len tile split_k", '#' starts a comment. */
int nmspmm_tuned_plan_set(const nmspmm_gemm_desc* key, int tile, int split_k);   /* add or replace one entry */
int nmspmm_tuned_plan_load(const char* path);                                    /* merge a file into the table */
int nmspmm_tuned_plan_clear(void);
int nmspmm_tuned_plan_count(void);

/* Tile order of the TF32 path's 128-row tiles (tuning and tests).  -1 (the default, or the value of the
 * environment variable NMSPMM_TILE_BAND when the library was loaded): the library walks the tiles in bands
 * of columns when the compressed B is too large to stay in L2 (8192 x 28672 x 8192, 8:32: DRAM reads of
 * one multiply 12.4 -> 4.0 GB, 4.49 -> 4.15 ms), row by row otherwise.  0: always row by row.  n > 0: bands of
 * n tile columns wherever there are more columns and at least two rows of tiles.  Returns the previous value. */
int nmspmm_set_tile_band(int band);

/* ------------------------------------------------------------------ testing
 * Makes the bounded device-side waits run out without faulting or hanging anything: while
 * enabled, the multiply's launchers encode the tensor map of B (of A for the TF32 form that
 * reads B with plain loads) with a box one row short, so every stage receives fewer bytes than
 * its mbarrier expects.  The kernels themselves are
 * unchanged: each wait gives up after about a second of SM clock, the CTA leaves through
 * its barriers without storing, C keeps its contents and nmspmm_device_status reports
 * NMSPMM_DEVICE_TIMEOUT.  Returns the previous setting.  Process-wide; for tests only (use a
 * problem of a few tiles: every CTA waits its second out). */
int nmspmm_test_short_fill(int enable);

#ifdef __cplusplus
}
#endif
#endif /* NMSPMM_B200_H */
