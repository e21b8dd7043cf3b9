// C-ABI of the library (include/nmspmm_b200.h): argument checks, plan selection
// (tile + split-K), scratch layout, and the host-buffer convenience forms.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <mutex>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string>
#include <unordered_map>
#include <vector>

#include "kernels.h"
#include "nmspmm_b200.h"

namespace nmspmm {

#define NMSPMM_VARIANT_TABLE(name)           \
    extern const FfmaVariant kFfma_##name[]; \
    extern const int kFfma_##name##_count;
NMSPMM_VARIANT_TABLE(low32)
NMSPMM_VARIANT_TABLE(low16)
NMSPMM_VARIANT_TABLE(low12)
NMSPMM_VARIANT_TABLE(low8)
NMSPMM_VARIANT_TABLE(high8)
NMSPMM_VARIANT_TABLE(high4)
NMSPMM_VARIANT_TABLE(low16p)
NMSPMM_VARIANT_TABLE(low12p)

const FfmaVariant* find_ffma_variant(int tile_id, int n_keep, int mode)
{
    struct Table { const FfmaVariant* v; int n; };
    const Table tables[] = { { kFfma_low32, kFfma_low32_count }, { kFfma_low16, kFfma_low16_count },
                             { kFfma_low12, kFfma_low12_count }, { kFfma_low8, kFfma_low8_count },
                             { kFfma_high8, kFfma_high8_count }, { kFfma_high4, kFfma_high4_count } };
    for (const Table& t : tables)
        for (int i = 0; i < t.n; ++i)
            if (t.v[i].tile_id == tile_id && t.v[i].n_keep == n_keep && t.v[i].mode == mode) return &t.v[i];
    return nullptr;
}

int g_test_short_fill = 0;

static thread_local int tl_last_cuda_error = 0;

static int cuda_fail(cudaError_t e)
{
    tl_last_cuda_error = static_cast<int>(e);
    return NMSPMM_CUDA_ERROR;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- per-device facts ---------------------------------------------------------
struct DeviceInfo {
    bool known = false;
    int sms = 0;
    int* status_word = nullptr;
};
static DeviceInfo g_dev[64];
static std::mutex g_dev_mutex;
__device__ int g_status_word;      // raised by kernels whose bounded waits gave up

static int device_info(DeviceInfo** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return NMSPMM_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.known) {
        e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e);
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status_word), g_status_word);
        if (e != cudaSuccess) return cuda_fail(e);
        e = cudaMemset(d.status_word, 0, sizeof(int));
        if (e != cudaSuccess) return cuda_fail(e);
        d.known = true;
    }
    *out = &d;
    return NMSPMM_OK;
}

// ---- plan -----------------------------------------------------------------------
struct Plan {
    const FfmaVariant* v = nullptr;
    const SlicedVariant* tv = nullptr;   // set instead of v on the tensor-core path and for the few-rows kernels of both paths
    int W = 0, ws = 0, n_win = 0;
    int tiles_x = 0, tiles_y = 0, n_tiles = 0;
    int band = 0;           // tile order: columns of tiles per band (gemm_args.h::tile_coords), 0 = row by row
    int split_k = 0;        // > 0 explicit slices per tile, 0 automatic
    int n_dp = 0;           // automatic: leading tiles computed whole
    int n_virtual = 0;      // unit ranges (= CTAs)
    int slots = 0;          // scratch slots for tile pieces
    int grid = 0;           // resident CTAs launched
    bool deferred = false;  // many pieces per tile: a second kernel adds them (else the last piece to arrive does)
    int first_split_tile = 0, n_split_tiles = 0;
    size_t counters_bytes = 0, partial_bytes = 0;
};

// The scratch of a split multiply starts with the per-tile arrival counters.  Their block has
// one size, NMSPMM_COUNTER_BYTES, for every plan of up to 16384 tiles (larger plans round up
// to a multiple of it), and every plan's slots start behind it, whether the plan uses the
// counters or not: whatever the shapes, paths and splits a buffer serves in turn, the block is
// only ever written by the arrival logic, which leaves it zero.
constexpr size_t kCounterBlock = NMSPMM_COUNTER_BYTES;
static size_t counter_block_bytes(long long n_tiles)
{
    const size_t need = static_cast<size_t>(n_tiles) * sizeof(unsigned);
    return need <= kCounterBlock ? kCounterBlock : (need + kCounterBlock - 1) / kCounterBlock * kCounterBlock;
}
// Set once a bounded wait has been seen to give up in this process: a CTA that left early
// did not arrive at its counter, so from then on every multiply clears the block itself.
static bool g_timeout_seen = false;

// Pieces per tile from which the reduction moves out of the multiply into its own
// kernel.  One CTA adding p pieces walks them one after the other (about 1.5 us per piece
// of a 128 x 128 tile); the kernel spreads that over the GPU for one launch (2-3 us).
constexpr int kDeferPieces = 4;

// any_rows: the caller's A is row-major and reaches the kernels through a padded transposed
// copy, so M need not be a multiple of 4 (the col-major A's k rows must start on 16 bytes).
static int check_desc(const nmspmm_gemm_desc* d, int* mode_out, bool any_rows = false)
{
    if (!d) return NMSPMM_INVALID_ARGUMENT;
    if (d->M <= 0 || d->N <= 0 || d->K <= 0) return NMSPMM_INVALID_ARGUMENT;
    if ((!any_rows && d->M % 4 != 0) || d->N % kVecLenHost != 0 || d->K % 32 != 0) return NMSPMM_INVALID_ARGUMENT;
    if (d->layout_ns != 32 && d->layout_ns != 64 && d->layout_ns != 128) return NMSPMM_INVALID_ARGUMENT;
    if (d->N % d->layout_ns != 0) return NMSPMM_INVALID_ARGUMENT;
    if (d->split_k < 0) return NMSPMM_INVALID_ARGUMENT;
    if (d->vec_len != 0 && d->vec_len != 32 && d->vec_len != 64) return NMSPMM_INVALID_ARGUMENT;
    if (d->vec_len == 64 && d->N % 64 != 0) return NMSPMM_INVALID_ARGUMENT;
    if (d->format == NMSPMM_FORMAT_LOW) {
        if (d->n_keep != 32 && d->n_keep != 16 && d->n_keep != 12 && d->n_keep != 8) return NMSPMM_UNSUPPORTED;
        *mode_out = kModeLow;
    } else if (d->format == NMSPMM_FORMAT_HIGH) {
        if (d->n_keep != 8 && d->n_keep != 4) return NMSPMM_UNSUPPORTED;
        if (d->K % 64 != 0) return NMSPMM_INVALID_ARGUMENT;
        *mode_out = kModeHigh;
    } else {
        return NMSPMM_INVALID_ARGUMENT;
    }
    return NMSPMM_OK;
}

static int pick_tile(const nmspmm_gemm_desc* d, int sms)
{
    (void)sms;
    if (d->M <= 16) return kTile16x128;
    if (d->M <= 32) return kTile32x128;
    if (d->M <= 64) return kTile64x128;
    const int pad128 = (d->M + 127) / 128 * 128, pad64 = (d->M + 63) / 64 * 64;
    return (pad64 < pad128) ? kTile64x128 : kTile128x128;
}

// ---- tuned plans ------------------------------------------------------------------
// (M, N, K, n_keep, format, path, vec_len) -> tile and split_k found by measurement
// (nm-spmm_b200/tuner.py).  A description that leaves both choices to the library
// (tile = 0, split_k = 0) takes a matching entry instead of the heuristics below.  The
// table is read once per process from the text file named by NMSPMM_TUNED_PLANS, else
// from tuned_plans.txt beside the library; nmspmm_tuned_plan_set adds entries at run time.
struct TunedPlan { int M, N, K, n_keep, format, path, vec_len, tile, split_k; };
static std::vector<TunedPlan> g_tuned;                     // the entries, and a hash index over them (shape -> position)
static std::unordered_multimap<uint64_t, int> g_tuned_index;
static uint64_t tuned_hash(int M, int N, int K, int n_keep, int format, int path, int vec_len)
{
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (uint64_t v : { static_cast<uint64_t>(M), static_cast<uint64_t>(N), static_cast<uint64_t>(K),
                        static_cast<uint64_t>(n_keep * 1024 + format * 256 + path * 128 + vec_len) })
        h = (h ^ v) * 0xBF58476D1CE4E5B9ull + (h >> 29);
    return h;
}
static std::mutex g_tuned_mutex;
static bool g_tuned_loaded = false;

static int vec_of(int v) { return v == 64 ? 64 : 32; }

static int tuned_find_locked(int M, int N, int K, int n_keep, int format, int path, int vec_len)
{
    auto range = g_tuned_index.equal_range(tuned_hash(M, N, K, n_keep, format, path, vec_len));
    for (auto it = range.first; it != range.second; ++it) {
        const TunedPlan& e = g_tuned[it->second];
        if (e.M == M && e.N == N && e.K == K && e.n_keep == n_keep && e.format == format && e.path == path && e.vec_len == vec_len)
            return it->second;
    }
    return -1;
}

static void tuned_set_locked(const TunedPlan& t)
{
    const int at = tuned_find_locked(t.M, t.N, t.K, t.n_keep, t.format, t.path, t.vec_len);
    if (at >= 0) {
        g_tuned[at] = t;
        return;
    }
    g_tuned_index.emplace(tuned_hash(t.M, t.N, t.K, t.n_keep, t.format, t.path, t.vec_len), static_cast<int>(g_tuned.size()));
    g_tuned.push_back(t);
}

static int tuned_load_file_locked(const char* path)
{
    FILE* f = fopen(path, "r");
    if (!f) return -1;
    char line[256];
    int n = 0;
    while (fgets(line, sizeof line, f)) {
        TunedPlan t;
        if (line[0] == '#') continue;
        if (sscanf(line, "%d %d %d %d %d %d %d %d %d", &t.M, &t.N, &t.K, &t.n_keep, &t.format, &t.path, &t.vec_len, &t.tile,
                   &t.split_k) == 9 && t.tile >= 0 && t.tile < kTileCount && t.split_k >= 0) {
            t.vec_len = vec_of(t.vec_len);
            tuned_set_locked(t);
            ++n;
        }
    }
    fclose(f);
    return n;
}

static void tuned_load_default_locked()
{
    if (g_tuned_loaded) return;
    g_tuned_loaded = true;
    if (const char* env = getenv("NMSPMM_TUNED_PLANS")) {
        if (env[0]) tuned_load_file_locked(env);
        return;                                            // set but empty: no table
    }
    Dl_info info;
    if (dladdr(reinterpret_cast<const void*>(&tuned_load_default_locked), &info) && info.dli_fname) {
        std::string dir(info.dli_fname);
        const size_t slash = dir.rfind('/');
        dir = (slash == std::string::npos) ? std::string(".") : dir.substr(0, slash);
        tuned_load_file_locked((dir + "/tuned_plans.txt").c_str());
    }
}

static bool tuned_lookup(const nmspmm_gemm_desc* d, int* tile, int* split_k)
{
    std::lock_guard<std::mutex> lock(g_tuned_mutex);
    tuned_load_default_locked();
    if (g_tuned.empty()) return false;
    const int at = tuned_find_locked(d->M, d->N, d->K, d->n_keep, d->format, d->path, vec_of(d->vec_len));
    if (at < 0) return false;
    *tile = g_tuned[at].tile;
    *split_k = g_tuned[at].split_k;
    return true;
}

static_assert(NMSPMM_TILE_128x128 == kTile128x128 && NMSPMM_TILE_64x128 == kTile64x128 && NMSPMM_TILE_32x128 == kTile32x128 &&
                  NMSPMM_TILE_16x128 == kTile16x128 && NMSPMM_TILE_128x256 == kTile128x256 && NMSPMM_TILE_16x256 == kTile16x256 &&
                  NMSPMM_TILE_32x256 == kTile32x256 && NMSPMM_TILE_128x256_GATHER == kTile128x256Gather &&
                  NMSPMM_TILE_128x256_EXPAND == kTile128x256Expand && NMSPMM_TILE_128x256_EXPAND + 1 == kTileCount,
              "the public tile ids are the library's");

// Whether the TF32 path should expand B rather than gather A when the caller leaves the choice
// to the library (32-k formats, tile 128 x 256).
static bool tf32_expand_pays(const nmspmm_gemm_desc* d)
{
    (void)d;
    return false;
}

static int g_tile_band = getenv("NMSPMM_TILE_BAND") ? atoi(getenv("NMSPMM_TILE_BAND")) : -1;   // see nmspmm_set_tile_band

// Band width of the tile order.  A compressed B that fits L2 comfortably stays there whatever
// the order.  A larger one (the large sharded configuration on one GPU: 235 MB against 126 MB of
// L2) would be streamed from HBM once per row of tiles; bands of about 32 MB of B are walked one
// after the other instead, each over all rows of tiles, and what is re-read per band is A.
// 8192 x 28672 x 8192 on the tensor-core path went from 4.49 to 4.15 ms.  The exact path is
// compute-bound on such shapes (B streams at under 1 TB/s); its 16:32 and unpruned kernels
// take the banded order too, the others, which were up to 10 % slower at 4096^3 with the band
// arithmetic in them, keep the plain order (gemm_ffma.cuh::tile_position).
static int tile_band(const nmspmm_gemm_desc* d, int W, int ns, int tiles_x, int tiles_y)
{
    const int forced = g_tile_band;                        // measurement / test knob: 0 = never, n = that width, -1 = the rule below
    if (forced >= 0) return (forced > 0 && forced < tiles_x && tiles_y >= 2) ? (forced > 127 ? 127 : forced) : 0;
    const double b_bytes = static_cast<double>(W) * d->N * sizeof(float);
    if (tiles_y < 2 || b_bytes <= 64e6) return 0;
    int band = static_cast<int>(32e6 / (static_cast<double>(W) * ns * sizeof(float)));
    if (band < 4) band = 4;
    if (band > 127) band = 127;
    return band < tiles_x ? band : 0;
}

// Rows of the few-rows tile that holds M rows (M <= 64).
static int few_rows_tile_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

// Plan of the few-rows kernels (gemm_tf32_few_rows.cu; `table` = their variants): one row of
// ms x 128 tiles, every tile cut into the same number of K slices, slices in scratch slots of
// ms x 128 floats.  NMSPMM_UNSUPPORTED when the ratio / format has no such variant, M does not
// fit the tile, or an explicit split leaves a slice more windows than a CTA's index list holds.
static int plan_few_rows(const nmspmm_gemm_desc* d, int mode, int sms, const SlicedVariant* table, int ms, Plan* p)
{
    const SlicedVariant* sv = nullptr;
    for (int i = 0; i < kFewRowsVariantCount; ++i)
        if (table[i].n_keep == d->n_keep && table[i].mode == mode && table[i].ms == ms) sv = &table[i];
    if (!sv || d->M > ms) return NMSPMM_UNSUPPORTED;
    const int W = d->K / 32 * d->n_keep;
    if (W % sv->ws != 0) return NMSPMM_UNSUPPORTED;
    const int n_win = W / sv->ws, n_tiles = (d->N + 127) / 128;
    const int least = (n_win + kFewRowsMaxWindows - 1) / kFewRowsMaxWindows;
    long long s = d->split_k;
    if (s <= 0) {
        // One wave, and about five CTAs per two SMs when more would fit: measured at
        // 16 x 11008 x 4096 (86 tiles), 8:32, TF32: 3 / 4 / 6 / 8 slices 19.4 / 15.4 / 16.5 / 17.8 us.
        const int per_sm = (227 * 1024) / (sv->smem_bytes + 1024) > 4 ? 4 : (227 * 1024) / (sv->smem_bytes + 1024);
        s = static_cast<long long>(sms) * per_sm / n_tiles;
        const long long want = (static_cast<long long>(sms) * 5 / 2 + n_tiles / 2) / n_tiles;
        if (s > want) s = want;
        if (s > n_win / 2) s = n_win / 2;                  // at least two windows per slice
        if (s < least) s = least;
    } else if (s < least) {
        return NMSPMM_UNSUPPORTED;
    }
    if (s > n_win) s = n_win;
    if (s < 1) s = 1;
    if (s * n_tiles >= (1LL << 30)) return NMSPMM_UNSUPPORTED;
    p->v = nullptr;
    p->tv = sv;
    p->ws = sv->ws;
    p->W = W;
    p->n_win = n_win;
    p->tiles_x = p->n_tiles = n_tiles;
    p->tiles_y = 1;
    p->split_k = static_cast<int>(s);
    p->n_dp = 0;
    p->n_virtual = p->grid = static_cast<int>(s * n_tiles);
    if (s > 1) {
        p->slots = p->grid;
        p->deferred = true;
        p->first_split_tile = 0;
        p->n_split_tiles = n_tiles;
        p->counters_bytes = counter_block_bytes(n_tiles);      // unused by these kernels; keeps the slots off the counter block
        p->partial_bytes = static_cast<size_t>(p->slots) * ms * 128 * sizeof(float);
    }
    return NMSPMM_OK;
}

// Whether the TF32 path should take the warp-level MMA tiles of 16 / 32 / 64 rows when the
// caller leaves the choice to the library.
static bool tf32_few_rows_pays(const nmspmm_gemm_desc* d)
{
    // 16 x 11008 x 4096, 8:32: 15.4 us against 30.4 us on the 128-row tensor-core tiles (and
    // 21.8 us on the exact path); 64 rows: 27.5 against 31.1 us.
    return d->M <= 64;
}

static int make_plan(const nmspmm_gemm_desc* d_in, int sms, Plan* p, bool any_rows = false)
{
    int mode = 0;
    int rc = check_desc(d_in, &mode, any_rows);
    if (rc != NMSPMM_OK) return rc;
    nmspmm_gemm_desc tuned = *d_in;
    const nmspmm_gemm_desc* d = d_in;
    if (d_in->tile == 0 && d_in->split_k == 0 && tuned_lookup(d_in, &tuned.tile, &tuned.split_k)) d = &tuned;
    if (sms <= 0) sms = 148;
    if (d->path == NMSPMM_PATH_TF32) {
        // Tensor-core path: one CTA per tile and K slice.  Tile 128 x 256 with one CTA per SM
        // wherever B is at least that wide: the gather instructions are twice as wide per
        // fetched window of A (measured at 4096^3, 16:32: 0.250 against 0.268 ms; on the
        // skinny and deep-K shapes, where K slices fill the SMs either way: 26.6 against 34.3 us
        // at 16 x 11008 x 4096, 60.4 against 65.8 us at 128 x 1024 x 131072); the caller's tile
        // wins over this.
        // Few rows of A (M <= 64): tiles of 16, 32 or 64 rows on warp-level MMA (gemm_tf32_few_rows.cu).
        const bool few_rows_tile = d->tile == kTile16x128 || d->tile == kTile32x128 || d->tile == kTile64x128;
        if (few_rows_tile || (d->tile == kTileAuto && tf32_few_rows_pays(d))) {
            const int ms = few_rows_tile ? (d->tile == kTile16x128 ? 16 : (d->tile == kTile32x128 ? 32 : 64)) : few_rows_tile_rows(d->M);
            const int rc_few = plan_few_rows(d, mode, sms, kTf32FewRowsVariants, ms, p);
            if (rc_few == NMSPMM_OK || few_rows_tile) return rc_few;
        }
        int want_ns = d->N >= 256 ? 256 : 128;
        if (d->tile == kTile128x256 || d->tile == kTile128x256Gather || d->tile == kTile128x256Expand) want_ns = 256;
        if (d->tile == kTile128x128) want_ns = 128;
        // Two forms on tile 128 x 256 (gemm_tf32.cu, gemm_tf32_expand.cu).  With B expanded the
        // tensor core issues 32 / n_keep times the useful work at its fastest instruction
        // shape; with A gathered, twice the useful work in small instructions.
        bool expand = (d->tile == kTile128x256Expand);
        if ((d->tile == kTileAuto || d->tile == kTile128x256) && want_ns == 256 && mode == kModeLow)
            expand = tf32_expand_pays(d);
        if (expand) {
            for (int i = 0; i < kTf32ExpandVariantCount; ++i)
                if (kTf32ExpandVariants[i].n_keep == d->n_keep && mode == kModeLow) p->tv = &kTf32ExpandVariants[i];
            if (!p->tv && d->tile == kTile128x256Expand) return NMSPMM_UNSUPPORTED;
        }
        // 64-wide vectors: the variants that gather once per 64 columns exist for tile 128 x 256
        if (d->vec_len == 64 && d->tile != kTile128x128 && !p->tv)
            for (int i = 0; i < kTf32GatherVariantCount; ++i)
                if (kTf32GatherVariants[i].n_keep == d->n_keep && kTf32GatherVariants[i].mode == mode && kTf32GatherVariants[i].vec_len == 64) {
                    p->tv = &kTf32GatherVariants[i];
                    want_ns = p->tv->ns;
                }
        for (int i = 0; i < kTf32GatherVariantCount && !p->tv; ++i)
            if (kTf32GatherVariants[i].n_keep == d->n_keep && kTf32GatherVariants[i].mode == mode && kTf32GatherVariants[i].vec_len == 32 &&
                kTf32GatherVariants[i].ns == want_ns)
                p->tv = &kTf32GatherVariants[i];
        if (!p->tv) return NMSPMM_UNSUPPORTED;
        p->ws = p->tv->ws;
        p->W = d->K / 32 * d->n_keep;
        if (p->W % p->ws != 0) return NMSPMM_UNSUPPORTED;
        p->n_win = p->W / p->ws;
        p->tiles_x = (d->N + p->tv->ns - 1) / p->tv->ns;
        p->tiles_y = (d->M + 127) / 128;
        const long long nt = static_cast<long long>(p->tiles_x) * p->tiles_y;
        if (nt >= (1LL << 26)) return NMSPMM_UNSUPPORTED;
        p->n_tiles = static_cast<int>(nt);
        p->band = tile_band(d, p->W, p->tv->ns, p->tiles_x, p->tiles_y);
        // K slices.  The caller's number applies to every tile.  Otherwise: tiles that fill
        // complete waves of resident CTAs run whole; the tiles of the partial last wave (all
        // tiles of a small problem) are cut into as many slices, of at least four windows,
        // as the free CTA slots allow -- with one CTA per SM a last wave that is 46 % full
        // (512 tiles on 148 SMs) otherwise costs as much as a full one.
        const int resident = sms * (want_ns == 256 ? 1 : 2);
        long long s = d->split_k, whole = 0;
        if (s <= 0) {
            whole = nt / resident * resident;
            const long long tail = nt - whole;
            s = tail > 0 ? resident / tail : 1;
            if (s > p->n_win / 4) s = p->n_win / 4;
            if (s > 16) s = (nt < resident) ? s : 16;
            // with two CTAs per SM a partial last wave is cheap (the lone CTA of an SM runs
            // faster) and slicing it measured 3 % slower: leave it whole
            if (want_ns == 128 && whole > 0) s = 1;
            if (s < 2) { s = 1; whole = nt; }
        }
        if (s > p->n_win) s = p->n_win;
        if (s < 1) s = 1;
        if (s == 1) whole = nt;
        const long long sliced_tiles = nt - whole;
        if (whole + sliced_tiles * s >= (1LL << 30)) return NMSPMM_UNSUPPORTED;
        p->split_k = static_cast<int>(s);
        p->n_dp = static_cast<int>(whole);
        p->n_virtual = p->grid = static_cast<int>(whole + sliced_tiles * s);
        if (sliced_tiles > 0) {
            p->slots = static_cast<int>(sliced_tiles * s);
            p->deferred = true;
            p->first_split_tile = p->n_dp;
            p->n_split_tiles = static_cast<int>(sliced_tiles);
            p->counters_bytes = counter_block_bytes(nt);      // unused by this path; keeps the slots off the counter block
            p->partial_bytes = static_cast<size_t>(p->slots) * 128 * want_ns * sizeof(float);
        }
        return NMSPMM_OK;
    }
    if (d->path != NMSPMM_PATH_FP32) return NMSPMM_UNSUPPORTED;
    const int tile = d->tile ? d->tile : pick_tile(d, sms);
    const FfmaVariant* v = find_ffma_variant(tile, d->n_keep, mode);
    if (!v) return NMSPMM_UNSUPPORTED;
    // 16:32 and 12:32 on the 128 x 128 tile: two 32-k windows per stage when K allows it
    // (half as many CTA barriers per k: 1.232 -> 1.190 ms at 4096^3, 16:32)
    if (mode == kModeLow && tile == kTile128x128 && d->K % 64 == 0 && d->K >= 512) {      // short K keeps the finer windows for splitting
        if (d->n_keep == 16 && kFfma_low16p_count > 0) v = &kFfma_low16p[0];
        if (d->n_keep == 12 && kFfma_low12p_count > 0) v = &kFfma_low12p[0];
    }
    p->v = v;
    p->ws = v->ws;
    const int ws = v->ws;
    p->W = d->K / 32 * d->n_keep;
    p->n_win = p->W / ws;
    p->tiles_x = (d->N + v->ns - 1) / v->ns;
    p->tiles_y = (d->M + v->ms - 1) / v->ms;
    const long long n_tiles = static_cast<long long>(p->tiles_x) * p->tiles_y;
    const long long units = n_tiles * p->n_win;
    if (units >= (1LL << 31) || n_tiles >= (1LL << 28)) return NMSPMM_UNSUPPORTED;
    p->n_tiles = static_cast<int>(n_tiles);
    if (mode == kModeLow && v->ws % 16 == 0)              // the variants compiled with the banded order (FfmaCfg::BANDED)
        p->band = tile_band(d, p->W, v->ns, p->tiles_x, p->tiles_y);
    const int resident = sms * v->min_blocks;
    if (d->split_k > 0) {
        // Explicit K slices: one unit range per (tile, slice); a single slice stores directly.
        int s = d->split_k < p->n_win ? d->split_k : p->n_win;
        if (n_tiles * s >= (1LL << 31)) return NMSPMM_UNSUPPORTED;
        p->split_k = s;
        p->n_virtual = static_cast<int>(n_tiles * s);
        p->slots = (s > 1) ? p->n_virtual : 0;
        p->deferred = s > kDeferPieces;
        p->first_split_tile = 0;
        p->n_split_tiles = p->n_tiles;
    } else {
        // Automatic: whole tiles for as many complete waves of resident CTAs as there are,
        // then the units of the remaining tiles in equal ranges, one per resident CTA, each
        // at least four windows long where the problem allows (never less than one).
        // (With two or more complete waves the whole-tile grid is used as it is: measured
        // on 4096^3, the partial last wave costs less than the split tiles' round trip
        // through scratch, because a CTA that has an SM to itself runs faster.)
        // Unless that last wave is nearly empty (under a quarter of the CTA slots): then its
        // few tiles would each hold an SM for a whole tile's time, and cutting them over all
        // the slots pays (8192 x 3584 x 8192, one rank's slab of eight: 1792 tiles = 6.05 waves).
        const long long full_waves = n_tiles / resident * resident;
        const bool sparse_tail = (n_tiles - full_waves) * 4 <= resident;
        const long long n_dp = (n_tiles >= 2LL * resident && !sparse_tail) ? n_tiles : full_waves;
        const long long tail_tiles = n_tiles - n_dp;
        long long n_sk = 0;
        if (tail_tiles > 0) {
            const long long tail_units = tail_tiles * p->n_win;
            n_sk = resident;
            const long long by_length = tail_units / 4 > tail_tiles ? tail_units / 4 : tail_tiles;
            if (n_sk > by_length) n_sk = by_length;
            if (n_sk > tail_units) n_sk = tail_units;
            if (n_sk < 1) n_sk = 1;
        }
        p->split_k = 0;
        p->n_dp = static_cast<int>(n_dp);
        p->n_virtual = static_cast<int>(n_dp + n_sk);
        // equal ranges that coincide with whole tiles need no scratch
        const bool aligned = (n_sk == 0) || (n_sk == tail_tiles);
        p->slots = aligned ? 0 : static_cast<int>(2 * n_sk);
        p->deferred = !aligned && n_sk > static_cast<long long>(kDeferPieces - 1) * tail_tiles;   // a tile sees up to n_sk / tail_tiles + 1 pieces
        p->first_split_tile = p->n_dp;
        p->n_split_tiles = static_cast<int>(tail_tiles);
    }
    p->grid = p->n_virtual;      // one unit range per CTA (the automatic schedule never exceeds the resident count)
    if (p->slots > 0) {
        p->counters_bytes = counter_block_bytes(p->n_tiles);
        p->partial_bytes = static_cast<size_t>(p->slots) * v->ms * v->ns * sizeof(float);
    }
    return NMSPMM_OK;
}

static int sm_count()
{
    DeviceInfo* di = nullptr;
    return device_info(&di) == NMSPMM_OK ? di->sms : 148;
}

// ---- cached scratch for the entry points whose signature has no workspace ---------
// One buffer per device and host thread: a thread that alternates between GPUs keeps each
// GPU's buffer (and never frees one device's memory with another device current).
struct Scratch {
    void* ptr = nullptr;
    size_t bytes = 0;
};
static thread_local Scratch tl_scratch[64];

static int scratch_reserve(size_t bytes, void** out, size_t* have)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return NMSPMM_UNSUPPORTED;
    Scratch& s = tl_scratch[dev];
    if (s.bytes < bytes) {
        if (s.ptr) {
            cudaDeviceSynchronize();                       // launches that still use the old buffer
            cudaFree(s.ptr);
            s.ptr = nullptr;
            s.bytes = 0;
        }
        size_t want = bytes < (size_t(8) << 20) ? (size_t(8) << 20) : bytes;
        e = cudaMalloc(&s.ptr, want);
        if (e != cudaSuccess) return cuda_fail(e);
        e = cudaMemset(s.ptr, 0, want);
        if (e != cudaSuccess) return cuda_fail(e);
        s.bytes = want;
    }
    *out = s.ptr;
    *have = s.bytes;
    return NMSPMM_OK;
}

// ---- arena of nmspmm_gemm_host ---------------------------------------------------
constexpr int kHostChunks = 8;       // at most this many row blocks of A / C are pipelined by nmspmm_gemm_host
struct Arena {
    void* ptr = nullptr;
    size_t bytes = 0;
    int device = -1;
    cudaStream_t stream = nullptr;          // compute (when the caller passes none)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr, in_done[kHostChunks] = {}, mm_done[kHostChunks] = {};
};
static thread_local Arena tl_arena[64];                   // per device, like the cached scratch

static int arena_reserve(size_t bytes, unsigned char** out, cudaStream_t* st, Arena** which)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return NMSPMM_UNSUPPORTED;
    Arena& a = tl_arena[dev];
    *which = &a;
    if (a.device != dev || a.bytes < bytes) {
        if (a.ptr) {
            cudaDeviceSynchronize();
            cudaFree(a.ptr);
            a.ptr = nullptr;
            a.bytes = 0;
        }
        e = cudaMalloc(&a.ptr, bytes);
        if (e != cudaSuccess) return cuda_fail(e);
        a.bytes = bytes;
        if (a.device != dev || !a.stream) {
            if ((e = cudaStreamCreateWithFlags(&a.stream, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e);
            if ((e = cudaStreamCreateWithFlags(&a.copy_in, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e);
            if ((e = cudaStreamCreateWithFlags(&a.copy_out, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e);
            if ((e = cudaEventCreateWithFlags(&a.fork, cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e);
            if ((e = cudaEventCreateWithFlags(&a.join, cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e);
            for (int i = 0; i < kHostChunks; ++i) {
                if ((e = cudaEventCreateWithFlags(&a.in_done[i], cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e);
                if ((e = cudaEventCreateWithFlags(&a.mm_done[i], cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e);
            }
        }
        a.device = dev;
    }
    *out = static_cast<unsigned char*>(a.ptr);
    *st = a.stream;
    return NMSPMM_OK;
}

static size_t round256(size_t b) { return (b + 255) / 256 * 256; }

}  // namespace nmspmm

using namespace nmspmm;

extern "C" {

const char* nmspmm_status_string(int status)
{
    switch (status) {
    case NMSPMM_OK: return "ok";
    case NMSPMM_INVALID_ARGUMENT: return "invalid argument";
    case NMSPMM_UNSUPPORTED: return "unsupported N:M ratio, layout or path";
    case NMSPMM_CUDA_ERROR: return "CUDA runtime error";
    case NMSPMM_WORKSPACE_TOO_SMALL: return "workspace too small";
    case NMSPMM_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    default: return "unknown status";
    }
}

int nmspmm_last_cuda_error(void) { return tl_last_cuda_error; }
int nmspmm_version(void) { return 0x000100; }

int nmspmm_trans_index_device(int* DT_dev, int W, int Q, int pruning_N, int pruning_M, void* stream)
{
    if (!DT_dev || W < 0 || Q <= 0 || pruning_N <= 0 || pruning_M <= 0) return NMSPMM_INVALID_ARGUMENT;
    if (W % (2 * pruning_N) != 0) return NMSPMM_INVALID_ARGUMENT;      // window pairs must be whole
    cudaError_t e = launch_trans_index(DT_dev, W, Q, pruning_N, pruning_M, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

int nmspmm_preprocess_low_device(const int* DT_dev, int* D_dev, int W, int Q, int Ns, void* stream)
{
    if (!DT_dev || !D_dev || W < 0 || Q <= 0) return NMSPMM_INVALID_ARGUMENT;
    if (Ns != 32 && Ns != 64 && Ns != 128) return NMSPMM_INVALID_ARGUMENT;
    const int Qs = Ns / kVecLenHost;
    if (Q % Qs != 0) return NMSPMM_INVALID_ARGUMENT;
    cudaError_t e = launch_retile(DT_dev, D_dev, W, Q, Qs, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

int nmspmm_preprocess_high_device(const int* DT_dev, int* D_dev, int* column_info_dev, int pruning_M, int pruning_N,
                                  int W, int Q, int Ns, int fuse_trans_index, int column_info_tail_ints, void* stream)
{
    if (!DT_dev || !D_dev || !column_info_dev || W < 0 || Q <= 0) return NMSPMM_INVALID_ARGUMENT;
    if (Ns != 32 && Ns != 64 && Ns != 128) return NMSPMM_INVALID_ARGUMENT;
    const int Qs = Ns / kVecLenHost;
    if (Q % Qs != 0 || column_info_tail_ints < 0) return NMSPMM_INVALID_ARGUMENT;
    int pm = pruning_M, pn = pruning_N;
    if (fuse_trans_index) {
        pm *= 2;
        pn *= 2;
    }
    if (pn <= 0 || pm <= 0 || pn > pm) return NMSPMM_INVALID_ARGUMENT;
    if (pm > 64) return NMSPMM_UNSUPPORTED;
    if (W % pn != 0) return NMSPMM_INVALID_ARGUMENT;
    cudaError_t e = launch_preprocess_high(DT_dev, D_dev, column_info_dev, pm, pn, W, Q, Qs, fuse_trans_index ? 1 : 0,
                                           column_info_tail_ints, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

// Host-pointer forms: device round trip with the reference's in-place semantics.
int nmspmm_trans_index_host(int* DT_host, int W, int N, int Q, int* pruning_N, int* pruning_M)
{
    (void)N;
    if (!DT_host || !pruning_N || !pruning_M) return NMSPMM_INVALID_ARGUMENT;
    const size_t bytes = static_cast<size_t>(W) * Q * sizeof(int);
    int* d = nullptr;
    cudaError_t e = cudaMalloc(&d, bytes ? bytes : 4);
    if (e != cudaSuccess) return cuda_fail(e);
    int rc = NMSPMM_OK;
    if ((e = cudaMemcpy(d, DT_host, bytes, cudaMemcpyHostToDevice)) != cudaSuccess) rc = cuda_fail(e);
    if (rc == NMSPMM_OK) rc = nmspmm_trans_index_device(d, W, Q, *pruning_N, *pruning_M, nullptr);
    if (rc == NMSPMM_OK && (e = cudaMemcpy(DT_host, d, bytes, cudaMemcpyDeviceToHost)) != cudaSuccess) rc = cuda_fail(e);
    cudaFree(d);
    if (rc == NMSPMM_OK) {
        *pruning_M *= 2;
        *pruning_N *= 2;
    }
    return rc;
}

int nmspmm_preprocess_low_host(int* DT_host, int W, int Q, int Ns)
{
    if (!DT_host) return NMSPMM_INVALID_ARGUMENT;
    const size_t bytes = static_cast<size_t>(W) * Q * sizeof(int);
    int* d = nullptr;
    cudaError_t e = cudaMalloc(&d, 2 * bytes + 4);
    if (e != cudaSuccess) return cuda_fail(e);
    int* out = d + static_cast<size_t>(W) * Q;
    int rc = NMSPMM_OK;
    if ((e = cudaMemcpy(d, DT_host, bytes, cudaMemcpyHostToDevice)) != cudaSuccess) rc = cuda_fail(e);
    if (rc == NMSPMM_OK) rc = nmspmm_preprocess_low_device(d, out, W, Q, Ns, nullptr);
    if (rc == NMSPMM_OK && (e = cudaMemcpy(DT_host, out, bytes, cudaMemcpyDeviceToHost)) != cudaSuccess) rc = cuda_fail(e);
    cudaFree(d);
    return rc;
}

int nmspmm_preprocess_high_host(int* column_info_host, int pruning_M, int pruning_N, int* DT_host, int W, int Q, int N,
                                int Ns)
{
    (void)N;
    if (!DT_host || !column_info_host || pruning_N <= 0 || Ns <= 0) return NMSPMM_INVALID_ARGUMENT;
    const size_t n_idx = static_cast<size_t>(W) * Q;
    const size_t n_ci = static_cast<size_t>(W / pruning_N) * (static_cast<size_t>(Q) * kVecLenHost / Ns) * pruning_M;
    int* d = nullptr;
    cudaError_t e = cudaMalloc(&d, (2 * n_idx + n_ci) * sizeof(int) + 4);
    if (e != cudaSuccess) return cuda_fail(e);
    int *out = d + n_idx, *ci = out + n_idx;
    int rc = NMSPMM_OK;
    if ((e = cudaMemcpy(d, DT_host, n_idx * sizeof(int), cudaMemcpyHostToDevice)) != cudaSuccess) rc = cuda_fail(e);
    if (rc == NMSPMM_OK) rc = nmspmm_preprocess_high_device(d, out, ci, pruning_M, pruning_N, W, Q, Ns, 0, 0, nullptr);
    if (rc == NMSPMM_OK && (e = cudaMemcpy(DT_host, out, n_idx * sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
        rc = cuda_fail(e);
    if (rc == NMSPMM_OK && (e = cudaMemcpy(column_info_host, ci, n_ci * sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess)
        rc = cuda_fail(e);
    cudaFree(d);
    return rc;
}

size_t nmspmm_gemm_workspace_bytes(const nmspmm_gemm_desc* desc)
{
    Plan p;
    if (make_plan(desc, sm_count(), &p) != NMSPMM_OK) return 0;
    return p.counters_bytes + p.partial_bytes;
}

int nmspmm_gemm_plan(const nmspmm_gemm_desc* desc, nmspmm_gemm_plan_info* out)
{
    if (!out) return NMSPMM_INVALID_ARGUMENT;
    Plan p;
    int rc = make_plan(desc, sm_count(), &p);
    if (rc != NMSPMM_OK) return rc;
    out->tile = p.v ? p.v->tile_id
                    : (p.tv->form == 2 ? (p.tv->ms == 16 ? kTile16x128 : (p.tv->ms == 32 ? kTile32x128 : kTile64x128))
                                       : (p.tv->ns == 128 ? kTile128x128 : (p.tv->form == 1 ? kTile128x256Expand : kTile128x256)));
    out->tile_m = p.v ? p.v->ms : (p.tv->ms ? p.tv->ms : 128);
    out->tile_n = p.v ? p.v->ns : p.tv->ns;
    out->split_k = p.split_k > 0 ? p.split_k
                                 : (p.n_tiles > p.n_dp ? (p.n_virtual - p.n_dp + p.n_tiles - p.n_dp - 1) / (p.n_tiles - p.n_dp) : 1);
    out->n_dp = p.n_dp;
    out->tiles_x = p.tiles_x;
    out->tiles_y = p.tiles_y;
    out->n_virtual = p.n_virtual;
    out->grid = p.grid;
    out->stream_k = p.split_k > 0 ? 0 : 1;
    out->threads = p.v ? p.v->threads : p.tv->threads;
    out->smem_bytes = p.v ? p.v->smem_bytes : p.tv->smem_bytes;
    out->stages = p.v ? p.v->stages : p.tv->stages;
    return NMSPMM_OK;
}

// The multiply with its outputs spelled out: n_out buffers, row stride ldc, first column col0.
static int gemm_launch(const nmspmm_gemm_desc* desc, const float* A_dev, const float* B_dev, const int* D_dev,
                       const int* column_info_dev, float* const* C_out, int n_out, long long ldc, int col0,
                       void* workspace_dev, size_t workspace_bytes, void* stream, int lda = 0)
{
    DeviceInfo* di = nullptr;
    int rc = device_info(&di);
    if (rc != NMSPMM_OK) return rc;
    Plan p;
    rc = make_plan(desc, di->sms, &p, lda != 0);
    if (rc != NMSPMM_OK) return rc;
    if (lda != 0 && (lda < desc->M || lda % 4 != 0)) return NMSPMM_INVALID_ARGUMENT;
    if (!A_dev || !B_dev || !D_dev || !C_out || n_out < 1 || n_out > kMaxOutputs) return NMSPMM_INVALID_ARGUMENT;
    if (desc->format == NMSPMM_FORMAT_HIGH && !column_info_dev) return NMSPMM_INVALID_ARGUMENT;
    if (!aligned16(A_dev) || !aligned16(B_dev) || !aligned16(D_dev)) return NMSPMM_INVALID_ARGUMENT;
    if (ldc < static_cast<long long>(col0) + desc->N || col0 < 0 || ldc % 4 != 0 || col0 % 4 != 0) return NMSPMM_INVALID_ARGUMENT;
    GemmArgs a {};
    a.A = A_dev;
    a.B = B_dev;
    a.D = D_dev;
    a.cinfo = column_info_dev;
    GemmOutputs outs {};
    for (int o = 0; o < n_out; ++o) {
        if (!C_out[o] || !aligned16(C_out[o])) return NMSPMM_INVALID_ARGUMENT;
        if (o == 0) a.C = C_out[o]; else outs.C_more[o - 1] = C_out[o];
    }
    outs.n_out = n_out;
    outs.ldc = ldc;
    outs.col0 = col0;
    outs.lda = lda;
    a.status = di->status_word;
    a.M = desc->M;
    a.N = desc->N;
    a.W = p.W;
    a.tiles_x = pack_tiles_x(p.tiles_x, p.band);
    a.sched.n_tiles = p.n_tiles;
    a.sched.n_win = p.n_win;
    a.sched.n_virtual = p.n_virtual;
    a.sched.split_k = p.split_k;
    a.sched.n_dp = p.n_dp;
    a.qs_shift = desc->layout_ns == 128 ? 2 : (desc->layout_ns == 64 ? 1 : 0);
    if (p.slots > 0) {
        if (!workspace_dev || !aligned16(workspace_dev)) return NMSPMM_INVALID_ARGUMENT;
        if (workspace_bytes < p.counters_bytes + p.partial_bytes) return NMSPMM_WORKSPACE_TOO_SMALL;
        a.counters = p.deferred ? nullptr : static_cast<unsigned*>(workspace_dev);
        a.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace_dev) + p.counters_bytes);
        if (a.counters && (p.counters_bytes > kCounterBlock || g_timeout_seen)) {
            // a block larger than the common one overlaps other plans' slots; and after a
            // timeout somewhere the counters can no longer be trusted to have been left zero
            cudaError_t me = cudaMemsetAsync(workspace_dev, 0, p.counters_bytes, static_cast<cudaStream_t>(stream));
            if (me != cudaSuccess) return cuda_fail(me);
        }
    }
    const bool plain = (n_out == 1 && ldc == desc->N && col0 == 0);
    cudaError_t e = p.v ? (plain ? p.v->launch : p.v->launch_multi)(a, outs, p.grid, static_cast<cudaStream_t>(stream))
                        : p.tv->launch(a, outs, p.grid, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess && p.v && p.slots > 0 && p.deferred)
        e = launch_reduce_pieces(p.v->tile_id, a, outs, p.first_split_tile, p.n_split_tiles, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess && p.tv && p.slots > 0)
        e = launch_reduce_slices(p.tv->ns, a, outs, p.first_split_tile, p.n_split_tiles, static_cast<cudaStream_t>(stream),
                                 p.tv->ms ? p.tv->ms : 128);
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

int nmspmm_gemm(const nmspmm_gemm_desc* desc, const float* A_dev, const float* B_dev, const int* D_dev,
                const int* column_info_dev, float* C_dev, void* workspace_dev, size_t workspace_bytes, void* stream)
{
    if (!desc) return NMSPMM_INVALID_ARGUMENT;
    float* out[1] = { C_dev };
    return gemm_launch(desc, A_dev, B_dev, D_dev, column_info_dev, out, 1, desc->N, 0, workspace_dev, workspace_bytes, stream);
}

// ---- A given row-major ----------------------------------------------------------------
static size_t row_major_copy_bytes(const nmspmm_gemm_desc* d)
{
    const size_t ld = (static_cast<size_t>(d->M) + 3) / 4 * 4;
    return round256(ld * static_cast<size_t>(d->K) * sizeof(float));
}

// The workspace of the row-major entries starts with what the multiply needs, so that the
// counter block has one place, and keeps its zeros, whatever M the workspace was last used
// with; a plan that needs nothing still leaves the block's bytes alone.  The copies follow.
static size_t row_major_head_bytes(const Plan& p)
{
    const size_t own = p.counters_bytes + p.partial_bytes;
    return own > 0 ? own : kCounterBlock;
}

size_t nmspmm_gemm_row_major_workspace_bytes(const nmspmm_gemm_desc* desc)
{
    Plan p;
    if (!desc || make_plan(desc, sm_count(), &p, true) != NMSPMM_OK) return 0;
    return row_major_head_bytes(p) + row_major_copy_bytes(desc);
}

int nmspmm_gemm_row_major(const nmspmm_gemm_desc* desc, const float* A_rows_dev, const float* B_dev, const int* D_dev,
                          const int* column_info_dev, float* C_dev, void* workspace_dev, size_t workspace_bytes, void* stream)
{
    if (!desc || !A_rows_dev || !workspace_dev || !aligned16(workspace_dev)) return NMSPMM_INVALID_ARGUMENT;
    Plan p;
    int rc = make_plan(desc, sm_count(), &p, true);
    if (rc != NMSPMM_OK) return rc;
    const size_t copy_bytes = row_major_copy_bytes(desc), own = p.counters_bytes + p.partial_bytes, head = row_major_head_bytes(p);
    if (workspace_bytes < head + copy_bytes) return NMSPMM_WORKSPACE_TOO_SMALL;
    const int ld = (desc->M + 3) / 4 * 4;
    float* A_cols = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace_dev) + head);
    cudaError_t e = launch_transpose_rows(A_rows_dev, A_cols, desc->M, desc->K, ld, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e);
    float* out[1] = { C_dev };
    return gemm_launch(desc, A_cols, B_dev, D_dev, column_info_dev, out, 1, desc->N, 0, own ? workspace_dev : nullptr, own, stream, ld);
}

// ---- activations and result in 16-bit storage ---------------------------------------------
static_assert(NMSPMM_DTYPE_F16 == kDtypeF16 && NMSPMM_DTYPE_BF16 == kDtypeBF16, "the public dtype ids are the library's");

static size_t result_copy_bytes(const nmspmm_gemm_desc* d)
{
    return round256(static_cast<size_t>(d->M) * d->N * sizeof(float));
}

size_t nmspmm_gemm_row_major_16_workspace_bytes(const nmspmm_gemm_desc* desc)
{
    Plan p;
    if (!desc || make_plan(desc, sm_count(), &p, true) != NMSPMM_OK) return 0;
    return row_major_head_bytes(p) + row_major_copy_bytes(desc) + result_copy_bytes(desc);
}

int nmspmm_gemm_row_major_16(const nmspmm_gemm_desc* desc, int dtype, const void* A_rows_dev, const float* B_dev, const int* D_dev,
                             const int* column_info_dev, void* C_dev, void* workspace_dev, size_t workspace_bytes, void* stream)
{
    if (!desc || !A_rows_dev || !C_dev || !workspace_dev || !aligned16(workspace_dev)) return NMSPMM_INVALID_ARGUMENT;
    if (dtype != NMSPMM_DTYPE_F16 && dtype != NMSPMM_DTYPE_BF16) return NMSPMM_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(C_dev) & 7u) != 0) return NMSPMM_INVALID_ARGUMENT;
    Plan p;
    int rc = make_plan(desc, sm_count(), &p, true);
    if (rc != NMSPMM_OK) return rc;
    const size_t copy_bytes = row_major_copy_bytes(desc), c_bytes = result_copy_bytes(desc);
    const size_t own = p.counters_bytes + p.partial_bytes, head = row_major_head_bytes(p);
    if (workspace_bytes < head + copy_bytes + c_bytes) return NMSPMM_WORKSPACE_TOO_SMALL;
    const int ld = (desc->M + 3) / 4 * 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned char* ws = static_cast<unsigned char*>(workspace_dev);
    float* A_cols = reinterpret_cast<float*>(ws + head);
    float* C32 = reinterpret_cast<float*>(ws + head + copy_bytes);
    cudaError_t e = launch_transpose_rows_16(dtype, A_rows_dev, A_cols, desc->M, desc->K, ld, st);
    if (e != cudaSuccess) return cuda_fail(e);
    float* out[1] = { C32 };
    rc = gemm_launch(desc, A_cols, B_dev, D_dev, column_info_dev, out, 1, desc->N, 0, own ? ws : nullptr, own, stream, ld);
    if (rc != NMSPMM_OK) return rc;
    e = launch_narrow(dtype, C32, C_dev, static_cast<size_t>(desc->M) * desc->N, st);
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

int nmspmm_widen_device(int dtype, const void* src_dev, float* dst_dev, size_t n, void* stream)
{
    if (!src_dev || !dst_dev || n % 4 != 0 || !aligned16(dst_dev) || (reinterpret_cast<uintptr_t>(src_dev) & 7u) != 0)
        return NMSPMM_INVALID_ARGUMENT;
    if (dtype != NMSPMM_DTYPE_F16 && dtype != NMSPMM_DTYPE_BF16) return NMSPMM_INVALID_ARGUMENT;
    cudaError_t e = launch_widen(dtype, src_dev, dst_dev, n, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

int nmspmm_gemm_gather(const nmspmm_gemm_desc* desc, const float* A_dev, const float* B_dev, const int* D_dev,
                       const int* column_info_dev, float* const* C_all, int n_out, long long ldc, int col0,
                       void* workspace_dev, size_t workspace_bytes, void* stream)
{
    return gemm_launch(desc, A_dev, B_dev, D_dev, column_info_dev, C_all, n_out, ldc, col0, workspace_dev, workspace_bytes, stream);
}

int nmspmm_device_status(int* status_out, int clear)
{
    DeviceInfo* di = nullptr;
    int rc = device_info(&di);
    if (rc != NMSPMM_OK) return rc;
    int word = 0;
    cudaError_t e = cudaMemcpy(&word, di->status_word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e);
    if (word != 0) g_timeout_seen = true;
    if (word != 0 && clear) {
        e = cudaMemset(di->status_word, 0, sizeof(int));
        if (e != cudaSuccess) return cuda_fail(e);
    }
    if (status_out) *status_out = word;
    return word == 0 ? NMSPMM_OK : NMSPMM_DEVICE_TIMEOUT;
}

int nmspmm_gemm_with_cached_workspace(const nmspmm_gemm_desc* desc, const float* A_dev, const float* B_dev,
                                      const int* D_dev, const int* column_info_dev, float* C_dev, void* stream)
{
    const size_t need = nmspmm_gemm_workspace_bytes(desc);
    void* ws = nullptr;
    size_t have = 0;
    if (need > 0) {
        int rc = scratch_reserve(need, &ws, &have);
        if (rc != NMSPMM_OK) return rc;
    }
    return nmspmm_gemm(desc, A_dev, B_dev, D_dev, column_info_dev, C_dev, ws, have, stream);
}

// ---- the entry point that allocates nothing --------------------------------------
// Scratch for split tiles lives in this file-scope device array: every GPU that loads the
// library carries these bytes until the process exits.  In host code the name below is
// only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[NMSPMM_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_ptr[64];      // per device, resolved on the first call there
static std::mutex g_static_scratch_mutex;

int nmspmm_gemm_static_scratch(const nmspmm_gemm_desc* desc, const float* A_dev, const float* B_dev, const int* D_dev,
                               const int* column_info_dev, float* C_dev, void* stream)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return NMSPMM_UNSUPPORTED;
    if (!desc) return NMSPMM_INVALID_ARGUMENT;
    nmspmm_gemm_desc d = *desc;
    size_t need = nmspmm_gemm_workspace_bytes(&d);
    if (need > static_cast<size_t>(NMSPMM_STATIC_SCRATCH_BYTES) && desc->split_k == 0) {
        // The automatic schedule sizes its ranges for the machine, not for this array (two
        // slots per resident CTA).  Fall back to the largest number of equal K slices per
        // tile whose slots fit; a single slice is a whole tile and needs no scratch at all.
        Plan p;
        DeviceInfo* di = nullptr;
        int rc = device_info(&di);
        if (rc != NMSPMM_OK) return rc;
        rc = make_plan(desc, di->sms, &p);
        if (rc != NMSPMM_OK) return rc;
        const size_t per_slot = p.slots > 0 ? p.partial_bytes / static_cast<size_t>(p.slots) : 0;
        long long s = per_slot ? static_cast<long long>(NMSPMM_STATIC_SCRATCH_BYTES / (per_slot * static_cast<size_t>(p.n_tiles))) : 1;
        if (s > p.n_win) s = p.n_win;
        for (; s >= 1; --s) {
            d.split_k = static_cast<int>(s);
            need = nmspmm_gemm_workspace_bytes(&d);
            if (need <= static_cast<size_t>(NMSPMM_STATIC_SCRATCH_BYTES)) break;
        }
        if (s < 1) d.split_k = 1, need = nmspmm_gemm_workspace_bytes(&d);
    }
    if (need > static_cast<size_t>(NMSPMM_STATIC_SCRATCH_BYTES)) {
        fprintf(stderr,
                "nmspmm_gemm_static_scratch: split_k = %d needs %zu bytes of scratch, the built-in array holds %zu; "
                "pass a smaller split_k (0 lets the library pick one that fits) or use nmspmm_gemm with caller scratch\n",
                desc->split_k, need, static_cast<size_t>(NMSPMM_STATIC_SCRATCH_BYTES));
        return NMSPMM_WORKSPACE_TOO_SMALL;
    }
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_ptr[dev]) {
            // once per device, with that device current: the array's address on this GPU
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess) return cuda_fail(e);
            g_static_scratch_ptr[dev] = p;
        }
        scratch = g_static_scratch_ptr[dev];
    }
    // (the arrival counters at the head of the scratch are cleared on the stream by the
    // multiply itself; the slots behind them are fully written before they are read)
    return nmspmm_gemm(&d, A_dev, B_dev, D_dev, column_info_dev, C_dev, need ? scratch : nullptr, need, stream);
}

int nmspmm_gemm_host(const nmspmm_gemm_desc* desc, const float* A_host, const float* B_host, const int* DT_host,
                     float* C_host, void* stream)
{
    if (!A_host || !B_host || !DT_host || !C_host) return NMSPMM_INVALID_ARGUMENT;
    DeviceInfo* di = nullptr;
    int rc = device_info(&di);
    if (rc != NMSPMM_OK) return rc;
    Plan p;
    rc = make_plan(desc, di->sms, &p);
    if (rc != NMSPMM_OK) return rc;
    const int M = desc->M, N = desc->N, K = desc->K, W = p.W, Q = N / kVecLenHost;
    const bool high = desc->format == NMSPMM_FORMAT_HIGH;
    const int pn_m = 2 * desc->n_keep, pm_m = 64;

    // Row blocks of A and C are pipelined: while block c is multiplied, block c+1 of A is on
    // its way in and block c-1 of C on its way out (the link is full duplex).  A is col-major,
    // so a row block is a strided 2-D copy that lands compact, [K][rows], on the device.
    int n_chunks = M / 1024;
    if (n_chunks > kHostChunks) n_chunks = kHostChunks;
    if (n_chunks < 1) n_chunks = 1;
    const int chunk_rows = (M / n_chunks + 127) / 128 * 128;
    n_chunks = (M + chunk_rows - 1) / chunk_rows;
    size_t ws_need = 0;
    for (int c = 0; c < n_chunks; ++c) {
        nmspmm_gemm_desc dc = *desc;
        dc.M = (c + 1 < n_chunks) ? chunk_rows : M - c * chunk_rows;
        Plan pc;
        rc = make_plan(&dc, di->sms, &pc);
        if (rc != NMSPMM_OK) return rc;
        if (pc.counters_bytes + pc.partial_bytes > ws_need) ws_need = pc.counters_bytes + pc.partial_bytes;
    }

    const size_t a_b = round256(sizeof(float) * M * static_cast<size_t>(K));
    const size_t b_b = round256(sizeof(float) * W * static_cast<size_t>(N));
    const size_t d_b = round256(sizeof(int) * W * static_cast<size_t>(Q));
    const size_t c_b = round256(sizeof(float) * M * static_cast<size_t>(N));
    const size_t ci_b = high ? round256(sizeof(int) * (static_cast<size_t>(W / pn_m) * (N / desc->layout_ns) + 1) * pm_m) : 0;
    const size_t ws_b = round256(ws_need);
    unsigned char* base = nullptr;
    cudaStream_t st = nullptr;
    Arena* arp = nullptr;
    rc = arena_reserve(a_b + b_b + 2 * d_b + c_b + ci_b + ws_b, &base, &st, &arp);
    if (rc != NMSPMM_OK) return rc;
    Arena& ar = *arp;
    if (stream) st = static_cast<cudaStream_t>(stream);
    float* dA = reinterpret_cast<float*>(base);
    float* dB = reinterpret_cast<float*>(base + a_b);
    int* dDT = reinterpret_cast<int*>(base + a_b + b_b);
    int* dD = reinterpret_cast<int*>(base + a_b + b_b + d_b);
    float* dC = reinterpret_cast<float*>(base + a_b + b_b + 2 * d_b);
    int* dCI = reinterpret_cast<int*>(base + a_b + b_b + 2 * d_b + c_b);
    unsigned char* dWS = base + a_b + b_b + 2 * d_b + c_b + ci_b;
    cudaError_t e;
#define NMSPMM_TRY(call) do { if ((e = (call)) != cudaSuccess) return cuda_fail(e); } while (0)
    // the copy streams start where the caller's stream is now
    NMSPMM_TRY(cudaEventRecord(ar.fork, st));
    NMSPMM_TRY(cudaStreamWaitEvent(ar.copy_in, ar.fork, 0));
    NMSPMM_TRY(cudaStreamWaitEvent(ar.copy_out, ar.fork, 0));
    // sparse operand first (it is needed by every block), then the blocks of A
    NMSPMM_TRY(cudaMemcpyAsync(dDT, DT_host, sizeof(int) * W * static_cast<size_t>(Q), cudaMemcpyHostToDevice, st));
    NMSPMM_TRY(cudaMemcpyAsync(dB, B_host, sizeof(float) * W * static_cast<size_t>(N), cudaMemcpyHostToDevice, st));
    for (int c = 0; c < n_chunks; ++c) {
        const int r0 = c * chunk_rows, rows = (c + 1 < n_chunks) ? chunk_rows : M - r0;
        float* dst = dA + static_cast<size_t>(r0) * K;            // blocks are stored one after the other
        NMSPMM_TRY(cudaMemcpy2DAsync(dst, sizeof(float) * rows, A_host + r0, sizeof(float) * M, sizeof(float) * rows, K,
                                     cudaMemcpyHostToDevice, ar.copy_in));
        NMSPMM_TRY(cudaEventRecord(ar.in_done[c], ar.copy_in));
    }
    if (high)
        rc = nmspmm_preprocess_high_device(dDT, dD, dCI, 32, desc->n_keep, W, Q, desc->layout_ns, 1, pm_m, st);
    else
        rc = nmspmm_preprocess_low_device(dDT, dD, W, Q, desc->layout_ns, st);
    if (rc != NMSPMM_OK) return rc;
    if (ws_b > 0) NMSPMM_TRY(cudaMemsetAsync(dWS, 0, kCounterBlock, st));   // the arena is carved anew per call: its counter block starts zero
    for (int c = 0; c < n_chunks; ++c) {
        const int r0 = c * chunk_rows, rows = (c + 1 < n_chunks) ? chunk_rows : M - r0;
        nmspmm_gemm_desc dc = *desc;
        dc.M = rows;
        NMSPMM_TRY(cudaStreamWaitEvent(st, ar.in_done[c], 0));
        rc = nmspmm_gemm(&dc, dA + static_cast<size_t>(r0) * K, dB, dD, high ? dCI : nullptr,
                         dC + static_cast<size_t>(r0) * N, ws_b ? dWS : nullptr, ws_b, st);
        if (rc != NMSPMM_OK) return rc;
        NMSPMM_TRY(cudaEventRecord(ar.mm_done[c], st));
        NMSPMM_TRY(cudaStreamWaitEvent(ar.copy_out, ar.mm_done[c], 0));
        NMSPMM_TRY(cudaMemcpyAsync(C_host + static_cast<size_t>(r0) * N, dC + static_cast<size_t>(r0) * N,
                                   sizeof(float) * rows * static_cast<size_t>(N), cudaMemcpyDeviceToHost, ar.copy_out));
    }
    NMSPMM_TRY(cudaEventRecord(ar.join, ar.copy_out));
    NMSPMM_TRY(cudaStreamWaitEvent(st, ar.join, 0));
    NMSPMM_TRY(cudaStreamSynchronize(st));
#undef NMSPMM_TRY
    return nmspmm_device_status(nullptr, 1);
}

int nmspmm_tuned_plan_set(const nmspmm_gemm_desc* key, int tile, int split_k)
{
    int mode = 0;
    if (check_desc(key, &mode, true) != NMSPMM_OK || tile < 0 || tile >= kTileCount || split_k < 0) return NMSPMM_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_tuned_mutex);
    tuned_load_default_locked();
    tuned_set_locked(TunedPlan { key->M, key->N, key->K, key->n_keep, key->format, key->path, vec_of(key->vec_len), tile, split_k });
    return NMSPMM_OK;
}

int nmspmm_tuned_plan_load(const char* path)
{
    if (!path) return NMSPMM_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_tuned_mutex);
    g_tuned_loaded = true;                                 // an explicit load replaces the default look-up
    return tuned_load_file_locked(path) >= 0 ? NMSPMM_OK : NMSPMM_INVALID_ARGUMENT;
}

int nmspmm_tuned_plan_clear(void)
{
    std::lock_guard<std::mutex> lock(g_tuned_mutex);
    g_tuned_loaded = true;
    g_tuned.clear();
    g_tuned_index.clear();
    return NMSPMM_OK;
}

int nmspmm_tuned_plan_count(void)
{
    std::lock_guard<std::mutex> lock(g_tuned_mutex);
    tuned_load_default_locked();
    return static_cast<int>(g_tuned.size());
}

int nmspmm_set_tile_band(int band)
{
    const int was = g_tile_band;
    g_tile_band = band;
    return was;
}

int nmspmm_test_short_fill(int enable)
{
    const int was = g_test_short_fill;
    g_test_short_fill = enable ? 1 : 0;
    return was;
}

int nmspmm_release_cached(void)
{
    // frees what the calling host thread holds on every device it used
    int current = 0;
    cudaGetDevice(&current);
    for (int dev = 0; dev < 64; ++dev) {
        Scratch& s = tl_scratch[dev];
        Arena& a = tl_arena[dev];
        if (!s.ptr && !a.ptr && !a.stream) continue;
        cudaSetDevice(dev);
        cudaDeviceSynchronize();
        if (s.ptr) cudaFree(s.ptr);
        s = Scratch();
        if (a.ptr) cudaFree(a.ptr);
        if (a.stream) {
            cudaStreamDestroy(a.stream);
            cudaStreamDestroy(a.copy_in);
            cudaStreamDestroy(a.copy_out);
            cudaEventDestroy(a.fork);
            cudaEventDestroy(a.join);
            for (int i = 0; i < kHostChunks; ++i) {
                cudaEventDestroy(a.in_done[i]);
                cudaEventDestroy(a.mm_done[i]);
            }
        }
        a = Arena();
    }
    cudaSetDevice(current);
    return NMSPMM_OK;
}

int nmspmm_measure_ffma_peak(double* tflops_out, int packed, void* stream)
{
    if (!tflops_out) return NMSPMM_INVALID_ARGUMENT;
    cudaError_t e = measure_ffma_peak(tflops_out, packed ? 1 : 0, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? NMSPMM_OK : cuda_fail(e);
}

}  // extern "C"
