// Kernel argument block of the multiply and the unit schedule shared by host and
// device (plain data and integer arithmetic, usable from host code).
#pragma once

#if defined(__CUDACC__)
#define NMSPMM_HD __host__ __device__ __forceinline__
#else
#define NMSPMM_HD inline
#endif

namespace nmspmm {

enum { kModeLow = 0, kModeHigh = 1 };
constexpr int kVecLenHost = 32;   // columns per vector (VEC_LEN of the reference API)

// CTA tiles compiled into the library (rows x columns of C).
enum nmspmm_tile {
    kTileAuto = 0,
    kTile128x128 = 1,
    kTile64x128 = 2,
    kTile32x128 = 3,
    kTile16x128 = 4,
    kTile128x256 = 5,
    kTile16x256 = 6,      // skinny activations: 1 KB of every B row per CTA, eight warps
    kTile32x256 = 7,
    kTile128x256Gather = 8,   // TF32 path only: tile 128 x 256, the form that gathers A with the tensor core
    kTile128x256Expand = 9,   // TF32 path only: tile 128 x 256, the form that expands B with zeros (32-k formats, 16 / 12 / 8 kept)
    kTileCount
};

// The unit schedule.  Units are numbered tile * n_win + window.
//   split_k > 0 : range v = K slice (v % split_k) of tile (v / split_k).
//   split_k == 0: the first n_dp ranges are the first n_dp tiles, whole (they run as
//                 ordinary full waves and keep neighbouring CTAs on neighbouring tiles
//                 and k windows, which is what the L2 likes); the units of the
//                 remaining tiles are cut into n_virtual - n_dp equal ranges that
//                 fill the last, partial wave evenly.
struct UnitSchedule {
    int n_tiles, n_win, n_virtual, split_k, n_dp;
};

constexpr int kMaxOutputs = 8;    // copies of C a launch can write (one per GPU of a box)

struct GemmArgs {
    const float* A;
    const float* B;
    const int* D;
    const int* cinfo;
    float* C;
    float* partial;        // scratch slots of tile pieces, [slot][float4 e][thread]
    unsigned* counters;    // one per tile, zero between calls; nullptr: pieces stay in scratch for the reduction kernel
    int* status;           // device status word (0 = ok)
    int M, N, W;
    int tiles_x;           // tiles per row of tiles, and the band width of the tile order (pack_tiles_x / tile_coords)
    UnitSchedule sched;    // n_tiles, n_win (k windows per tile, W / WS), ranges
    int qs_shift;          // log2 of the vectors per packed index block (layout_ns / 32): 0, 1 or 2
};

// Where finished tiles go when there is more than the private M x N matrix C: n_out row-major
// buffers (args.C, then C_more[0 .. n_out-2]) with row stride ldc, this problem's columns
// starting at column col0 of each.  A column-sharded rank that also gathers passes its own
// full-width C and every peer's (peer-mapped pointers; plain stores over NVLink).  A
// separate block, handed only to the kernels compiled for it: the plain kernels' register
// allocation is sensitive even to the size of their argument block.
struct GemmOutputs {
    float* C_more[kMaxOutputs - 1];
    int n_out;
    int col0;
    long long ldc;
    int lda;               // host side only (tensor-map encoding): floats between consecutive k rows of A; 0 = M
};
NMSPMM_HD float* output_of(const GemmArgs& a, const GemmOutputs& o, int i) { return i == 0 ? a.C : o.C_more[i - 1]; }

// Tile order.  GemmArgs::tiles_x carries the tiles per row of tiles in its low 24 bits and a band
// width in tiles above them.  Band width 0: tiles are numbered row by row.  Otherwise the columns
// of tiles are cut into bands of that many, the bands are walked one after the other and each
// band row by row: the CTAs resident at one time then share a band of B that stays in L2 (and a
// few row panels of A) instead of streaming all of B once per row of tiles.  The planner bands
// problems whose compressed B outgrows L2 (make_plan), except on those of the exact path's
// kernels that number their tiles row by row (gemm_ffma.cuh::tile_position).
constexpr int kTileBandShift = 24;
NMSPMM_HD int pack_tiles_x(int tiles_x, int band) { return tiles_x | (band << kTileBandShift); }
NMSPMM_HD void tile_coords(int tile, int tiles_x_packed, int tiles_y, int& ty, int& tx)
{
    const int tiles_x = tiles_x_packed & ((1 << kTileBandShift) - 1), band = tiles_x_packed >> kTileBandShift;
    if (band == 0) {
        ty = tile / tiles_x;
        tx = tile - ty * tiles_x;
        return;
    }
    const int per_band = band * tiles_y, b = tile / per_band, r = tile - b * per_band;
    const int x0 = b * band, w = (tiles_x - x0 < band) ? tiles_x - x0 : band;     // the last band may be narrower
    ty = r / w;
    tx = x0 + (r - ty * w);
}

// Which windows (of n_win) slice z of split_k owns: the first n_win % split_k
// slices get one extra window (the split of src/kernel_64x128_8x8.cu:21-37 of the
// reference, kept so that a given SPLIT_K covers the same k ranges).
NMSPMM_HD void slice_range(int n_win, int split_k, int z, int& first, int& count)
{
    const int base = n_win / split_k, rem = n_win % split_k;
    if (z < rem) {
        count = base + 1;
        first = z * (base + 1);
    } else {
        count = base;
        first = rem * (base + 1) + (z - rem) * base;
    }
}

// Units of virtual CTA v: [u0, u1).
NMSPMM_HD void virtual_range(const UnitSchedule& sc, int v, long long& u0, long long& u1)
{
    if (sc.split_k > 0) {
        int first, count;
        slice_range(sc.n_win, sc.split_k, v % sc.split_k, first, count);
        u0 = static_cast<long long>(v / sc.split_k) * sc.n_win + first;
        u1 = u0 + count;
    } else if (v < sc.n_dp) {
        u0 = static_cast<long long>(v) * sc.n_win;
        u1 = u0 + sc.n_win;
    } else {
        const long long base = static_cast<long long>(sc.n_dp) * sc.n_win;
        const long long total = static_cast<long long>(sc.n_tiles - sc.n_dp) * sc.n_win;
        const int n_sk = sc.n_virtual - sc.n_dp;
        u0 = base + (v - sc.n_dp) * total / n_sk;
        u1 = base + (v - sc.n_dp + 1) * total / n_sk;
    }
}

// First and last virtual CTA holding a piece of `tile` (consecutive; every one in
// between holds a piece too, provided the equal ranges are not more than the units).
NMSPMM_HD void tile_contributors(const UnitSchedule& sc, int tile, int& v_first, int& v_last)
{
    if (sc.split_k > 0) {
        v_first = tile * sc.split_k;
        v_last = v_first + sc.split_k - 1;
    } else if (tile < sc.n_dp) {
        v_first = v_last = tile;
    } else {
        const long long total = static_cast<long long>(sc.n_tiles - sc.n_dp) * sc.n_win;
        const int n_sk = sc.n_virtual - sc.n_dp;
        const long long x0 = static_cast<long long>(tile - sc.n_dp) * sc.n_win, x1 = x0 + sc.n_win - 1;
        v_first = sc.n_dp + static_cast<int>(((x0 + 1) * n_sk - 1) / total);
        v_last = sc.n_dp + static_cast<int>(((x1 + 1) * n_sk - 1) / total);
    }
}

// Scratch slot of the piece of `tile` held by range v.  Explicit split: one slot per
// range.  Automatic: two per equal range, the second for a tile that the range
// entered part-way through its own course (it started in an earlier tile).
NMSPMM_HD long long piece_slot(const UnitSchedule& sc, int v, int tile)
{
    if (sc.split_k > 0) return v;
    long long u0, u1;
    virtual_range(sc, v, u0, u1);
    return 2LL * (v - sc.n_dp) + ((u0 < static_cast<long long>(tile) * sc.n_win) ? 1 : 0);
}

}  // namespace nmspmm
