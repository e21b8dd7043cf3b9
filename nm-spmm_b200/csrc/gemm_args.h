// Kernel argument block of the multiply (plain data, usable from host code).
#pragma once

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
    kTileCount
};

struct GemmArgs {
    const float* A;
    const float* B;
    const int* D;
    const int* cinfo;
    float* C;
    float* partial;        // split-K scratch, [tile][slice][float4 e][thread]
    unsigned* counters;    // one per tile, zero between calls
    int* status;           // device status word (0 = ok)
    int M, N, W;
    int n_win;             // W / WS
    int split_k;
    int qs_l;              // vectors per packed index block (layout_ns / 32)
};

}  // namespace nmspmm
