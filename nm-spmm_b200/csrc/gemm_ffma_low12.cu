// FFMA multiply variants for 12 kept rows per 32-k window (kModeLow): 12 rows of B and
// 32 rows of A per staged window.
// The index hand-off by shuffle (the default) tips this variant's 128 x 128 and 128 x 256
// tiles over the 128-register budget (88 bytes of spills in the k loop); with every thread
// holding the window's twelve row offsets itself the compiler fits them (24 bytes).
#define NMSPMM_IDX_SHFL 0
#include "gemm_ffma.cuh"

namespace nmspmm {
extern const FfmaVariant kFfma_low12[] = { NMSPMM_FFMA_TILES(12, 12, 32, kModeLow) };
extern const int kFfma_low12_count = sizeof(kFfma_low12) / sizeof(kFfma_low12[0]);
}  // namespace nmspmm
