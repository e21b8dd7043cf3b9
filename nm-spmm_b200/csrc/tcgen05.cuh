// Thin wrappers over the sm_100a tensor-core instructions (tcgen05) and Tensor Memory.
#pragma once
#include <stdint.h>

namespace nmspmm {

// Tensor Memory addresses: lane in bits [31:16], 32-bit column in bits [15:0].
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col)
{
    return base + (static_cast<uint32_t>(lane) << 16) + static_cast<uint32_t>(col);
}

// Whole warp: allocates `cols` (power of two >= 32) TMEM columns; the base address is
// written to the shared-memory word at `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// The mbarrier gets one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Whole warp: each thread stores 8 consecutive 32-bit columns of its own lane
// (lane = 32 * (warp % 4) + laneid; the address names the warp's first lane).
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&v)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

// Whole warp: each thread loads 32 consecutive 32-bit columns of its own lane.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// Shared-memory descriptor of an MN-major TF32 operand: (n_blocks x 32) values along MN by 8
// rows along K.  MN-major 32-bit operands have one legal layout: 128-byte rows of 32 values
// whose 32-byte chunks are XOR-ed with (row % 4) -- layout type 1 of the descriptor, which is
// what a TMA copy with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B writes.  Its atom is 4 rows
// (512 bytes), so K = 8 spans two atoms `sbo_bytes` apart (512 when the k rows follow one
// another); blocks of 32 values along MN are `lbo_bytes` apart (not applied when MN = 32).
// The start address must be 512-byte aligned.  Addresses and strides are in 16-byte units;
// bits 46-47 = 1 is the descriptor version of sm_100.
__device__ __forceinline__ uint64_t umma_desc_mn_tf32(uint32_t smem_addr, uint32_t lbo_bytes = 512, uint32_t sbo_bytes = 512)
{
    uint64_t d = static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;   // leading byte offset: next 32 values along MN
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;   // stride byte offset: next 4 rows of K
    d |= 1ull << 46;
    d |= 1ull << 61;                                  // SWIZZLE_128B_BASE32B
    return d;
}

// Instruction descriptor of kind::tf32: FP32 accumulate, A and B TF32, B MN-major (n
// contiguous in shared memory), M x N tile.  A is K-major when it comes from Tensor Memory;
// a_mn_major = true for an A taken from shared memory with m contiguous.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n, bool a_mn_major = false)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | (a_mn_major ? (1u << 15) : 0u) | (1u << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// One thread: D[tmem] (+)= A[tmem] * B[smem], M x N x 8 TF32.
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}

// One thread: D[tmem] (+)= A[smem] * B[smem], M x N x 8 TF32.
__device__ __forceinline__ void umma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}

}  // namespace nmspmm
