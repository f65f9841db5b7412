// Tile helpers for the tensor-core (bf16) pipeline.
//
// Every intermediate matrix X[rows x cols] of the bf16 pipeline is kept, in global memory and in
// shared memory alike, in one blocked layout called C8 here: 16-byte chunks of 8 consecutive
// column elements, chunk (r, cg) stored at chunk index cg*rows + r.  A C8 tile is contiguous
// (rows*cols*2 bytes), so it moves between global and shared memory with ONE bulk asynchronous
// copy, a column slice [c0, c1) of it is contiguous too, and -- the point of the layout -- the
// same bytes are a valid un-swizzled tcgen05 operand in both orientations:
//   contraction over the columns:  K-major,  k-group stride (LBO) = rows*16 B, row-group stride (SBO) = 128 B
//   contraction over the rows:     MN-major, k-group stride (LBO) = 128 B,     column-group stride (SBO) = rows*16 B
// so X and X^T are both usable without a transpose.  Accumulators come back from TMEM one row per
// thread (lane = row), and a thread turns 8 consecutive columns into one chunk, so a warp writes 32
// consecutive chunks (512 B): conflict-free in shared memory, coalesced in global memory.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace hdla {
namespace t8 {

struct Tile {
    uint32_t addr;     // shared-memory byte address
    uint32_t rows;
};

__device__ __forceinline__ Tile tile(const void* smem_ptr, uint32_t rows) { return Tile{sm100::smem_u32(smem_ptr), rows}; }

// contraction over columns starting at column k0 (multiple of 8); MN rows start at row0 (multiple of 8)
__device__ __forceinline__ uint64_t desc_k(Tile t, int k0, int row0) {
    return sm100::make_smem_desc(t.addr + (uint32_t)(k0 >> 3) * t.rows * 16u + (uint32_t)row0 * 16u, t.rows * 16u, 128u);
}
// contraction over rows starting at row k0 (multiple of 8); MN columns start at mn0 (multiple of 8)
__device__ __forceinline__ uint64_t desc_mn(Tile t, int k0, int mn0) {
    return sm100::make_smem_desc(t.addr + (uint32_t)(mn0 >> 3) * t.rows * 16u + (uint32_t)k0 * 16u, 128u, t.rows * 16u);
}

// D[128 x N] (+)= op(A) * op(B)^T over kdim (multiple of 16). One thread issues.
//   A_MN = false: A rows are tile rows (from a_mn0), contraction over tile columns (from a_k0)
//   A_MN = true : A rows are tile columns (from a_mn0), contraction over tile rows (from a_k0); same for B.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_chain(uint32_t tmem_d, Tile A, int a_k0, int a_mn0, Tile B, int b_k0, int b_mn0,
                                          int N, int kdim, bool accumulate) {
    const uint32_t idesc = sm100::make_idesc_bf16(128, N, A_MN ? 1 : 0, B_MN ? 1 : 0);
    for (int ks = 0; ks < kdim; ks += 16) {
        const uint64_t da = A_MN ? desc_mn(A, a_k0 + ks, a_mn0) : desc_k(A, a_k0 + ks, a_mn0);
        const uint64_t db = B_MN ? desc_mn(B, b_k0 + ks, b_mn0) : desc_k(B, b_k0 + ks, b_mn0);
        sm100::umma_bf16(tmem_d, da, db, idesc, (accumulate || ks > 0) ? 1u : 0u);
    }
}

__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 r;
    r.x = sm100::pack_bf16(f[0], f[1]); r.y = sm100::pack_bf16(f[2], f[3]);
    r.z = sm100::pack_bf16(f[4], f[5]); r.w = sm100::pack_bf16(f[6], f[7]);
    return r;
}
__device__ __forceinline__ void unpack8(uint4 c, float* f) {
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// TMEM address of (lane group of this warp, column col) relative to base
__device__ __forceinline__ uint32_t taddr(uint32_t base, int warp, int col) {
    return base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col;
}

}  // namespace t8

// 64 accumulator columns of this thread's row -> registers (two 32-column loads, one wait)
__device__ __forceinline__ void tmem_row64(uint32_t addr, float* f) {
    uint32_t a[32], b[32];
    sm100::tmem_ld_x32(addr, a);
    sm100::tmem_ld_x32(addr + 32, b);
    sm100::tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) { f[j] = __uint_as_float(a[j]); f[32 + j] = __uint_as_float(b[j]); }
}

}  // namespace hdla
