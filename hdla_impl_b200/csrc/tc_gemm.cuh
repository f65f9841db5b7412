// Batched small GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), one CTA per chunk.
//
//   C[M,N] (+)= alpha * A[M,L] * B[L,N]      M, N <= 128, L <= 128, bf16 operands, fp32 accumulate
//
// Both operands are read from global memory (fp32 or bf16, either index contiguous), rounded to
// bf16 and laid out in shared memory as 16-byte chunks in the un-swizzled canonical form the MMA
// descriptors describe: an operand whose contraction index is contiguous is staged "K-major"
// (chunk = 8 consecutive k of one row), one whose row index is contiguous "MN-major" (chunk = 8
// consecutive rows of one k), so no transpose is ever materialised.  One thread issues L/16
// tcgen05.mma instructions into a 128-lane TMEM accumulator, commits to an mbarrier, and the four
// warps read their 32 lanes back with tcgen05.ld for the masked / scaled / accumulating epilogue.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace hdla {

struct TcOperand {
    const void* p;
    long long sbh, sn;      // strides over (batch*head) and chunk, in elements
    long long rs, cs;       // logical row / column stride, in elements (one of them is 1)
    int dt;                 // HDLA_F32 | HDLA_BF16
};

struct TcGemmP {
    TcOperand A, B;         // A(i,l), B(l,j)
    void* C;
    long long cbh, cn, rsC, csC;
    int cdt;
    int M, N, L, NT;
    float alpha;
    int accumulate;
    int mask, ri, rj;       // as in the CUDA-core GEMM: 1 keep (i/ri) >= (j/rj), 2 keep (i/ri) > (j/rj)
    const float* col_scale; // optional per-column factor, [chunk][N] (batch stride N*NT / N)
    const float* row_scale; // optional per-row factor,   [chunk][M]
    int* status;            // device error word (set non-zero if a bounded wait ran out)
};

namespace tc {

constexpr int kRows = 128;                    // operand rows are always padded to 128
constexpr int kSmemOperand = 128 * 128 * 2;   // 32 KB per operand
constexpr uint32_t kLBO = 128 * 16;           // bytes between k-groups of 8
constexpr uint32_t kSBO = 128;                // bytes between row-groups of 8

__device__ __forceinline__ uint4 load_chunk8(const void* base, long long off, long long stride, int n_valid, int dt) {
    // 8 elements base[off + t*stride], t < n_valid, as packed bf16; the rest zero.
    float f[8];
    if (stride == 1 && n_valid == 8 && (off & 7) == 0) {
        if (dt == HDLA_F32) {
            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
            float4 x = p[0], y = p[1];
            f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w; f[4] = y.x; f[5] = y.y; f[6] = y.z; f[7] = y.w;
        } else {
            return *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + off);
        }
    } else {
#pragma unroll
        for (int t = 0; t < 8; ++t) f[t] = t < n_valid ? ld_elem(base, (size_t)(off + t * stride), dt) : 0.f;
    }
    uint4 r;
    r.x = sm100::pack_bf16(f[0], f[1]); r.y = sm100::pack_bf16(f[2], f[3]);
    r.z = sm100::pack_bf16(f[4], f[5]); r.w = sm100::pack_bf16(f[6], f[7]);
    return r;
}

// Stage a [rows x L] operand (element (r,l) at base[r*rs + l*cs]) into `dst`; returns 1 if MN-major.
__device__ __forceinline__ int stage_operand(uint4* dst, const void* base, long long rs, long long cs, int rows,
                                             int L, int Lp, int dt) {
    const int tid = threadIdx.x;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    if (cs == 1) {                                    // K-major: chunk (r, kc) at index kc*128 + r
        const int nchunks = kRows * (Lp / 8);
        for (int idx = tid; idx < nchunks; idx += blockDim.x) {
            const int r = idx & 127, kc = idx >> 7;
            uint4 v = zero;
            const int nv = min(8, L - kc * 8);
            if (r < rows && nv > 0) v = load_chunk8(base, r * rs + kc * 8, 1, nv, dt);
            dst[idx] = v;
        }
        return 0;
    }
    // MN-major: chunk (r8, l) at index ((l/8)*16 + r8)*8 + l%8
    const int nchunks = 16 * Lp;
    for (int idx = tid; idx < nchunks; idx += blockDim.x) {
        const int l8 = idx & 7, r8 = (idx >> 3) & 15, lg = idx >> 7;
        const int l = lg * 8 + l8;
        uint4 v = zero;
        const int nv = min(8, rows - r8 * 8);
        if (l < L && nv > 0) v = load_chunk8(base, (long long)l * cs + r8 * 8 * rs, rs, nv, dt);
        dst[idx] = v;
    }
    return 1;
}

}  // namespace tc
}  // namespace hdla
