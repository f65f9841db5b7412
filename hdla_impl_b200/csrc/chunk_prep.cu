// Forward chunk preparation of the bf16 tensor-core pipeline in ONE kernel per (chunk, head) tile:
//   cumulative log decay and hat operands       (fla chunk_rwkv6_fwd_cumsum, call site HRDPLR/hrdplr.py:44;
//                                                gating of HRDPLR/fwd_triton.py:222-245)
//   Aqk, Aqb, Aak, Aab                          (HRDPLR/fwd_triton.py:13-290 and :295-514)
//   M = (I - Aab)^-1                            (HRDPLR/fwd_triton.py:588-667; HRDPLR/naive.py:189-192)
//   P = Aak v, Wh = M Ah, u = M P               (HRDPLR/fwd_triton.py:674-790; HRDPLR/naive.py:195-196)
// The raw q, k, v, a, b, gk rows of the tile are read once from the public tensors; the hat operands
// are formed directly as C8 operand tiles in shared memory, the score matrices go from TMEM to shared
// memory, the inverse is computed in place, and only what later kernels read goes to global memory:
// Qh, Kh, Bh, Vc, Aqk, Aqb, Wh, u, E for the scan and the output, plus Ah, Aak, M, P and the
// un-gating factors when a backward pass will follow.  Aab and the cumulative sums never leave the SM.
//
// 112 KB of shared memory and 256 TMEM columns per CTA: two CTAs share an SM, so one tile's loads
// run under the other's products and epilogues.
//
// Thread mapping of the streaming part (128 threads): lane = (r8 = lane % 8, column group within
// the warp = lane / 8), warp w owns column groups 4w..4w+3 (a column group is 8 channels = one
// 16-byte chunk).  A thread handles rows r8, r8+8, ..., r8+56 of its column group, so a warp-wide
// load covers 8 rows x 64 contiguous bytes (whole sectors) and a quarter-warp writes 8 consecutive
// chunks of a C8 tile (conflict free).  The chunk-local cumulative sum of gk runs in registers: a
// segmented shuffle scan over the 8 lanes of a column group, then a serial prefix over the thread's
// eight row blocks.
#include "tc_plan.cuh"

namespace hdla {
namespace {

using namespace sm100;
using namespace tc;
using t8::Tile;

struct ChunkPrepP {
    const __nv_bfloat16 *q, *k, *v, *a, *b;
    const void* gk;
    uint4 *Qh, *Kh, *Ah, *Bh, *Vc, *Aqk, *Aqb, *Aak, *M, *W, *P, *U;
    float* E;
    __nv_bfloat16* ghat;                  // e^{gi - half} per (token, channel), bf16 row-major [64][128]
    float scale;
    int T, H, NT, gdt;
    int save_bwd;                         // also store Ah, Aak, M, P, ghat (read only by the backward kernels)
    int* status;
};

struct In6 { uint4 q, k, a0, a1, b0, b1; };

__device__ __forceinline__ In6 load6(const ChunkPrepP& p, int b, int h, int t0, int valid, int row, int cg) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    In6 x{zero, zero, zero, zero, zero, zero};
    if (row < valid) {
        const size_t src = (((size_t)b * p.T + t0 + row) * p.H + h) * K + cg * 8;
        const size_t sa0 = (((size_t)b * p.T * R + (size_t)(t0 + row) * R) * p.H + h) * K + cg * 8;
        const size_t sa1 = sa0 + (size_t)p.H * K;
        x.q = __ldg(reinterpret_cast<const uint4*>(p.q + src));
        x.k = __ldg(reinterpret_cast<const uint4*>(p.k + src));
        x.a0 = __ldg(reinterpret_cast<const uint4*>(p.a + sa0));
        x.a1 = __ldg(reinterpret_cast<const uint4*>(p.a + sa1));
        x.b0 = __ldg(reinterpret_cast<const uint4*>(p.b + sa0));
        x.b1 = __ldg(reinterpret_cast<const uint4*>(p.b + sa1));
    }
    return x;
}

__device__ __forceinline__ uint4 scaled8(uint4 raw, const float* f) {
    float x[8];
    t8::unpack8(raw, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= f[j];
    return t8::pack8(x);
}

__device__ __forceinline__ float c8_elem(const uint4* tile, int rows, int r, int c) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(tile + (c >> 3) * rows + r);
    return __bfloat162float(p[c & 7]);
}

constexpr int kPrepSmem = 16384 + 16384 + 32768 + 32768 + 16384;      // 112 KB

__global__ void __launch_bounds__(128, 2) chunk_prep_tc_kernel(ChunkPrepP p) {
    // (un-swizzled operand tiles and bulk copies need 16-byte alignment only; a small alignment keeps the static
    //  part of the allocation small enough for two CTAs per SM)
    extern __shared__ __align__(128) unsigned char smem[];
    uint4* sQ = reinterpret_cast<uint4*>(smem);      // 16 KB  Qh [64 x 128]   -> Aak [128 x 64]  -> P (with sK)
    uint4* sK = sQ + CH64;                           // 16 KB  Kh [64 x 128]                      -> P, second half
    uint4* sA = sK + CH64;                           // 32 KB  Ah [128 x 128]
    uint4* sD = sA + CH128;                          // 32 KB  Bh [128 x 128]  -> Aab -> M
    uint4* sV = sD + CH128;                          // 16 KB  v  [64 x 128]
    uint4* sP = sQ;
    __shared__ __align__(8) uint64_t mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
    const int b = bh / p.H, h = bh % p.H;
    const int t0 = n * C;
    const int valid = min(C, p.T - t0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r8 = lane & 7, cg = warp * 4 + (lane >> 3);
    const unsigned full = 0xffffffffu;
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    if (tid == 0) { mbar_init(&mma_bar, 1); fence_mbar_init(); }

    // ---- the operand pieces of the first four row blocks are requested before anything else: they do not
    //      depend on the decay sums, and four blocks in flight per thread keep the SM's share of HBM busy
    In6 in[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) in[j] = load6(p, b, h, t0, valid, 8 * j + r8, cg);

    // ---- chunk-local cumulative sum of gk (inclusive), in registers
    float gi[8][8];
    {
        const size_t rstride = (size_t)p.H * K;
        const size_t e0 = (((size_t)b * p.T + t0 + r8) * p.H + h) * K + cg * 8;
        if (p.gdt == HDLA_F32) {
            const float* src = static_cast<const float*>(p.gk) + e0;
            float4 lo[8], hi[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool ok = 8 * j + r8 < valid;
                lo[j] = ok ? __ldg(reinterpret_cast<const float4*>(src + (size_t)(8 * j) * rstride)) : make_float4(0.f, 0.f, 0.f, 0.f);
                hi[j] = ok ? __ldg(reinterpret_cast<const float4*>(src + (size_t)(8 * j) * rstride + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                gi[j][0] = lo[j].x; gi[j][1] = lo[j].y; gi[j][2] = lo[j].z; gi[j][3] = lo[j].w;
                gi[j][4] = hi[j].x; gi[j][5] = hi[j].y; gi[j][6] = hi[j].z; gi[j][7] = hi[j].w;
            }
        } else {
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.gk) + e0;
            uint4 raw[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                raw[j] = 8 * j + r8 < valid ? __ldg(reinterpret_cast<const uint4*>(src + (size_t)(8 * j) * rstride))
                                            : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) t8::unpack8(raw[j], gi[j]);
        }
    }
    float half[8];
    {
        float run[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) run[c] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float x = gi[j][c];
#pragma unroll
                for (int d = 1; d < 8; d <<= 1) {                 // inclusive scan over the 8 rows of the block
                    const float y = __shfl_up_sync(full, x, d, 8);
                    if (r8 >= d) x += y;
                }
                const float tot = __shfl_sync(full, x, 7, 8);      // sum of the block
                gi[j][c] = x + run[c];
                run[c] += tot;
            }
        }
        float worst = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            half[c] = 0.5f * run[c];
            const float m = fabsf(run[c]);
            worst = (m > worst || !(m == m)) ? m : worst;          // NaN propagates into worst
        }
        if (r8 == 0) {
            float4* e = reinterpret_cast<float4*>(p.E + (size_t)g * K + cg * 8);
            e[0] = make_float4(__expf(half[0]), __expf(half[1]), __expf(half[2]), __expf(half[3]));
            e[1] = make_float4(__expf(half[4]), __expf(half[5]), __expf(half[6]), __expf(half[7]));
            if (!(worst <= kMaxChunkDecay)) atomicExch(p.status + kStatusDecay, 1);        // also catches NaN
            if (worst == worst && __float_as_int(worst) > *reinterpret_cast<volatile int*>(p.status + kStatusMaxDecay))
                atomicMax(p.status + kStatusMaxDecay, __float_as_int(worst));
        }
    }

    // ---- hat operands, straight into the C8 operand tiles
    {
        float ep_prev[8];                                         // e^{gi - half} of this lane's row in the previous block
#pragma unroll
        for (int c = 0; c < 8; ++c) ep_prev[c] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const In6 cur = in[j & 3];
            if (j + 4 < 8) in[j & 3] = load6(p, b, h, t0, valid, 8 * (j + 4) + r8, cg);
            const int row = 8 * j + r8;
            float ep[8], em[8], ea[8], qs[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                ep[c] = __expf(gi[j][c] - half[c]);
                em[c] = __frcp_rn(ep[c]);
                qs[c] = ep[c] * p.scale;
                // e^{ge - half}: ge of a row is gi of the row before it (0 before the chunk's first row)
                const float up = __shfl_up_sync(full, ep[c], 1, 8);
                const float last = __shfl_sync(full, ep_prev[c], 7, 8);
                ea[c] = r8 > 0 ? up : (j > 0 ? last : __expf(-half[c]));
                ep_prev[c] = ep[c];
            }
            sQ[cg * 64 + row] = scaled8(cur.q, qs);
            sK[cg * 64 + row] = scaled8(cur.k, em);
            sA[cg * 128 + 2 * row] = scaled8(cur.a0, ea);
            sA[cg * 128 + 2 * row + 1] = scaled8(cur.a1, ea);
            sD[cg * 128 + 2 * row] = scaled8(cur.b0, em);
            sD[cg * 128 + 2 * row + 1] = scaled8(cur.b1, em);
            // the un-gating factors of the backward pass, e^{gi - half}, in bf16 (their error, 2^-9, is below
            // the rounding of the bf16 gradients they scale)
            if (p.save_bwd)
                *reinterpret_cast<uint4*>(p.ghat + (size_t)g * C * K + (size_t)row * K + cg * 8) = t8::pack8(ep);
        }
    }
    // v rows of the tile: requested now, stored to shared memory after the first products are issued
    uint4 vv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int row = 8 * j + r8;
        vv[j] = row < valid ? __ldg(reinterpret_cast<const uint4*>(p.v + (((size_t)b * p.T + t0 + row) * p.H + h) * V + cg * 8))
                            : make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const Tile tQ = t8::tile(sQ, 64), tK = t8::tile(sK, 64), tA = t8::tile(sA, 128), tB = t8::tile(sD, 128);
    uint32_t phase = 0;
    if (tid == 0) {
        // hat operands for the scan, the output and the backward kernels
        bulk_s2g(p.Qh + g * CH64, sQ, 16384);
        bulk_s2g(p.Kh + g * CH64, sK, 16384);
        bulk_s2g(p.Bh + g * CH128, sD, 32768);
        if (p.save_bwd) bulk_s2g(p.Ah + g * CH128, sA, 32768);
        bulk_commit();
        // [Aqk | Aqb] = Qh [Kh ; Bh]^T.  Qh has 64 rows: the upper 64 lanes of this M = 128 product read past the
        // tile (still inside this CTA's shared memory) and are never used.
        t8::mma_chain<false, false>(tmem, tQ, 0, 0, tK, 0, 0, 64, K, false);
        t8::mma_chain<false, false>(tmem + 64, tQ, 0, 0, tB, 0, 0, 128, K, false);
        umma_commit(&mma_bar);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sV[cg * 64 + 8 * j + r8] = vv[j];
    if (warp < 2) {
        wait_or_flag(&mma_bar, phase, p.status, 20);
        tc_fence_after();
        const int i = tid;
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, 0), f);              // Aqk: j <= i
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) if (!((c8 * 8 + j) <= i)) f[c8 * 8 + j] = 0.f;
            p.Aqk[g * 512 + c8 * 64 + i] = t8::pack8(f + c8 * 8);
        }
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {                      // Aqb: column token <= i
            tmem_row64(t8::taddr(tmem, warp, 64 + hh * 64), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) if (!(((hh * 64 + c8 * 8 + j) >> 1) <= i)) f[c8 * 8 + j] = 0.f;
                p.Aqb[g * CH64 + (hh * 8 + c8) * 64 + i] = t8::pack8(f + c8 * 8);
            }
        }
    }
    phase ^= 1;
    fence_proxy_async();                                       // v tile -> visible to the copy engine and the MMAs
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
        // [Aak | Aab] = Ah [Kh ; Bh]^T
        t8::mma_chain<false, false>(tmem, tA, 0, 0, tK, 0, 0, 64, K, false);
        t8::mma_chain<false, false>(tmem + 64, tA, 0, 0, tB, 0, 0, 128, K, false);
        umma_commit(&mma_bar);
        bulk_s2g(p.Vc + g * CH64, sV, 16384);
        bulk_commit();
        bulk_wait_read<1>();                                   // the hat tiles have been read: their slots may be reused
    }
    __syncthreads();
    wait_or_flag(&mma_bar, phase, p.status, 21);
    phase ^= 1;
    tc_fence_after();
    {   // Aak (strict mask) replaces Qh, Aab (strict mask in tokens) replaces Bh
        const int r = tid, i = r >> 1;
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, 0), f);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) if (!((c8 * 8 + j) < i)) f[c8 * 8 + j] = 0.f;
            sQ[c8 * 128 + r] = t8::pack8(f + c8 * 8);          // [128 x 64] tile: 8 column groups of 128 rows
        }
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
            tmem_row64(t8::taddr(tmem, warp, 64 + hh * 64), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) if (!(((hh * 64 + c8 * 8 + j) >> 1) < i)) f[c8 * 8 + j] = 0.f;
                sD[(hh * 8 + c8) * 128 + r] = t8::pack8(f + c8 * 8);
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0 && p.save_bwd) {
        bulk_s2g(p.Aak + g * CH64, sQ, 16384);
        bulk_commit();
    }

    // ---- M = (I - Aab)^-1 in place: 16 x 16 diagonal blocks by forward substitution in registers, then three
    //      doubling levels.  A block of L = Aab is read for the last time at the level that produces the block of
    //      M at the same place.  The X blocks of a level (at most 64 x 64 in all) live in the tile's upper right
    //      quadrant (rows 0..63, columns 64..127), which is zero in L and in M and which the products read only
    //      into accumulator rows that are never used; it is cleared again at the end.
    {   // diagonal 16x16 blocks: thread = (block, column)
        const int blk = tid >> 4, c = tid & 15, base = blk * 16;
        float mcol[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float s = (i == c) ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < i) s = fmaf(c8_elem(sD, 128, base + i, base + j), mcol[j], s);
            mcol[i] = s;
        }
        __syncthreads();                               // every column of a block is computed before the block is replaced
        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(sD);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int row = base + i, col = base + c;
            d[((size_t)(col >> 3) * 128 + row) * 8 + (col & 7)] = __float2bfloat16_rn(mcol[i]);
        }
    }
    fence_proxy_async();
    __syncthreads();
    // Doubling: with the diagonal blocks of size bs inverted, the block below the diagonal of every pair
    // (even block J, odd block I = J+1) is  M[I,J] = D[I,I] L[I,J] D[J,J].  Each product is restricted to the
    // pair's own column range (N = bs) and contraction range (K = bs); the accumulator rows outside block I
    // are computed but never read.  Pair pr uses accumulator columns [pr bs, (pr+1) bs).
    const Tile tD = t8::tile(sD, 128);
#pragma unroll 1
    for (int bs = 16; bs <= 64; bs <<= 1) {
        const int npair = 64 / bs;
        if (tid == 0) {
            tc_fence_after();
            for (int pr = 0; pr < npair; ++pr) {
                const int J = 2 * pr * bs;
                t8::mma_chain<false, true>(tmem + pr * bs, tD, J, 0, tD, J, J, bs, bs, false);     // X = L[:, J] D[J, J]
            }
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, phase, p.status, 22);
        phase ^= 1;
        tc_fence_after();
        const int blk = tid / bs, pr = blk >> 1;                // pr is uniform within a warp
        const bool odd = blk & 1;
        const int rr = tid - blk * bs;
        {
            uint4* xt = sD + (8 + ((pr * bs) >> 3)) * 128;      // rows 0..bs-1, columns 64 + pr bs .. of the tile
            for (int c8 = 0; c8 < (bs >> 3); ++c8) {
                uint32_t v[8]; float f[8];
                tmem_ld_x8(t8::taddr(tmem, warp, pr * bs + c8 * 8), v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
                if (odd) xt[c8 * 128 + rr] = t8::pack8(f);
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            for (int pr2 = 0; pr2 < npair; ++pr2) {
                const int I = (2 * pr2 + 1) * bs;
                t8::mma_chain<false, true>(tmem + pr2 * bs, tD, I, 0, tD, 0, 64 + pr2 * bs, bs, bs, false);   // Y = D[:, I] X
            }
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, phase, p.status, 23);
        phase ^= 1;
        tc_fence_after();
        {
            const int cg0 = (2 * pr * bs) >> 3;                 // first column group of block J in the full tile
            for (int c8 = 0; c8 < (bs >> 3); ++c8) {
                uint32_t v[8]; float f[8];
                tmem_ld_x8(t8::taddr(tmem, warp, pr * bs + c8 * 8), v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
                if (odd) sD[(cg0 + c8) * 128 + tid] = t8::pack8(f);
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
    }
    for (int e = tid; e < 512; e += 128) sD[(8 + (e >> 6)) * 128 + (e & 63)] = make_uint4(0, 0, 0, 0);    // the quadrant
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- P = Aak v, Wh = M Ah, then u = M P
    const Tile tAak = t8::tile(sQ, 128), tV = t8::tile(sV, 64), tP = t8::tile(sP, 128);
    if (tid == 0) {
        t8::mma_chain<false, true>(tmem, tAak, 0, 0, tV, 0, 0, 128, 64, false);          // P = Aak v
        t8::mma_chain<false, true>(tmem + 128, tD, 0, 0, tA, 0, 0, 128, 128, false);     // Wh = M Ah
        umma_commit(&mma_bar);
        if (p.save_bwd) {
            bulk_s2g(p.M + g * CH128, sD, 32768);
            bulk_commit();
            bulk_wait_read<1>();                               // Aak has been read: P may take its place
        }
    }
    __syncthreads();
    wait_or_flag(&mma_bar, phase, p.status, 24);
    phase ^= 1;
    tc_fence_after();
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) sP[(hh * 8 + c8) * 128 + tid] = t8::pack8(f + c8 * 8);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        t8::mma_chain<false, true>(tmem, tD, 0, 0, tP, 0, 0, 128, 128, false);           // u = M P
        umma_commit(&mma_bar);
        if (p.save_bwd) {
            bulk_s2g(p.P + g * CH128, sP, 32768);
            bulk_commit();
        }
    }
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {                                                      // Wh while u runs
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, 128 + hh * 64), f);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) p.W[g * CH128 + (hh * 8 + c8) * 128 + tid] = t8::pack8(f + c8 * 8);
    }
    wait_or_flag(&mma_bar, phase, p.status, 25);
    tc_fence_after();
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) p.U[g * CH128 + (hh * 8 + c8) * 128 + tid] = t8::pack8(f + c8 * 8);
    }
    if (tid == 0) bulk_wait_read<0>();                         // shared memory stays valid until the copies have read it
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

int tc_launch_chunk_prep(const TcPlan& pl, const HdlaDims& d, const void* q, const void* k, const void* v,
                         const void* a, const void* b, const void* gk, float scale, unsigned char* ws, bool save_bwd,
                         cudaStream_t st) {
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(chunk_prep_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem);
        if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_dev = dev;
    }
    auto U4 = [&](size_t off) { return reinterpret_cast<uint4*>(ws + off); };
    typedef const __nv_bfloat16* bp;
    ChunkPrepP pp{(bp)q, (bp)k, (bp)v, (bp)a, (bp)b, gk,
                  U4(pl.Qh), U4(pl.Kh), U4(pl.Ah), U4(pl.Bh), U4(pl.Vc), U4(pl.Aqk), U4(pl.Aqb), U4(pl.Aak), U4(pl.M),
                  U4(pl.W), U4(pl.P), U4(pl.U), reinterpret_cast<float*>(ws + pl.E),
                  reinterpret_cast<__nv_bfloat16*>(ws + pl.ghat), scale, d.T, d.H, pl.NT, d.gk_dtype, save_bwd ? 1 : 0,
                  reinterpret_cast<int*>(ws + pl.status)};
    chunk_prep_tc_kernel<<<(unsigned)pl.G, 128, kPrepSmem, st>>>(pp);
    HDLA_CHECK_LAUNCH("chunk_prep_tc_kernel");
    return HDLA_OK;
}

}  // namespace hdla
