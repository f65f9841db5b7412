// Tensor-core (tcgen05 / TMEM / bulk-copy) pipeline of the chunked HDLA operator for bf16 inputs,
// chunk 64, rank 2, K = V = 128.
//
// Scaled ("hat") operands.  With gi / ge the inclusive / exclusive chunk-local cumulative log
// decay and half = gi[last]/2 (per chunk and channel), E = exp(half):
//     Qh = scale q e^{gi-half}   Ah = a e^{ge-half}   Kh = k e^{half-gi}   Bh = b e^{half-gi}
// Every decay-weighted product of the algorithm factorises over them, e.g.
//     Aqk = tril(Qh Kh^T), Aab = stril(Ah Bh^T)           (HRDPLR/naive.py:136-184)
//     w = (M Ah) diag(E) =: Wh diag(E), kg = Kh diag(E), bg = Bh diag(E), qg = Qh diag(E)
// so with the row-scaled state St = E (.) S the chunk recurrence (HRDPLR/naive.py:232-255) reads
//     v2 = Wh St + u ;  o = Qh St + Aqk v + Aqb v2 ;  S' = E (.) (St + Kh^T v + Bh^T v2)
// and no product needs an operand scaled by more than e^{|g_last|/2}.
//
// All matrices between kernels are bf16 in the C8 blocked layout (tc_tiles.cuh) and move with
// bulk asynchronous copies; all products run on tcgen05.mma with fp32 accumulation in TMEM.
#include <cstring>

#include "tc_tiles.cuh"

namespace hdla {
namespace {

using namespace sm100;
using t8::Tile;

constexpr int C = 64, K = 128, V = 128, R = 2, m = 128;
constexpr int CH64 = 16 * 64;      // chunks (16 B) of a [64 x 128] tile
constexpr int CH128 = 16 * 128;    // chunks of a [128 x 128] tile

// ------------------------------------------------------------------------------------------
// workspace plan (byte offsets)
// ------------------------------------------------------------------------------------------
struct TcPlan {
    int B, T, H, NT, BH;
    long long G;
    size_t status, Qh, Kh, Ah, Bh, Vc, E, ghat, Aqk, Aqb, Aak, Aab, M, W, P, U, Hs, V2;
    size_t total_fwd, total;
};

TcPlan make_tc_plan(const HdlaDims& d) {
    TcPlan p{};
    p.B = d.B; p.T = d.T; p.H = d.H;
    p.NT = (d.T + C - 1) / C;
    p.BH = d.B * d.H;
    p.G = (long long)p.BH * p.NT;
    size_t off = 0;
    auto take = [&](size_t bytes_per_chunk) {
        size_t o = off;
        off += ((bytes_per_chunk * (size_t)p.G + 255) / 256) * 256;
        return o;
    };
    p.status = off; off += 256;
    p.Qh = take(16384); p.Kh = take(16384); p.Ah = take(32768); p.Bh = take(32768); p.Vc = take(16384);
    p.E = take(K * 4); p.ghat = take(C * K * 4);
    p.Aqk = take(8192); p.Aqb = take(16384); p.Aak = take(16384); p.Aab = take(32768); p.M = take(32768);
    p.W = take(32768); p.P = take(32768); p.U = take(32768); p.Hs = take(32768); p.V2 = take(32768);
    p.total_fwd = off;
    p.total = off;
    return p;
}

// bounded wait on an mbarrier; records a failure in the device status word and carries on
__device__ __forceinline__ void wait_or_flag(uint64_t* bar, uint32_t parity, int* status, int code) {
    if (!mbar_wait(bar, parity)) {
        if (status) atomicExch(status, code);
    }
}

// ------------------------------------------------------------------------------------------
// K1: cumulative decay and hat operands (CUDA cores, streaming)
//   gi = inclusive cumsum of gk within the chunk; ge = gi - gk (fla chunk_rwkv6_fwd_cumsum, call
//   site HRDPLR/hrdplr.py:44); gating as HRDPLR/fwd_triton.py:222-245 but around half = g_last/2.
// ------------------------------------------------------------------------------------------
struct PrepP {
    const __nv_bfloat16 *q, *k, *v, *a, *b;
    const void* gk;
    uint4 *Qh, *Kh, *Ah, *Bh, *Vc;
    float *E, *ghat;
    float scale;
    int T, H, NT, gdt;
};

__global__ void __launch_bounds__(128) prep_hat_kernel(PrepP p) {
    __shared__ float gis[C][K + 4];
    __shared__ float halfs[K];
    const long long g = blockIdx.x;
    const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
    const int b = bh / p.H, h = bh % p.H;
    const int t0 = n * C;
    const int valid = min(C, p.T - t0);
    const int tid = threadIdx.x;
    {
        float run = 0.f;
        for (int i = 0; i < C; ++i) {
            float gv = 0.f;
            if (i < valid) gv = ld_elem(p.gk, (((size_t)b * p.T + t0 + i) * p.H + h) * K + tid, p.gdt);
            run += gv;
            gis[i][tid] = run;
        }
        halfs[tid] = 0.5f * run;
        p.E[(size_t)g * K + tid] = __expf(0.5f * run);
    }
    __syncthreads();
    const int r = tid & 63;
    const bool rowok = r < valid;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int s = 0; s < 8; ++s) {
        const int kc = (tid >> 6) * 8 + s;
        float gi[8], ge[8], hf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            gi[j] = gis[r][kc * 8 + j];
            ge[j] = r > 0 ? gis[r - 1][kc * 8 + j] : 0.f;
            hf[j] = halfs[kc * 8 + j];
        }
        const size_t src = (((size_t)b * p.T + t0 + r) * p.H + h) * K + kc * 8;
        float x[8], y[8];
        t8::unpack8(rowok ? *reinterpret_cast<const uint4*>(p.q + src) : zero, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * p.scale * __expf(gi[j] - hf[j]);
        p.Qh[(size_t)g * CH64 + kc * 64 + r] = t8::pack8(y);
        t8::unpack8(rowok ? *reinterpret_cast<const uint4*>(p.k + src) : zero, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * __expf(hf[j] - gi[j]);
        p.Kh[(size_t)g * CH64 + kc * 64 + r] = t8::pack8(y);
        p.Vc[(size_t)g * CH64 + kc * 64 + r] =
            rowok ? *reinterpret_cast<const uint4*>(p.v + (((size_t)b * p.T + t0 + r) * p.H + h) * V + kc * 8) : zero;
#pragma unroll
        for (int rr = 0; rr < R; ++rr) {
            const size_t sa = (((size_t)b * p.T * R + (size_t)(t0 + r) * R + rr) * p.H + h) * K + kc * 8;
            t8::unpack8(rowok ? *reinterpret_cast<const uint4*>(p.a + sa) : zero, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[j] * __expf(ge[j] - hf[j]);
            p.Ah[(size_t)g * CH128 + kc * 128 + r * R + rr] = t8::pack8(y);
            t8::unpack8(rowok ? *reinterpret_cast<const uint4*>(p.b + sa) : zero, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[j] * __expf(hf[j] - gi[j]);
            p.Bh[(size_t)g * CH128 + kc * 128 + r * R + rr] = t8::pack8(y);
        }
        float4* gh = reinterpret_cast<float4*>(p.ghat + (size_t)g * C * K + (size_t)r * K + kc * 8);
        gh[0] = make_float4(gi[0] - hf[0], gi[1] - hf[1], gi[2] - hf[2], gi[3] - hf[3]);
        gh[1] = make_float4(gi[4] - hf[4], gi[5] - hf[5], gi[6] - hf[6], gi[7] - hf[7]);
    }
}

// ------------------------------------------------------------------------------------------
// K2: the four intra-chunk score matrices on tensor cores
//   [Aak | Aab] = Ah [Kh ; Bh]^T (strict mask), [Aqk | Aqb] = Qh [Kh ; Bh]^T (inclusive mask)
//   (HRDPLR/fwd_triton.py:13-290 and :295-514 computed these per 16x16 sub-block)
// ------------------------------------------------------------------------------------------
struct GramP {
    const uint4 *Qh, *Kh, *Ah, *Bh;
    uint4 *Aqk, *Aqb, *Aak, *Aab;
    int* status;
};

__global__ void __launch_bounds__(128) gram_tc_kernel(GramP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sQ = reinterpret_cast<uint4*>(smem);                  // [64 x 128]  16 KB
    uint4* sK = sQ + CH64;                                       // [64 x 128]  16 KB
    uint4* sA = sK + CH64;                                       // [128 x 128] 32 KB
    uint4* sB = sA + CH128;                                      // [128 x 128] 32 KB
    __shared__ __align__(8) uint64_t ld_bar, mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 98304);
        bulk_g2s(sQ, p.Qh + g * CH64, 16384, &ld_bar);
        bulk_g2s(sK, p.Kh + g * CH64, 16384, &ld_bar);
        bulk_g2s(sA, p.Ah + g * CH128, 32768, &ld_bar);
        bulk_g2s(sB, p.Bh + g * CH128, 32768, &ld_bar);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const Tile tQ = t8::tile(sQ, 64), tK = t8::tile(sK, 64), tA = t8::tile(sA, 128), tB = t8::tile(sB, 128);
    wait_or_flag(&ld_bar, 0, p.status, 2);
    if (tid == 0) {
        t8::mma_chain<false, false>(tmem, tA, 0, 0, tK, 0, 0, 64, K, false);
        t8::mma_chain<false, false>(tmem + 64, tA, 0, 0, tB, 0, 0, 128, K, false);
        umma_commit(&mma_bar);
    }
    wait_or_flag(&mma_bar, 0, p.status, 3);
    tc_fence_after();
    {
        const int r = tid, i = r >> 1;
        for (int cg = 0; cg < 8; ++cg) {                      // Aak: columns j < i
            uint32_t v[8]; float f[8];
            tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = (cg * 8 + j) < i ? __uint_as_float(v[j]) : 0.f;
            p.Aak[g * CH64 + cg * 128 + r] = t8::pack8(f);    // [128 x 64] tile: 8 column groups of 128 rows
        }
        for (int cg = 0; cg < 16; ++cg) {                     // Aab: column token < row token
            uint32_t v[8]; float f[8];
            tmem_ld_x8(t8::taddr(tmem, warp, 64 + cg * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = ((cg * 8 + j) >> 1) < i ? __uint_as_float(v[j]) : 0.f;
            p.Aab[g * CH128 + cg * 128 + r] = t8::pack8(f);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
        // Qh has 64 rows: the upper 64 lanes of this M=128 product read past the tile and are ignored
        t8::mma_chain<false, false>(tmem, tQ, 0, 0, tK, 0, 0, 64, K, false);
        t8::mma_chain<false, false>(tmem + 64, tQ, 0, 0, tB, 0, 0, 128, K, false);
        umma_commit(&mma_bar);
    }
    wait_or_flag(&mma_bar, 1, p.status, 4);
    tc_fence_after();
    if (warp < 2) {
        const int i = tid;
        for (int cg = 0; cg < 8; ++cg) {                      // Aqk: j <= i
            uint32_t v[8]; float f[8];
            tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = (cg * 8 + j) <= i ? __uint_as_float(v[j]) : 0.f;
            p.Aqk[g * 512 + cg * 64 + i] = t8::pack8(f);
        }
        for (int cg = 0; cg < 16; ++cg) {                     // Aqb: column token <= i
            uint32_t v[8]; float f[8];
            tmem_ld_x8(t8::taddr(tmem, warp, 64 + cg * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = ((cg * 8 + j) >> 1) <= i ? __uint_as_float(v[j]) : 0.f;
            p.Aqb[g * CH64 + cg * 64 + i] = t8::pack8(f);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------
// K3: M = (I - Aab)^-1   (HRDPLR/naive.py:189-192; reference kernel HRDPLR/fwd_triton.py:588-667)
//   16x16 diagonal blocks by forward substitution in registers, then three doubling levels
//   M21 = M22 L21 M11, each evaluated for all block pairs at once as two full 128^3 tensor-core
//   products (X = L D, Y = D X with D the current block-diagonal inverse).
// ------------------------------------------------------------------------------------------
struct InvP {
    const uint4* Aab;
    uint4* M;
    int* status;
};

__device__ __forceinline__ float c8_elem(const uint4* tile, int rows, int r, int c) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(tile + (c >> 3) * rows + r);
    return __bfloat162float(p[c & 7]);
}

__global__ void __launch_bounds__(128) inverse_tc_kernel(InvP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sL = reinterpret_cast<uint4*>(smem);
    uint4* sD = sL + CH128;
    uint4* sX = sD + CH128;
    __shared__ __align__(8) uint64_t ld_bar, mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 128); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 32768);
        bulk_g2s(sL, p.Aab + g * CH128, 32768, &ld_bar);
    }
    for (int e = tid; e < CH128; e += 128) sD[e] = make_uint4(0, 0, 0, 0);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    wait_or_flag(&ld_bar, 0, p.status, 5);
    {   // diagonal 16x16 blocks: thread = (block, column)
        const int blk = tid >> 4, c = tid & 15, base = blk * 16;
        float mcol[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float s = (i == c) ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < i) s = fmaf(c8_elem(sL, 128, base + i, base + j), mcol[j], s);
            mcol[i] = s;
        }
        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(sD);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int row = base + i, col = base + c;
            d[((size_t)(col >> 3) * 128 + row) * 8 + (col & 7)] = __float2bfloat16_rn(mcol[i]);
        }
    }
    fence_proxy_async();
    __syncthreads();
    const Tile tL = t8::tile(sL, 128), tD = t8::tile(sD, 128), tX = t8::tile(sX, 128);
    uint32_t phase = 0;
    for (int bs = 16; bs <= 64; bs <<= 1) {
        if (tid == 0) {
            tc_fence_after();
            t8::mma_chain<false, true>(tmem, tL, 0, 0, tD, 0, 0, 128, 128, false);   // X = L D
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, phase, p.status, 6);
        phase ^= 1;
        tc_fence_after();
        for (int cg = 0; cg < 16; ++cg) {
            uint32_t v[8]; float f[8];
            tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
            sX[cg * 128 + tid] = t8::pack8(f);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            t8::mma_chain<false, true>(tmem, tD, 0, 0, tX, 0, 0, 128, 128, false);   // Y = D X
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, phase, p.status, 7);
        phase ^= 1;
        tc_fence_after();
        {
            // rows of an odd block I take the columns of block I-1; the column range is warp-uniform
            const int row_lo = warp * 32;
            const int I_hi = (row_lo + 31) / bs;                // block of the warp's last row
            const int I_odd = (I_hi & 1) ? I_hi : -1;
            if (I_odd > 0 && (I_odd * bs) < row_lo + 32) {
                const int c_lo = (I_odd - 1) * bs;
                const bool mine = (tid / bs) == I_odd;
                for (int cg = c_lo >> 3; cg < (c_lo + bs) >> 3; ++cg) {
                    uint32_t v[8]; float f[8];
                    tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
                    if (mine) sD[cg * 128 + tid] = t8::pack8(f);
                }
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
    }
    for (int e = tid; e < CH128; e += 128) p.M[g * CH128 + e] = sD[e];
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// ------------------------------------------------------------------------------------------
// K4: P = Aak v ; u = M P ; Wh = M Ah     (HRDPLR/naive.py:195-196; HRDPLR/fwd_triton.py:674-790)
// ------------------------------------------------------------------------------------------
struct WuP {
    const uint4 *M, *Ah, *Aak, *Vc;
    uint4 *P, *U, *W;
    int* status;
};

__global__ void __launch_bounds__(128) wu_tc_kernel(WuP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sM = reinterpret_cast<uint4*>(smem);                  // 32 KB
    uint4* sA = sM + CH128;                                      // 32 KB  Ah
    uint4* sAak = sA + CH128;                                    // 16 KB  [128 x 64]
    uint4* sV = sAak + CH64;                                     // 16 KB  [64 x 128]
    uint4* sP = sAak;                                            // P overlays Aak + v once they are consumed
    __shared__ __align__(8) uint64_t ld_bar, mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 98304);
        bulk_g2s(sAak, p.Aak + g * CH64, 16384, &ld_bar);
        bulk_g2s(sV, p.Vc + g * CH64, 16384, &ld_bar);
        bulk_g2s(sM, p.M + g * CH128, 32768, &ld_bar);
        bulk_g2s(sA, p.Ah + g * CH128, 32768, &ld_bar);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const Tile tM = t8::tile(sM, 128), tA = t8::tile(sA, 128), tAak = t8::tile(sAak, 128), tV = t8::tile(sV, 64),
               tP = t8::tile(sP, 128);
    wait_or_flag(&ld_bar, 0, p.status, 8);
    if (tid == 0) {
        t8::mma_chain<false, true>(tmem, tAak, 0, 0, tV, 0, 0, 128, 64, false);          // P = Aak v
        t8::mma_chain<false, true>(tmem + 128, tM, 0, 0, tA, 0, 0, 128, 128, false);     // Wh = M Ah
        umma_commit(&mma_bar);
    }
    wait_or_flag(&mma_bar, 0, p.status, 9);
    tc_fence_after();
    for (int cg = 0; cg < 16; ++cg) {
        uint32_t v[8]; float f[8];
        tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
        const uint4 c = t8::pack8(f);
        sP[cg * 128 + tid] = c;
        p.P[g * CH128 + cg * 128 + tid] = c;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        t8::mma_chain<false, true>(tmem, tM, 0, 0, tP, 0, 0, 128, 128, false);           // u = M P
        umma_commit(&mma_bar);
    }
    for (int cg = 0; cg < 16; ++cg) {                                                     // Wh while u runs
        uint32_t v[8]; float f[8];
        tmem_ld_x8(t8::taddr(tmem, warp, 128 + cg * 8), v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
        p.W[g * CH128 + cg * 128 + tid] = t8::pack8(f);
    }
    wait_or_flag(&mma_bar, 1, p.status, 10);
    tc_fence_after();
    for (int cg = 0; cg < 16; ++cg) {
        uint32_t v[8]; float f[8];
        tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
        p.U[g * CH128 + cg * 128 + tid] = t8::pack8(f);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------
// K5: inter-chunk state scan   (HRDPLR/fwd_triton.py:795-968; HRDPLR/naive.py:232-255)
//   per chunk:  St = E (.) S ;  v2 = Wh St + u ;  S <- E (.) (St + Kh^T v + Bh^T v2)
// One CTA (8 warps) per (batch, head).  The fp32 state lives in registers: thread (k = lane of
// warp%4, column half = warp/4) owns S[k, 64 columns].  The operands of the next chunk are
// prefetched by bulk copies as soon as the product that reads their buffer has completed.
// ------------------------------------------------------------------------------------------
struct ScanTcP {
    const uint4 *W, *U, *Kh, *Bh, *Vc;
    const float* E;
    const float* h0;
    uint4 *Hs, *V2;
    float* ht;
    int NT;
    int* status;
};

__global__ void __launch_bounds__(256) scan_fwd_tc_kernel(ScanTcP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sW = reinterpret_cast<uint4*>(smem);      // 32 KB
    uint4* sU = sW + CH128;                          // 32 KB
    uint4* sKh = sU + CH128;                         // 16 KB
    uint4* sV = sKh + CH64;                          // 16 KB
    uint4* sBh = sV + CH64;                          // 32 KB
    uint4* sSt = sBh + CH128;                        // 32 KB  St [k x v]
    uint4* sV2 = sSt + CH128;                        // 32 KB  v2 [128 x v]
    __shared__ __align__(8) uint64_t ldA, ldB, barA, barB;
    __shared__ uint32_t tmem_s;
    const int bh = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = (warp & 3) * 32 + lane;          // TMEM lane = k (state) or a/b row (v2)
    const int half = warp >> 2;                      // which 64 columns
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    const long long g0 = (long long)bh * p.NT;
    if (tid == 0) {
        mbar_init(&ldA, 1); mbar_init(&ldB, 1); mbar_init(&barA, 1); mbar_init(&barB, 1); fence_mbar_init();
        mbar_expect_tx(&ldA, 65536);
        bulk_g2s(sW, p.W + g0 * CH128, 32768, &ldA);
        bulk_g2s(sU, p.U + g0 * CH128, 32768, &ldA);
        mbar_expect_tx(&ldB, 65536);
        bulk_g2s(sKh, p.Kh + g0 * CH64, 16384, &ldB);
        bulk_g2s(sV, p.Vc + g0 * CH64, 16384, &ldB);
        bulk_g2s(sBh, p.Bh + g0 * CH128, 32768, &ldB);
    }
    float S[64];
    if (p.h0) {
        const float4* src = reinterpret_cast<const float4*>(p.h0 + ((size_t)bh * K + row) * V + half * 64);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float4 x = src[j];
            S[4 * j] = x.x; S[4 * j + 1] = x.y; S[4 * j + 2] = x.z; S[4 * j + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) S[j] = 0.f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const Tile tW = t8::tile(sW, 128), tKh = t8::tile(sKh, 64), tV = t8::tile(sV, 64), tBh = t8::tile(sBh, 128),
               tSt = t8::tile(sSt, 128), tV2 = t8::tile(sV2, 128);
    for (int n = 0; n < p.NT; ++n) {
        const long long g = g0 + n;
        const uint32_t ph = n & 1;
        const float e = p.E[(size_t)g * K + row];
        // St = E (.) S  -> operand tile and checkpoint
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = e * S[c8 * 8 + j];
            const uint4 c = t8::pack8(f);
            const int cg = half * 8 + c8;
            sSt[cg * 128 + row] = c;
            p.Hs[g * CH128 + cg * 128 + row] = c;
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            wait_or_flag(&ldA, ph, p.status, 11);
            tc_fence_after();
            t8::mma_chain<false, true>(tmem, tW, 0, 0, tSt, 0, 0, 128, 128, false);      // Wh St
            umma_commit(&barA);
        }
        wait_or_flag(&barA, ph, p.status, 12);
        wait_or_flag(&ldA, ph, p.status, 13);         // u is read from shared memory below
        tc_fence_after();
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
            const int cg = half * 8 + c8;
            uint32_t v[8]; float f[8], u[8];
            tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
            t8::unpack8(sU[cg * 128 + row], u);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]) + u[j];
            const uint4 c = t8::pack8(f);
            sV2[cg * 128 + row] = c;
            p.V2[g * CH128 + cg * 128 + row] = c;
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            if (n + 1 < p.NT) {                        // W and u buffers are free: prefetch the next chunk's
                mbar_expect_tx(&ldA, 65536);
                bulk_g2s(sW, p.W + (g + 1) * CH128, 32768, &ldA);
                bulk_g2s(sU, p.U + (g + 1) * CH128, 32768, &ldA);
            }
            wait_or_flag(&ldB, ph, p.status, 14);
            tc_fence_after();
            t8::mma_chain<true, true>(tmem + 128, tKh, 0, 0, tV, 0, 0, 128, 64, false);  // Kh^T v
            t8::mma_chain<true, true>(tmem + 128, tBh, 0, 0, tV2, 0, 0, 128, 128, true); // + Bh^T v2
            umma_commit(&barB);
        }
        wait_or_flag(&barB, ph, p.status, 15);
        tc_fence_after();
        if (tid == 0 && n + 1 < p.NT) {
            mbar_expect_tx(&ldB, 65536);
            bulk_g2s(sKh, p.Kh + (g + 1) * CH64, 16384, &ldB);
            bulk_g2s(sV, p.Vc + (g + 1) * CH64, 16384, &ldB);
            bulk_g2s(sBh, p.Bh + (g + 1) * CH128, 32768, &ldB);
        }
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
            uint32_t v[8];
            tmem_ld_x8(t8::taddr(tmem, warp, 128 + (half * 8 + c8) * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) S[c8 * 8 + j] = e * fmaf(e, S[c8 * 8 + j], __uint_as_float(v[j]));
        }
        tc_fence_before();
    }
    if (p.ht) {
        float4* dst = reinterpret_cast<float4*>(p.ht + ((size_t)bh * K + row) * V + half * 64);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------
// K6: o = Qh St + Aqk v + Aqb v2     (HRDPLR/fwd_triton.py:973-1094)
// ------------------------------------------------------------------------------------------
struct OutP {
    const uint4 *Qh, *Aqk, *Aqb, *Vc, *Hs, *V2;
    __nv_bfloat16* o;
    int T, H, NT;
    int* status;
};

__global__ void __launch_bounds__(128) out_tc_kernel(OutP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sQ = reinterpret_cast<uint4*>(smem);      // 16 KB [64 x 128]
    uint4* sAqk = sQ + CH64;                         //  8 KB [64 x 64]
    uint4* sAqb = sAqk + 512;                        // 16 KB [64 x 128]
    uint4* sV = sAqb + CH64;                         // 16 KB [64 x 128]
    uint4* sH = sV + CH64;                           // 32 KB [128 x 128]
    uint4* sV2 = sH + CH128;                         // 32 KB [128 x 128]
    __shared__ __align__(8) uint64_t ld_bar, mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 128); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 122880);
        bulk_g2s(sQ, p.Qh + g * CH64, 16384, &ld_bar);
        bulk_g2s(sH, p.Hs + g * CH128, 32768, &ld_bar);
        bulk_g2s(sAqk, p.Aqk + g * 512, 8192, &ld_bar);
        bulk_g2s(sV, p.Vc + g * CH64, 16384, &ld_bar);
        bulk_g2s(sAqb, p.Aqb + g * CH64, 16384, &ld_bar);
        bulk_g2s(sV2, p.V2 + g * CH128, 32768, &ld_bar);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    wait_or_flag(&ld_bar, 0, p.status, 16);
    if (tid == 0) {
        // the three A operands have 64 rows; lanes 64..127 of the accumulator are never read
        t8::mma_chain<false, true>(tmem, t8::tile(sQ, 64), 0, 0, t8::tile(sH, 128), 0, 0, 128, 128, false);
        t8::mma_chain<false, true>(tmem, t8::tile(sAqk, 64), 0, 0, t8::tile(sV, 64), 0, 0, 128, 64, true);
        t8::mma_chain<false, true>(tmem, t8::tile(sAqb, 64), 0, 0, t8::tile(sV2, 128), 0, 0, 128, 128, true);
        umma_commit(&mma_bar);
    }
    wait_or_flag(&mma_bar, 0, p.status, 17);
    tc_fence_after();
    if (warp < 2) {
        const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
        const int b = bh / p.H, h = bh % p.H;
        const int t = n * C + tid;
        uint4* dst = reinterpret_cast<uint4*>(p.o + (((size_t)b * p.T + t) * p.H + h) * V);
        for (int cg = 0; cg < 16; ++cg) {
            uint32_t v[8]; float f[8];
            tmem_ld_x8(t8::taddr(tmem, warp, cg * 8), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
            if (t < p.T) dst[cg] = t8::pack8(f);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// debugging aid: C8 bf16 tile -> fp32 row-major
__global__ void c8_to_rowmajor_kernel(const uint4* src, float* dst, int rows, int cols) {
    const long long g = blockIdx.x;
    const int nch = rows * cols / 8;
    for (int e = threadIdx.x; e < nch; e += blockDim.x) {
        const int cg = e / rows, r = e % rows;
        float f[8];
        t8::unpack8(src[g * nch + e], f);
        for (int j = 0; j < 8; ++j) dst[(size_t)g * rows * cols + (size_t)r * cols + cg * 8 + j] = f[j];
    }
}

template <typename Kern>
int set_smem(Kern kern, int bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return HDLA_OK;
}

}  // namespace

bool tc_supported(const HdlaDims& d) {
    return d.dtype == HDLA_BF16 && !(d.flags & HDLA_FLAG_FORCE_SIMT) && effective_chunk(d.T, d.C) == C && d.R == R &&
           d.K == K && d.V == V && (long long)d.B * d.H * ((d.T + C - 1) / C) < 0x7fffffffLL;
}

size_t tc_workspace_bytes(const HdlaDims& d, int with_backward) {
    TcPlan pl = make_tc_plan(d);
    return with_backward ? pl.total : pl.total_fwd;
}

#define TRY(x) do { int rc__ = (x); if (rc__ != HDLA_OK) return rc__; } while (0)

int tc_chunk_fwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                 const void* gk, float scale, const float* h0, void* o, float* ht, unsigned char* ws, bool need_o,
                 cudaStream_t st) {
    const TcPlan pl = make_tc_plan(d);
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        TRY(set_smem(gram_tc_kernel, 98304 + 1024));
        TRY(set_smem(inverse_tc_kernel, 98304));
        TRY(set_smem(wu_tc_kernel, 98304));
        TRY(set_smem(scan_fwd_tc_kernel, 196608));
        TRY(set_smem(out_tc_kernel, 122880));
        attr_dev = dev;
    }
    auto U4 = [&](size_t off) { return reinterpret_cast<uint4*>(ws + off); };
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    int* status = reinterpret_cast<int*>(ws + pl.status);
    const unsigned G = (unsigned)pl.G;
    typedef const __nv_bfloat16* bp;
    PrepP pp{(bp)q, (bp)k, (bp)v, (bp)a, (bp)b, gk, U4(pl.Qh), U4(pl.Kh), U4(pl.Ah), U4(pl.Bh), U4(pl.Vc), F(pl.E),
             F(pl.ghat), scale, d.T, d.H, pl.NT, d.gk_dtype};
    prep_hat_kernel<<<G, 128, 0, st>>>(pp);
    HDLA_CHECK_LAUNCH("prep_hat_kernel");
    GramP gp{U4(pl.Qh), U4(pl.Kh), U4(pl.Ah), U4(pl.Bh), U4(pl.Aqk), U4(pl.Aqb), U4(pl.Aak), U4(pl.Aab), status};
    gram_tc_kernel<<<G, 128, 98304 + 1024, st>>>(gp);
    HDLA_CHECK_LAUNCH("gram_tc_kernel");
    InvP ivp{U4(pl.Aab), U4(pl.M), status};
    inverse_tc_kernel<<<G, 128, 98304, st>>>(ivp);
    HDLA_CHECK_LAUNCH("inverse_tc_kernel");
    WuP wp{U4(pl.M), U4(pl.Ah), U4(pl.Aak), U4(pl.Vc), U4(pl.P), U4(pl.U), U4(pl.W), status};
    wu_tc_kernel<<<G, 128, 98304, st>>>(wp);
    HDLA_CHECK_LAUNCH("wu_tc_kernel");
    ScanTcP sp{U4(pl.W), U4(pl.U), U4(pl.Kh), U4(pl.Bh), U4(pl.Vc), F(pl.E), h0, U4(pl.Hs), U4(pl.V2), ht, pl.NT,
               status};
    scan_fwd_tc_kernel<<<pl.BH, 256, 196608, st>>>(sp);
    HDLA_CHECK_LAUNCH("scan_fwd_tc_kernel");
    if (need_o) {
        OutP op{U4(pl.Qh), U4(pl.Aqk), U4(pl.Aqb), U4(pl.Vc), U4(pl.Hs), U4(pl.V2), (__nv_bfloat16*)o, d.T, d.H,
                pl.NT, status};
        out_tc_kernel<<<G, 128, 122880, st>>>(op);
        HDLA_CHECK_LAUNCH("out_tc_kernel");
    }
    return HDLA_OK;
}

// debugging aid: named bf16 tile buffer of the tensor-core workspace -> fp32 row-major [G][rows][cols]
int tc_debug_buffer(const HdlaDims& d, const unsigned char* ws, const char* name, float* out, cudaStream_t st) {
    const TcPlan pl = make_tc_plan(d);
    struct Ent { const char* n; size_t off; int rows, cols; };
    const Ent tab[] = {{"Qh", pl.Qh, 64, 128}, {"Kh", pl.Kh, 64, 128}, {"Ah", pl.Ah, 128, 128}, {"Bh", pl.Bh, 128, 128},
                       {"Vc", pl.Vc, 64, 128}, {"Aqk", pl.Aqk, 64, 64}, {"Aqb", pl.Aqb, 64, 128},
                       {"Aak", pl.Aak, 128, 64}, {"Aab", pl.Aab, 128, 128}, {"M", pl.M, 128, 128},
                       {"W", pl.W, 128, 128}, {"P", pl.P, 128, 128}, {"U", pl.U, 128, 128}, {"Hs", pl.Hs, 128, 128},
                       {"V2", pl.V2, 128, 128}};
    for (const Ent& e : tab)
        if (!strcmp(e.n, name)) {
            c8_to_rowmajor_kernel<<<(unsigned)pl.G, 128, 0, st>>>(reinterpret_cast<const uint4*>(ws + e.off), out,
                                                                  e.rows, e.cols);
            HDLA_CHECK_LAUNCH("c8_to_rowmajor_kernel");
            return HDLA_OK;
        }
    if (!strcmp(name, "E")) {
        cudaMemcpyAsync(out, ws + pl.E, (size_t)pl.G * K * 4, cudaMemcpyDeviceToDevice, st);
        return HDLA_OK;
    }
    if (!strcmp(name, "status")) {
        cudaMemcpyAsync(out, ws + pl.status, 4, cudaMemcpyDeviceToDevice, st);
        return HDLA_OK;
    }
    return fail(HDLA_ERR_INVALID, "unknown debug buffer '%s'", name);
}

}  // namespace hdla
