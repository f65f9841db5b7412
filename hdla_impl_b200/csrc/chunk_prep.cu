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
    const int2* chunk_tab;                // variable-length batches: (first token, tokens) per chunk, else null
};

struct In6 { uint4 q, k, a0, a1, b0, b1; };

// 16-byte read-only load that stays where it is written: the loads of the streaming part are issued long before
// their use on purpose (a whole tile phase ahead), and an ordinary load may be moved down to its use.
__device__ __forceinline__ uint4 ld_pinned(const void* ptr) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(ptr) : "memory");
    return r;
}

// The six operand pieces of (row, column group cg).  Unconditional: a row beyond the sequence's end is read from
// the last row that exists and zeroed when it is used (a conditional load would tie the data to a register move at
// the point of the condition and so bring the wait for the data forward to there).
__device__ __forceinline__ In6 load6(const ChunkPrepP& p, int b, int h, int t0, int valid, int row, int cg) {
    const int rr = min(row, valid - 1);
    const size_t src = (((size_t)b * p.T + t0 + rr) * p.H + h) * K + cg * 8;
    const size_t sa0 = (((size_t)b * p.T * R + (size_t)(t0 + rr) * R) * p.H + h) * K + cg * 8;
    const size_t sa1 = sa0 + (size_t)p.H * K;
    In6 x;
    x.q = ld_pinned(p.q + src);
    x.k = ld_pinned(p.k + src);
    x.a0 = ld_pinned(p.a + sa0);
    x.a1 = ld_pinned(p.a + sa1);
    x.b0 = ld_pinned(p.b + sa0);
    x.b1 = ld_pinned(p.b + sa1);
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

// 32 accumulator columns [col0, col0 + 32) of this thread's row -> four bf16 chunks, keep(column) says which
// entries survive the mask; emit(chunk number within the 32 columns, chunk).  32 columns at a time keep the
// epilogues' register footprint small next to the requests held for the next tile.
template <typename Keep, typename Emit>
__device__ __forceinline__ void epilogue32(uint32_t taddr, int col0, Keep keep, Emit emit) {
    uint32_t a[32];
    tmem_ld_x32(taddr, a);
    tmem_wait_ld();
#pragma unroll
    for (int c8 = 0; c8 < 4; ++c8) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = keep(col0 + c8 * 8 + j) ? __uint_as_float(a[c8 * 8 + j]) : 0.f;
        emit(c8, t8::pack8(f));
    }
}

constexpr int kPrepSmem = 16384 + 16384 + 32768 + 32768 + 16384;      // 112 KB

// 16-byte asynchronous copy global -> shared without a register stage; with ok == false nothing is read and the
// destination is filled with zeros.
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                 ::"r"(smem_u32(dst_smem)), "l"(src), "r"(ok ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Raw gk pieces of one thread: rows r8 + 8 j, j = 0..7, of its column group (8 channels each).
template <bool GK32> struct GkRaw { uint4 r[GK32 ? 16 : 8]; };

// What a thread requests ahead of a tile: its gk pieces and the operand pieces of the first four row blocks.
template <bool GK32> struct TileHead { GkRaw<GK32> gk; In6 in[4]; };

struct TileCoord { int b, h, t0, valid; };

__device__ __forceinline__ TileCoord tile_coord(const ChunkPrepP& p, long long g) {
    const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
    TileCoord c;
    c.b = bh / p.H; c.h = bh % p.H;
    chunk_tokens(p.chunk_tab, n, p.T, c.t0, c.valid);
    return c;
}

// The requests are issued in small batches at several points of the preceding tile's tensor-core phases: the SM
// tracks a limited number of outstanding loads, and a burst of all of them at once holds up every later memory
// instruction of the warp (the epilogues' stores among them) until the burst has drained.
template <bool GK32>
__device__ __forceinline__ void load_head_gk(TileHead<GK32>& hd, const ChunkPrepP& p, const TileCoord& tc, int r8, int cg) {
    const size_t rstride = (size_t)p.H * K;
    const size_t e0 = (((size_t)tc.b * p.T + tc.t0 + r8) * p.H + tc.h) * K + cg * 8;
    if (GK32) {
        const float* src = static_cast<const float*>(p.gk) + e0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long off = (long long)(min(8 * j + r8, tc.valid - 1) - r8) * (long long)rstride;
            hd.gk.r[GK32 ? 2 * j : 0] = ld_pinned(src + off);
            hd.gk.r[GK32 ? 2 * j + 1 : 0] = ld_pinned(src + off + 4);
        }
    } else {
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.gk) + e0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            hd.gk.r[GK32 ? 0 : j] = ld_pinned(src + (long long)(min(8 * j + r8, tc.valid - 1) - r8) * (long long)rstride);
    }
}

template <bool GK32>
__device__ __forceinline__ void load_head_in(TileHead<GK32>& hd, const ChunkPrepP& p, const TileCoord& tc, int r8, int cg,
                                             int j) {
    hd.in[j] = load6(p, tc.b, tc.h, tc.t0, tc.valid, 8 * j + r8, cg);
}

// v rows of a tile -> the v slot in shared memory, by asynchronous copies (no registers held meanwhile)
__device__ __forceinline__ void request_v(const ChunkPrepP& p, const TileCoord& tc, uint4* sV, int r8, int cg) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int row = 8 * j + r8;
        const bool ok = row < tc.valid;
        const size_t src = (((size_t)tc.b * p.T + tc.t0 + (ok ? row : 0)) * p.H + tc.h) * V + cg * 8;
        cp_async16(sV + cg * 64 + row, p.v + src, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Persistent: the grid is two CTAs per SM and every CTA walks over the tiles g = blockIdx.x, blockIdx.x +
// gridDim.x, ...  While a tile's products, inverse and epilogues run, the thread already holds the requests for the
// NEXT tile's gk and first operand pieces in registers and the next tile's v is on its way to shared memory, so
// the load latency of a tile lies under the tensor-core phases of the tile before it.
template <bool GK32>
__global__ void __launch_bounds__(128, 2) chunk_prep_tc_kernel(ChunkPrepP p, long long G) {
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
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r8 = lane & 7, cg = warp * 4 + (lane >> 3);
    const unsigned full = 0xffffffffu;
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    if (tid == 0) { mbar_init(&mma_bar, 1); fence_mbar_init(); }
    long long g = blockIdx.x;
    TileCoord tc = tile_coord(p, g);
    TileHead<GK32> head;
    load_head_gk<GK32>(head, p, tc, r8, cg);
#pragma unroll
    for (int j = 0; j < 4; ++j) load_head_in<GK32>(head, p, tc, r8, cg, j);
    request_v(p, tc, sV, r8, cg);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    uint32_t phase = 0;
#pragma unroll 1
    for (; g < G; g += gridDim.x) {
    const long long gn = g + gridDim.x;
    const bool more = gn < G;
    const int b = tc.b, h = tc.h, t0 = tc.t0, valid = tc.valid;
    if (tid == 0) TL(0);

    // ---- chunk-local cumulative sum of gk (inclusive), in registers
    float gi[8][8];
    if (GK32) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 lo = head.gk.r[GK32 ? 2 * j : 0], hi = head.gk.r[GK32 ? 2 * j + 1 : 0];
            gi[j][0] = __uint_as_float(lo.x); gi[j][1] = __uint_as_float(lo.y); gi[j][2] = __uint_as_float(lo.z); gi[j][3] = __uint_as_float(lo.w);
            gi[j][4] = __uint_as_float(hi.x); gi[j][5] = __uint_as_float(hi.y); gi[j][6] = __uint_as_float(hi.z); gi[j][7] = __uint_as_float(hi.w);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) t8::unpack8(head.gk.r[GK32 ? 0 : j], gi[j]);
    }
    if (valid < C) {                                           // ragged last chunk: rows beyond the end decay by nothing
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (8 * j + r8 >= valid) {
#pragma unroll
                for (int c = 0; c < 8; ++c) gi[j][c] = 0.f;
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

    if (tid == 0) TL(1);
    // ---- hat operands, straight into the C8 operand tiles
    {
        float ep_prev[8];                                         // e^{gi - half} of this lane's row in the previous block
#pragma unroll
        for (int c = 0; c < 8; ++c) ep_prev[c] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            In6 cur = head.in[j & 3];
            if (j + 4 < 8) head.in[j & 3] = load6(p, b, h, t0, valid, 8 * (j + 4) + r8, cg);
            const int row = 8 * j + r8;
            if (row >= valid) {                                // rows beyond the sequence's end are zero
                const uint4 zero = make_uint4(0, 0, 0, 0);
                cur.q = zero; cur.k = zero; cur.a0 = zero; cur.a1 = zero; cur.b0 = zero; cur.b1 = zero;
            }
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
    if (tid == 0) TL(2);
    cp_async_wait_all();                                       // this tile's v has landed in its slot
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) TL(3);
    const Tile tQ = t8::tile(sQ, 64), tK = t8::tile(sK, 64), tA = t8::tile(sA, 128), tB = t8::tile(sD, 128);
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
    // the registers of the streaming part are free: request the next tile's gk and first operand pieces now
    // (unconditionally -- the last tile of a CTA requests its own pieces once more -- so that no condition ties the
    //  data to this point)
    tc = tile_coord(p, more ? gn : g);
    load_head_gk<GK32>(head, p, tc, r8, cg);
    if (warp < 2) {
        wait_or_flag(&mma_bar, phase, p.status, 20);
        tc_fence_after();
        const int i = tid;
#pragma unroll 1
        for (int q4 = 0; q4 < 2; ++q4)                         // Aqk: j <= i
            epilogue32(t8::taddr(tmem, warp, q4 * 32), q4 * 32, [&](int c) { return c <= i; },
                       [&](int c8, uint4 ch) { p.Aqk[g * 512 + (q4 * 4 + c8) * 64 + i] = ch; });
#pragma unroll 1
        for (int q4 = 0; q4 < 4; ++q4)                         // Aqb: column token <= i
            epilogue32(t8::taddr(tmem, warp, 64 + q4 * 32), q4 * 32, [&](int c) { return (c >> 1) <= i; },
                       [&](int c8, uint4 ch) { p.Aqb[g * CH64 + (q4 * 4 + c8) * 64 + i] = ch; });
    }
    phase ^= 1;
    if (tid == 0) TL(4);
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
    if (tid == 0) TL(5);
    {   // Aak (strict mask) replaces Qh, Aab (strict mask in tokens) replaces Bh
        const int r = tid, i = r >> 1;
#pragma unroll 1
        for (int q4 = 0; q4 < 2; ++q4)                         // [128 x 64] tile: 8 column groups of 128 rows
            epilogue32(t8::taddr(tmem, warp, q4 * 32), q4 * 32, [&](int c) { return c < i; },
                       [&](int c8, uint4 ch) { sQ[(q4 * 4 + c8) * 128 + r] = ch; });
#pragma unroll 1
        for (int q4 = 0; q4 < 4; ++q4)
            epilogue32(t8::taddr(tmem, warp, 64 + q4 * 32), q4 * 32, [&](int c) { return (c >> 1) < i; },
                       [&](int c8, uint4 ch) { sD[(q4 * 4 + c8) * 128 + r] = ch; });
    }
    load_head_in<GK32>(head, p, tc, r8, cg, 0);                // next tile: first row block
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0 && p.save_bwd) {
        bulk_s2g(p.Aak + g * CH64, sQ, 16384);
        bulk_commit();
    }
    if (tid == 0) TL(6);

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
    if (tid == 0) TL(7);
    load_head_in<GK32>(head, p, tc, r8, cg, 1);
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
    if (tid == 0) TL(8);
    load_head_in<GK32>(head, p, tc, r8, cg, 2);
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
    if (tid == 0) TL(9);
    load_head_in<GK32>(head, p, tc, r8, cg, 3);
    if (more) request_v(p, tc, sV, r8, cg);                    // P = Aak v is complete: the v slot takes the next tile's
#pragma unroll 1
    for (int q4 = 0; q4 < 4; ++q4)
        epilogue32(t8::taddr(tmem, warp, q4 * 32), 0, [](int) { return true; },
                   [&](int c8, uint4 ch) { sP[(q4 * 4 + c8) * 128 + tid] = ch; });
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
    // Wh while u runs: into the Ah slot (Wh = M Ah is complete, Ah's copy to global memory was waited for before
    // the Aak epilogue), from where one bulk copy takes it to global memory
#pragma unroll 1
    for (int q4 = 0; q4 < 4; ++q4)
        epilogue32(t8::taddr(tmem, warp, 128 + q4 * 32), 0, [](int) { return true; },
                   [&](int c8, uint4 ch) { sA[(q4 * 4 + c8) * 128 + tid] = ch; });
    if (tid == 0) TL(10);
    wait_or_flag(&mma_bar, phase, p.status, 25);
    phase ^= 1;
    tc_fence_after();
    if (tid == 0) TL(11);
#pragma unroll 1
    for (int q4 = 0; q4 < 4; ++q4)
        epilogue32(t8::taddr(tmem, warp, q4 * 32), 0, [](int) { return true; },
                   [&](int c8, uint4 ch) { p.U[g * CH128 + (q4 * 4 + c8) * 128 + tid] = ch; });
    if (tid == 0) TL(12);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        bulk_s2g(p.W + g * CH128, sA, 32768);
        bulk_commit();
        bulk_wait_read<0>();                                   // the tiles are rewritten / released only after the copies read them
    }
    __syncthreads();
    tc_fence_after();
    if (tid == 0) TL(13);
    }
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
        cudaError_t e = cudaFuncSetAttribute(chunk_prep_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(chunk_prep_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem);
        if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_dev = dev;
    }
    auto U4 = [&](size_t off) { return reinterpret_cast<uint4*>(ws + off); };
    typedef const __nv_bfloat16* bp;
    ChunkPrepP pp{(bp)q, (bp)k, (bp)v, (bp)a, (bp)b, gk,
                  U4(pl.Qh), U4(pl.Kh), U4(pl.Ah), U4(pl.Bh), U4(pl.Vc), U4(pl.Aqk), U4(pl.Aqb), U4(pl.Aak), U4(pl.M),
                  U4(pl.W), U4(pl.P), U4(pl.U), reinterpret_cast<float*>(ws + pl.E),
                  reinterpret_cast<__nv_bfloat16*>(ws + pl.ghat), scale, d.T, d.H, pl.NT, d.gk_dtype, save_bwd ? 1 : 0,
                  reinterpret_cast<int*>(ws + pl.status),
                  pl.nseq ? reinterpret_cast<const int2*>(ws + pl.chunk_tab) : nullptr};
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const long long slots = 2LL * sms;                     // two CTAs per SM, persistent
    const unsigned grid = (unsigned)(pl.G < slots ? pl.G : slots);
    if (d.gk_dtype == HDLA_F32) launch(chunk_prep_tc_kernel<true>, dim3(grid), dim3(128), kPrepSmem, st, pp, pl.G);
    else                        launch(chunk_prep_tc_kernel<false>, dim3(grid), dim3(128), kPrepSmem, st, pp, pl.G);
    HDLA_CHECK_LAUNCH("chunk_prep_tc_kernel");
    return HDLA_OK;
}

}  // namespace hdla

#ifdef HDLA_TIMELINE
extern "C" __attribute__((visibility("default"))) int hdla_debug_timeline_prep(unsigned long long* host_dst, size_t count) {
    return (int)cudaMemcpyFromSymbol(host_dst, hdla::tc::g_timeline, count * sizeof(unsigned long long));
}
#endif
