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

#include <vector>

#include "tc_plan.cuh"

namespace hdla {
namespace {

using namespace sm100;
using namespace tc;
using t8::Tile;

// ------------------------------------------------------------------------------------------
// K1: cumulative decay and hat operands (CUDA cores, streaming)
//   gi = inclusive cumsum of gk within the chunk; ge = gi - gk (fla chunk_rwkv6_fwd_cumsum, call
//   site HRDPLR/hrdplr.py:44); gating as HRDPLR/fwd_triton.py:222-245 but around half = g_last/2.
// ------------------------------------------------------------------------------------------
struct PrepP {
    const __nv_bfloat16 *q, *k, *v, *a, *b;
    const void* gk;
    uint4 *Qh, *Kh, *Ah, *Bh, *Vc;
    float* E;
    __nv_bfloat16* ghat;                  // e^{gi - half} per (token, channel), bf16 row-major [64][128]
    float scale;
    int T, H, NT, gdt;
    int* status;
    int Kd, Vd;                           // head dims of the public tensors (multiples of 8, <= 128); the tiles are padded with zeros
    const int2* chunk_tab;                // variable-length batches: (first token, tokens) per chunk, else null
    const __nv_bfloat16* beta;            // in-operator a/b parametrisation: [B,T,H]; a and b are not read, gk is log_f
    int norm_k;                           // ... with k normalised on the way: k <- k / sqrt(sum_K k^2 + kNormEps)
};

// the seven 16-byte input pieces one thread handles per step: (row r, column group kc) of q, k, v, a0, a1, b0, b1
// (with the in-operator a/b parametrisation only q, k, v are read)
struct PrepIn { uint4 q, k, v, a0, a1, b0, b1; };

// Unconditional: a position outside the chunk's tokens or the head's channels is read from a clamped one and
// replaced by zeros where the data is used (a load inside a condition, merged with a default after it, can be waited
// for where the condition ends, which would undo the request one step ahead).
template <bool AB>
__device__ __forceinline__ PrepIn prep_load(const PrepP& p, int b, int h, int t0, int valid, int blk, int lane) {
    const int r = (blk >> 2) * 8 + (lane & 7);
    const int kc = (blk & 3) * 4 + (lane >> 3);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const bool row_ok = r < valid, k_ok = row_ok && kc * 8 < p.Kd, v_ok = row_ok && kc * 8 < p.Vd;
    const int rc = row_ok ? r : valid - 1;
    const size_t tok = (size_t)b * p.T + t0 + rc;
    const size_t src = (tok * p.H + h) * p.Kd + (k_ok ? kc * 8 : 0);
    const size_t sa0 = ((tok * R) * p.H + h) * p.Kd + (k_ok ? kc * 8 : 0);
    const size_t sa1 = sa0 + (size_t)p.H * p.Kd;
    PrepIn x;
    x.q = __ldg(reinterpret_cast<const uint4*>(p.q + src));
    x.k = __ldg(reinterpret_cast<const uint4*>(p.k + src));
    if (!AB) {
        x.a0 = __ldg(reinterpret_cast<const uint4*>(p.a + sa0));
        x.a1 = __ldg(reinterpret_cast<const uint4*>(p.a + sa1));
        x.b0 = __ldg(reinterpret_cast<const uint4*>(p.b + sa0));
        x.b1 = __ldg(reinterpret_cast<const uint4*>(p.b + sa1));
    } else {
        x.a0 = x.a1 = x.b0 = x.b1 = zero;
    }
    x.v = __ldg(reinterpret_cast<const uint4*>(p.v + (tok * p.H + h) * p.Vd + (v_ok ? kc * 8 : 0)));
    return x;                    // (the caller masks what lies outside: prep_mask)
}

// AB: the layer's a/b parametrisation (HRDPLR/hdla_custom.py:19-43) on the way:  with ef = e^{log_f} (log_f = gk),
//   a0 = -beta k,  a1 = a0 (ef + s),  s = -beta sum_K ef k^2,  b0 = ef k,  b1 = k      (rows 2t, 2t+1 of a / b)
// s needs whole rows: the cumulative-sum phase, where a warp holds 16 complete rows of log_f, also loads those rows
// of k and reduces ef k^2 over the warp; ef of a piece in the hat loop is e^{gi - ge}.  With norm_k the layer's
// l2_norm of k (HRDPLR/hdla_custom.py:248, normalizations/l2_norm.py:4-14) happens here too: the same phase reduces
// k^2, and every use of k below is k / sqrt(sum_K k^2 + eps).
template <bool AB>
__global__ void __launch_bounds__(128) prep_hat_kernel(PrepP p) {
    __shared__ float gis[C][K + 4];
    __shared__ float tot[4][K];
    __shared__ float4 beta_s[AB ? C : 1];           // (beta, s, 1 / |k| or 1) per row
    const long long g = blockIdx.x;
    const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
    const int b = bh / p.H, h = bh % p.H;
    int t0, valid;
    chunk_tokens(p.chunk_tab, n, p.T, t0, valid);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // The kernel is a stream: keep loads in flight at all times. The first step's operand pieces are requested
    // before the decay sums (they do not depend on them), and inside the loop the next step's pieces are
    // requested before the current step's arithmetic and stores.
    if (tid == 0) TL(0);
    PrepIn cur = prep_load<AB>(p, b, h, t0, valid, warp * 8, lane);
    {   // two-level cumulative sum: warp w owns rows [16w, 16w+16), lane owns 4 columns
        // (all sixteen loads are issued before the first value is used: the dtype branch stays outside the loops)
        float4 x[16];
        const size_t row0 = (((size_t)b * p.T + t0 + warp * 16) * p.H + h) * p.Kd + lane * 4;
        const size_t rstride = (size_t)p.H * p.Kd;
        const int nrow = lane * 4 < p.Kd ? valid - warp * 16 : 0;     // rows of this warp that exist (none in the padding)
        if (p.gdt == HDLA_F32) {
            const float* src = static_cast<const float*>(p.gk) + row0;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                x[i] = i < nrow ? __ldg(reinterpret_cast<const float4*>(src + i * rstride)) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.gk) + row0;
            uint2 raw[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                raw[i] = i < nrow ? __ldg(reinterpret_cast<const uint2*>(src + i * rstride)) : make_uint2(0u, 0u);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                x[i] = make_float4(__uint_as_float(raw[i].x << 16), __uint_as_float(raw[i].x & 0xffff0000u),
                                   __uint_as_float(raw[i].y << 16), __uint_as_float(raw[i].y & 0xffff0000u));
        }
        if (AB) {
            const __nv_bfloat16* ksrc = p.k + row0;
            uint2 kraw[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                kraw[i] = i < nrow ? __ldg(reinterpret_cast<const uint2*>(ksrc + i * rstride)) : make_uint2(0u, 0u);
            const int myrow = warp * 16 + (lane & 15);
            const float beta = myrow < valid ? __bfloat162float(p.beta[((size_t)b * p.T + t0 + myrow) * p.H + h]) : 0.f;
            float mine = 0.f, mine2 = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float k0 = __uint_as_float(kraw[i].x << 16), k1 = __uint_as_float(kraw[i].x & 0xffff0000u);
                const float k2 = __uint_as_float(kraw[i].y << 16), k3 = __uint_as_float(kraw[i].y & 0xffff0000u);
                float part = __expf(x[i].x) * k0 * k0 + __expf(x[i].y) * k1 * k1 + __expf(x[i].z) * k2 * k2 +
                             __expf(x[i].w) * k3 * k3;
                float sq = k0 * k0 + k1 * k1 + k2 * k2 + k3 * k3;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) {
                    part += __shfl_xor_sync(0xffffffffu, part, d);
                    sq += __shfl_xor_sync(0xffffffffu, sq, d);
                }
                if ((lane & 15) == i) { mine = part; mine2 = sq; }
            }
            const float rn = p.norm_k ? rsqrtf(mine2 + kNormEps) : 1.f;
            if (lane < 16) beta_s[myrow] = make_float4(beta, -beta * mine * rn * rn, rn, 0.f);
        }
        float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            run.x += x[i].x; run.y += x[i].y; run.z += x[i].z; run.w += x[i].w;
            x[i] = run;
        }
        *reinterpret_cast<float4*>(&tot[warp][lane * 4]) = run;
        if (tid == 0) TL(10);
        __syncthreads();
        if (tid == 0) TL(11);
        float4 off = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int w = 0; w < warp; ++w) {
            const float4 t = *reinterpret_cast<const float4*>(&tot[w][lane * 4]);
            off.x += t.x; off.y += t.y; off.z += t.z; off.w += t.w;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i)
            *reinterpret_cast<float4*>(&gis[warp * 16 + i][lane * 4]) =
                make_float4(x[i].x + off.x, x[i].y + off.y, x[i].z + off.z, x[i].w + off.w);
    }
    __syncthreads();
    if (tid == 0) TL(1);
    if (tid < K) {
        const float gl = gis[C - 1][tid];
        p.E[(size_t)g * K + tid] = __expf(0.5f * gl);
        if (!(fabsf(gl) <= kMaxChunkDecay)) atomicExch(p.status + kStatusDecay, 1);      // also catches NaN
        // largest chunk decay of the call (status word 2): warp maximum, then one filtered atomic per warp
        float worst = fabsf(gl);
        worst = worst == worst ? worst : 0.f;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) worst = fmaxf(worst, __shfl_xor_sync(0xffffffffu, worst, d));
        if (lane == 0 && __float_as_int(worst) > *reinterpret_cast<volatile int*>(p.status + kStatusMaxDecay))
            atomicMax(p.status + kStatusMaxDecay, __float_as_int(worst));
    }
    // hat operands: per instruction a warp covers 8 rows x 4 column groups, so every global access
    // is a run of full 32-byte sectors (64 B per row in, 128 B per column group out)
#pragma unroll 2
    for (int it = 0; it < 8; ++it) {
        const int blk = warp * 8 + it;                 // 32 blocks of (8 rows x 4 column groups)
        const int r = (blk >> 2) * 8 + (lane & 7);
        const int kc = (blk & 3) * 4 + (lane >> 3);
        PrepIn nxt = cur;
        if (it < 7) nxt = prep_load<AB>(p, b, h, t0, valid, blk + 1, lane);
        float gi[8], ge[8], hf[8];
        {
            const float4 g0 = *reinterpret_cast<const float4*>(&gis[r][kc * 8]);
            const float4 g1 = *reinterpret_cast<const float4*>(&gis[r][kc * 8 + 4]);
            const float4 l0 = *reinterpret_cast<const float4*>(&gis[C - 1][kc * 8]);
            const float4 l1 = *reinterpret_cast<const float4*>(&gis[C - 1][kc * 8 + 4]);
            float4 e0 = make_float4(0.f, 0.f, 0.f, 0.f), e1 = e0;
            if (r > 0) {
                e0 = *reinterpret_cast<const float4*>(&gis[r - 1][kc * 8]);
                e1 = *reinterpret_cast<const float4*>(&gis[r - 1][kc * 8 + 4]);
            }
            gi[0] = g0.x; gi[1] = g0.y; gi[2] = g0.z; gi[3] = g0.w; gi[4] = g1.x; gi[5] = g1.y; gi[6] = g1.z; gi[7] = g1.w;
            ge[0] = e0.x; ge[1] = e0.y; ge[2] = e0.z; ge[3] = e0.w; ge[4] = e1.x; ge[5] = e1.y; ge[6] = e1.z; ge[7] = e1.w;
            hf[0] = .5f * l0.x; hf[1] = .5f * l0.y; hf[2] = .5f * l0.z; hf[3] = .5f * l0.w;
            hf[4] = .5f * l1.x; hf[5] = .5f * l1.y; hf[6] = .5f * l1.z; hf[7] = .5f * l1.w;
        }
        // positions outside the chunk's tokens or the head's channels hold clamped reads: their factors are zero
        const float mk = (r < valid && kc * 8 < p.Kd) ? 1.f : 0.f;
        float x[8], y[8], ep[8], em[8], ea[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ep[j] = __expf(gi[j] - hf[j]); em[j] = mk * __frcp_rn(ep[j]); ea[j] = mk * __expf(ge[j] - hf[j]);
        }
        t8::unpack8(cur.q, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * (p.scale * mk) * ep[j];
        p.Qh[(size_t)g * CH64 + kc * 64 + r] = t8::pack8(y);
        t8::unpack8(cur.k, x);
        if (AB) {
            const float rn = beta_s[r].z;
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] *= rn;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = x[j] * em[j];
        p.Kh[(size_t)g * CH64 + kc * 64 + r] = t8::pack8(y);
        p.Vc[(size_t)g * CH64 + kc * 64 + r] = (r < valid && kc * 8 < p.Vd) ? cur.v : make_uint4(0, 0, 0, 0);
        if (AB) {   // x still holds this piece of k
            const float4 bs = beta_s[r];
            float a0[8], z[8];
            uint4 c0, c1;
#pragma unroll
            for (int j = 0; j < 8; ++j) { a0[j] = -bs.x * x[j]; y[j] = a0[j] * ea[j]; }
            c0 = t8::pack8(y);
#pragma unroll
            for (int j = 0; j < 8; ++j) { z[j] = __expf(gi[j] - ge[j]); y[j] = a0[j] * (z[j] + bs.y) * ea[j]; }
            c1 = t8::pack8(y);
            sm100::st_global_32B(p.Ah + (size_t)g * CH128 + kc * 128 + r * R, c0, c1);
#pragma unroll
            for (int j = 0; j < 8; ++j) { y[j] = z[j] * x[j] * em[j]; z[j] = x[j] * em[j]; }
            c0 = t8::pack8(y);
            c1 = t8::pack8(z);
            sm100::st_global_32B(p.Bh + (size_t)g * CH128 + kc * 128 + r * R, c0, c1);
            *reinterpret_cast<uint4*>(p.ghat + (size_t)g * C * K + (size_t)r * K + kc * 8) = t8::pack8(ep);
        } else {   // rows 2r, 2r+1 of Ah / Bh are adjacent chunks: one 32-byte store each
            uint4 c0, c1;
            t8::unpack8(cur.a0, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[j] * ea[j];
            c0 = t8::pack8(y);
            t8::unpack8(cur.a1, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[j] * ea[j];
            c1 = t8::pack8(y);
            sm100::st_global_32B(p.Ah + (size_t)g * CH128 + kc * 128 + r * R, c0, c1);
            t8::unpack8(cur.b0, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[j] * em[j];
            c0 = t8::pack8(y);
            t8::unpack8(cur.b1, x);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[j] * em[j];
            c1 = t8::pack8(y);
            sm100::st_global_32B(p.Bh + (size_t)g * CH128 + kc * 128 + r * R, c0, c1);
            // the un-gating factors of the backward pass, e^{gi - half}, in bf16 (their error, 2^-9, is below the
            // rounding of the bf16 gradients they scale)
            *reinterpret_cast<uint4*>(p.ghat + (size_t)g * C * K + (size_t)r * K + kc * 8) = t8::pack8(ep);
        }
        cur = nxt;
        if (tid == 0) TL(2 + it);
    }
    if (tid == 0) TL(12);
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
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, 0), f);              // Aak: columns j < i
#pragma unroll
        for (int cg = 0; cg < 8; ++cg) {
#pragma unroll
            for (int j = 0; j < 8; ++j) if (!((cg * 8 + j) < i)) f[cg * 8 + j] = 0.f;
            p.Aak[g * CH64 + cg * 128 + r] = t8::pack8(f + cg * 8);   // [128 x 64] tile: 8 column groups of 128 rows
        }
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {                      // Aab: column token < row token
            tmem_row64(t8::taddr(tmem, warp, 64 + hh * 64), f);
#pragma unroll
            for (int cg = 0; cg < 8; ++cg) {
#pragma unroll
                for (int j = 0; j < 8; ++j) if (!(((hh * 64 + cg * 8 + j) >> 1) < i)) f[cg * 8 + j] = 0.f;
                p.Aab[g * CH128 + (hh * 8 + cg) * 128 + r] = t8::pack8(f + cg * 8);
            }
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
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, 0), f);              // Aqk: j <= i
#pragma unroll
        for (int cg = 0; cg < 8; ++cg) {
#pragma unroll
            for (int j = 0; j < 8; ++j) if (!((cg * 8 + j) <= i)) f[cg * 8 + j] = 0.f;
            p.Aqk[g * 512 + cg * 64 + i] = t8::pack8(f + cg * 8);
        }
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {                      // Aqb: column token <= i
            tmem_row64(t8::taddr(tmem, warp, 64 + hh * 64), f);
#pragma unroll
            for (int cg = 0; cg < 8; ++cg) {
#pragma unroll
                for (int j = 0; j < 8; ++j) if (!(((hh * 64 + cg * 8 + j) >> 1) <= i)) f[cg * 8 + j] = 0.f;
                p.Aqb[g * CH64 + (hh * 8 + cg) * 64 + i] = t8::pack8(f + cg * 8);
            }
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
    // One 32 KB tile holds L = Aab and, block by block, the inverse that replaces it: a block of L is read for the
    // last time at the level that produces the block of M at the same place (later levels read it only into
    // accumulator rows that are never used).
    // The X blocks of a level (at most 64 x 64 in all) live in the tile's upper right quadrant (rows 0..63, columns
    // 64..127), which is zero in L and in M and which the products read only into accumulator rows that are never
    // used; it is cleared again before M is stored.  32 KB per CTA: seven CTAs per SM.
    uint4* sD = reinterpret_cast<uint4*>(smem);      // 32 KB: L, overwritten by M
    __shared__ __align__(8) uint64_t ld_bar, mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 64); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 32768);
        bulk_g2s(sD, p.Aab + g * CH128, 32768, &ld_bar);
    }
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
    // are computed but never read.  Pair p uses accumulator columns [p bs, (p+1) bs).
    const Tile tD = t8::tile(sD, 128);
    uint32_t phase = 0;
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
        wait_or_flag(&mma_bar, phase, p.status, 6);
        phase ^= 1;
        tc_fence_after();
        const int blk = tid / bs, pr = blk >> 1;                // pr is uniform within a warp
        const bool odd = blk & 1;
        const int rr = tid - blk * bs;
        {
            uint4* xt = sD + (8 + ((pr * bs) >> 3)) * 128;      // rows 0..bs-1, columns 64 + pr bs .. of the tile
            for (int cg = 0; cg < (bs >> 3); ++cg) {
                uint32_t v[8]; float f[8];
                tmem_ld_x8(t8::taddr(tmem, warp, pr * bs + cg * 8), v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
                if (odd) xt[cg * 128 + rr] = t8::pack8(f);
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
        wait_or_flag(&mma_bar, phase, p.status, 7);
        phase ^= 1;
        tc_fence_after();
        {
            const int cg0 = (2 * pr * bs) >> 3;                 // first column group of block J in the full tile
            for (int cg = 0; cg < (bs >> 3); ++cg) {
                uint32_t v[8]; float f[8];
                tmem_ld_x8(t8::taddr(tmem, warp, pr * bs + cg * 8), v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
                if (odd) sD[(cg0 + cg) * 128 + tid] = t8::pack8(f);
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
    }
    for (int e = tid; e < 512; e += 128) sD[(8 + (e >> 6)) * 128 + (e & 63)] = make_uint4(0, 0, 0, 0);    // the quadrant
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
        bulk_s2g(p.M + g * CH128, sD, 32768);
        bulk_commit();
        bulk_wait_read<0>();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 64);
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
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
        for (int cg = 0; cg < 8; ++cg) {
            const uint4 c = t8::pack8(f + cg * 8);
            sP[(hh * 8 + cg) * 128 + tid] = c;
            p.P[g * CH128 + (hh * 8 + cg) * 128 + tid] = c;
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        t8::mma_chain<false, true>(tmem, tM, 0, 0, tP, 0, 0, 128, 128, false);           // u = M P
        umma_commit(&mma_bar);
    }
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {                                                      // Wh while u runs
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, 128 + hh * 64), f);
#pragma unroll
        for (int cg = 0; cg < 8; ++cg) p.W[g * CH128 + (hh * 8 + cg) * 128 + tid] = t8::pack8(f + cg * 8);
    }
    wait_or_flag(&mma_bar, 1, p.status, 10);
    tc_fence_after();
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        float f[64];
        tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
        for (int cg = 0; cg < 8; ++cg) p.U[g * CH128 + (hh * 8 + cg) * 128 + tid] = t8::pack8(f + cg * 8);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------
// K5: inter-chunk state scans, forward and reverse, one kernel
//   forward (HRDPLR/fwd_triton.py:795-968; HRDPLR/naive.py:232-255), per chunk n = 0..NT-1:
//       St = E (.) S ;  v2 = Wh St + u ;  S <- E (.) (St + Kh^T v + Bh^T v2)
//   reverse (HRDPLR/bwd_triton.py:110-222), per chunk n = NT-1..0, dS the gradient of the state
//   leaving the chunk:
//       dSt = E (.) dS ;  dv2 = Bh dSt + dv2_intra ;  dS <- E (.) (dSt + Qh^T dO + Wh^T dv2)
//   and the gradient of the chunk-end log decay, dgl[k] = sum_v dS[k,v] S_{n+1}[k,v]
//   (every term of S_{n+1} carries the factor e^{g_last}; HRDPLR/bwd_triton.py:400,442,457-459).
// Both have the form  T = E(.)X ; Y = A1 T + ADD ; X <- E(.)(T + L1^T R1 + L2^T Y).
// One CTA (8 warps) per (batch, head).  The fp32 state lives in registers: thread (row = lane of
// warp%4, column half = warp/4) owns X[row, 64 columns].  The operands of the next chunk are
// prefetched by bulk copies as soon as the product that reads their buffer has completed.
// ------------------------------------------------------------------------------------------
struct ScanTcP {
    const uint4 *A1, *ADD, *L1, *R1, *L2;   // fwd: Wh, u, Kh, v, Bh      rev: Bh, dv2_intra, Qh, dO, Wh
    const float* E;
    const float* init;                       // fwd: h0, rev: dht (may be null)
    uint4 *CK, *Y;                           // fwd: Hs (St checkpoints), v2     rev: dSt checkpoints, dv2
    float* fin;                              // fwd: final state, rev: dh0 (may be null)
    float* fin2;                             // second copy of the final value (workspace), may be null
    const uint4* Hs;                         // rev only: forward checkpoints, for dgl
    const float* HT;                         // rev only: forward final state
    float* dgl;                              // rev only
    int NT, reverse;
    int* status;
    int add_stride, r1_stride;               // chunk strides of ADD and of L1 / R1 in tiles: 1, or 0 for one shared (zero) tile
                                             // (with R1 = 0 the product L1^T R1 vanishes, so L1 is not fetched either)
    int no_store;                            // 1: do not write CK, Y, dgl (state-only passes)
    int init_identity;                       // 1: start from the K x K identity (transition pass, needs K == V)
    // two-level scan: the chunks of a sequence are cut into nseg segments of seg_len chunks, one CTA each
    // (grid.x = B*H*nseg).  State buffers are then indexed by slot = bh*nseg + seg where *_by_slot is set.
    int nseg, seg_len;
    int init_by_slot, fin_by_slot;
    int fin_last_only;                       // write fin / fin2 only from the segment that ends the scan
    // dual mode (grid.y = 2): CTAs with blockIdx.y == 1 run the transition pass instead (identity start, no
    // inputs) and write their result to fin_transition[slot]
    const uint4* zero_tile;
    float* fin_transition;
    // a launch may cover the segments [seg_off, seg_off + seg_cnt) only (seg_cnt == 0: all of them)
    int seg_off, seg_cnt;
    // lead_real: the CTA of the first segment in scan order (0 forward, nseg-1 reverse) runs the real scan from
    // lead_init (indexed by batch*head, may be null) with stores; its transition twin exits at once
    int lead_real;
    const float* lead_init;
    // head dims of the PUBLIC state tensors (h0 / ht / dht / dh0, [.., Kd, Vd]); states kept in the workspace
    // (the by-slot ones, the transition result and fin2) are always K x V = 128 x 128
    int Kd, Vd;
    // variable-length batches: pair bh = (sequence, head) scans chunks seq_tab[sequence] = (first chunk, chunks) of
    // head h's row of tiles (tile = h * NT + chunk); null for uniform batches (pair bh scans tiles bh * NT ..)
    const int2* seq_tab;
    int H;
};

__global__ void __launch_bounds__(256) scan_tc_kernel(ScanTcP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sA1 = reinterpret_cast<uint4*>(smem);     // 32 KB
    uint4* sADD = sA1 + CH128;                       // 32 KB
    uint4* sL1 = sADD + CH128;                       // 16 KB
    uint4* sR1 = sL1 + CH64;                         // 16 KB
    uint4* sL2 = sR1 + CH64;                         // 32 KB
    uint4* sT = sL2 + CH128;                         // 32 KB  T [k x v]
    uint4* sY = sT + CH128;                          // 32 KB  Y [128 x v]
    __shared__ __align__(8) uint64_t ldA, ldB, barA, barB;
    __shared__ uint32_t tmem_s;
    __shared__ float red[K];
    const int seg_cnt = p.seg_cnt ? p.seg_cnt : p.nseg;
    const int bh = blockIdx.x / seg_cnt, seg = p.seg_off + blockIdx.x % seg_cnt;
    const long long slot = (long long)bh * p.nseg + seg;
    if (p.lead_real && seg == (p.reverse ? p.nseg - 1 : 0)) {
        if (blockIdx.y == 1) return;         // no transition is needed where the entering state is known
        p.init = p.lead_init; p.init_by_slot = 0; p.no_store = 0;
    } else
    if (blockIdx.y == 1) {                   // transition twin of this segment
        p.ADD = p.zero_tile; p.R1 = p.zero_tile; p.L1 = p.zero_tile; p.add_stride = 0; p.r1_stride = 0;
        p.init_identity = 1; p.init = nullptr; p.fin = p.fin_transition; p.fin2 = nullptr;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = (warp & 3) * 32 + lane;
    const int half = warp >> 2;
    TLS(0);
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    long long g0 = (long long)bh * p.NT;
    int NTp = p.NT;                               // chunks of this pair
    if (p.seq_tab) {
        const int2 e = p.seq_tab[bh / p.H];
        g0 = (long long)(bh % p.H) * p.NT + e.x;
        NTp = e.y;
    }
    const int n_lo = seg * p.seg_len, n_hi = min(NTp, n_lo + p.seg_len);
    const int steps = n_hi - n_lo;
    const int n_first = p.reverse ? n_hi - 1 : n_lo, dn = p.reverse ? -1 : 1;
    if (tid == 0) {
        const long long g = g0 + n_first;
        mbar_init(&ldA, 1); mbar_init(&ldB, 1); mbar_init(&barA, 1); mbar_init(&barB, 1); fence_mbar_init();
        // (an empty sequence of a packed batch has no chunk: nothing is requested -- nothing would wait for it and
        //  the CTA must not leave with copies into its shared memory in flight -- and its final state is its initial one)
        if (steps > 0) {
            mbar_expect_tx(&ldA, 65536);
            bulk_g2s(sA1, p.A1 + g * CH128, 32768, &ldA);
            bulk_g2s(sADD, p.ADD + g * p.add_stride * CH128, 32768, &ldA);
            mbar_expect_tx(&ldB, 65536);
            bulk_g2s(sL1, p.L1 + g * p.r1_stride * CH64, 16384, &ldB);
            bulk_g2s(sR1, p.R1 + g * p.r1_stride * CH64, 16384, &ldB);
            bulk_g2s(sL2, p.L2 + g * CH128, 32768, &ldB);
        }
    }
    float S[64];
    if (p.init_identity) {
#pragma unroll
        for (int j = 0; j < 64; ++j) S[j] = (half * 64 + j == row) ? 1.f : 0.f;
    } else if (p.init) {
        const size_t is = p.init_by_slot ? (size_t)slot : (size_t)bh;
        const int kd = p.init_by_slot ? K : p.Kd, vd = p.init_by_slot ? V : p.Vd;
        const float4* src = reinterpret_cast<const float4*>(p.init + (is * kd + row) * vd + half * 64);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float4 x = (row < kd && half * 64 + 4 * j < vd) ? src[j] : make_float4(0.f, 0.f, 0.f, 0.f);
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
    const Tile tA1 = t8::tile(sA1, 128), tL1 = t8::tile(sL1, 64), tR1 = t8::tile(sR1, 64), tL2 = t8::tile(sL2, 128),
               tT = t8::tile(sT, 128), tY = t8::tile(sY, 128);
    float e_next = steps > 0 ? p.E[(size_t)(g0 + n_first) * K + row] : 0.f;
    const bool want_dgl = p.reverse && !p.no_store;
    uint4 hs[8];                                                 // reverse scan: St of the following chunk, for dgl
    float e_hs = 1.f;                                            // ... and that chunk's E
    if (want_dgl && steps > 0 && n_first + 1 < NTp) {            // a segment that does not end the sequence
        e_hs = p.E[(size_t)(g0 + n_first + 1) * K + row];
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) hs[c8] = __ldg(p.Hs + (g0 + n_first + 1) * CH128 + (half * 8 + c8) * 128 + row);
    }
    TLS(1);
    for (int it = 0; it < steps; ++it) {
        if (it >= 1 && it <= 10) TLS(1 + it);
        const int n = n_first + it * dn;
        const long long g = g0 + n;
        const uint32_t ph = it & 1;
        const bool more = it + 1 < steps;
        const float e = e_next;                                  // loaded one chunk ahead: off the critical path
        if (more) e_next = p.E[(size_t)(g + dn) * K + row];
        if (want_dgl && it > 0) {
            // this thread's piece of the forward checkpoint of the chunk AFTER this one (its factor E is the previous
            // step's): requested here, used after the first product is issued -- the pack, the barrier and the issue
            // in between cover most of the round trip
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) hs[c8] = __ldg(p.Hs + (g + 1) * CH128 + (half * 8 + c8) * 128 + row);
        }
        // T = E (.) X  -> operand tile and checkpoint
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = e * S[c8 * 8 + j];
            const uint4 c = t8::pack8(f);
            const int cg = half * 8 + c8;
            sT[cg * 128 + row] = c;
            if (!p.no_store) p.CK[g * CH128 + cg * 128 + row] = c;
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            wait_or_flag(&ldA, ph, p.status, 11);
            tc_fence_after();
            t8::mma_chain<false, true>(tmem, tA1, 0, 0, tT, 0, 0, 128, 128, false);      // A1 T
            umma_commit(&barA);
            // L1^T R1 does not depend on Y: it runs on the tensor pipe while the threads turn A1 T into Y
            wait_or_flag(&ldB, ph, p.status, 14);
            t8::mma_chain<true, true>(tmem + 128, tL1, 0, 0, tR1, 0, 0, 128, 64, false);   // L1^T R1
        }
        float part = 0.f;
        if (p.reverse && !p.no_store) {       // dgl = rowsum(dS (.) S_{n+1}), computed while the product runs
            if (n + 1 < NTp) {
                const float inv = 1.f / e_hs;
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                    float f[8];
                    t8::unpack8(hs[c8], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) part = fmaf(S[c8 * 8 + j], f[j] * inv, part);
                }
            } else {
                const float4* src = reinterpret_cast<const float4*>(p.HT + ((size_t)bh * K + row) * V + half * 64);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float4 x = src[j];
                    part = fmaf(S[4 * j], x.x, part); part = fmaf(S[4 * j + 1], x.y, part);
                    part = fmaf(S[4 * j + 2], x.z, part); part = fmaf(S[4 * j + 3], x.w, part);
                }
            }
            if (half == 1) red[row] = part;
            e_hs = e;                                            // the next step's following chunk is this one
        }
        wait_or_flag(&barA, ph, p.status, 12);
        wait_or_flag(&ldA, ph, p.status, 13);         // ADD is read from shared memory below
        tc_fence_after();
        {
            float acc[64];
            tmem_row64(t8::taddr(tmem, warp, half * 64), acc);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                const int cg = half * 8 + c8;
                float u[8];
                t8::unpack8(sADD[cg * 128 + row], u);
#pragma unroll
                for (int j = 0; j < 8; ++j) u[j] += acc[c8 * 8 + j];
                const uint4 c = t8::pack8(u);
                sY[cg * 128 + row] = c;
                if (!p.no_store) p.Y[g * CH128 + cg * 128 + row] = c;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (p.reverse && !p.no_store && half == 0) p.dgl[(size_t)g * K + row] = part + red[row];
        if (tid == 0) {
            if (more) {                                // A1 and ADD buffers are free: prefetch the next chunk's
                mbar_expect_tx(&ldA, 65536);
                bulk_g2s(sA1, p.A1 + (g + dn) * CH128, 32768, &ldA);
                bulk_g2s(sADD, p.ADD + (g + dn) * p.add_stride * CH128, 32768, &ldA);
            }
            tc_fence_after();
            t8::mma_chain<true, true>(tmem + 128, tL2, 0, 0, tY, 0, 0, 128, 128, true);    // + L2^T Y
            umma_commit(&barB);
        }
        wait_or_flag(&barB, ph, p.status, 15);
        tc_fence_after();
        if (tid == 0 && more) {
            mbar_expect_tx(&ldB, 65536);
            bulk_g2s(sL1, p.L1 + (g + dn) * p.r1_stride * CH64, 16384, &ldB);
            bulk_g2s(sR1, p.R1 + (g + dn) * p.r1_stride * CH64, 16384, &ldB);
            bulk_g2s(sL2, p.L2 + (g + dn) * CH128, 32768, &ldB);
        }
        {
            float acc[64];
            tmem_row64(t8::taddr(tmem, warp, 128 + half * 64), acc);
#pragma unroll
            for (int j = 0; j < 64; ++j) S[j] = e * fmaf(e, S[j], acc[j]);
        }
        tc_fence_before();
    }
    TLS(12);
    const bool ends_scan = p.reverse ? (seg == 0) : (seg == p.nseg - 1);
    if (!p.fin_last_only || ends_scan) {
        const size_t fs = p.fin_by_slot ? (size_t)slot : (size_t)bh;
        const int kd = p.fin_by_slot ? K : p.Kd, vd = p.fin_by_slot ? V : p.Vd;
        const size_t off = (fs * kd + row) * vd + half * 64;
        const size_t off2 = ((size_t)bh * K + row) * V + half * 64;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float4 x = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
            if (p.fin && row < kd && half * 64 + 4 * j < vd) reinterpret_cast<float4*>(p.fin + off)[j] = x;
            if (p.fin2) reinterpret_cast<float4*>(p.fin2 + off2)[j] = x;
        }
    }
    __syncthreads();
    TLS(13);
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------
// backward through the WY representation, one kernel per chunk   (HRDPLR/bwd_triton.py:489-612)
//   dWh = dv2 St^T ; dP = M^T dv2 ; dAak = smask(dP v^T) ; dM = dv2 P^T + dWh Ah^T ;
//   dAab = smask(M^T dM M^T)
// Six operand tiles are loaded once (176 KB); dWh, dP, dM and M^T dM are produced as bf16 operand
// tiles in shared memory (over buffers whose contents are no longer needed) and feed the next
// product directly, so only dWh, dP, dAak and dAab go back to HBM.
// ------------------------------------------------------------------------------------------
struct WyBwdP {
    const uint4 *M, *DV2, *Hs, *Vc, *P, *Ah;
    uint4 *dW, *dP, *dAak, *dAab;
    int* status;
    long long G;           // number of tiles; the grid is persistent
};

// Persistent: one CTA per SM walks over the tiles g = blockIdx.x, blockIdx.x + gridDim.x, ...  The 208 KB of operand
// slots leave no room for a second CTA, so the next tile's operands are requested as soon as the slot they go to has
// been read for the last time (St, v, Ah after phase 2, dv2 after phase 3, M and P after phase 4): the loads of tile
// n+1 run under phases 3 and 4 of tile n.
__global__ void __launch_bounds__(128) wy_bwd_tc_kernel(WyBwdP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* bM = reinterpret_cast<uint4*>(smem);      // M
    uint4* bDV2 = bM + CH128;                        // dv2, later dM
    uint4* bHs = bDV2 + CH128;                       // St, later dWh
    uint4* bP = bHs + CH128;                         // P, later M^T dM
    uint4* bAh = bP + CH128;                         // Ah
    uint4* bdP = bAh + CH128;                        // dP
    uint4* bVc = bdP + CH128;                        // v  [64 x 128]
    __shared__ __align__(8) uint64_t ld1, ld2, mma_bar;
    __shared__ uint32_t tmem_s;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld1, 1); mbar_init(&ld2, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        const long long g = blockIdx.x;
        if (g < p.G) {
            mbar_expect_tx(&ld1, 98304);
            bulk_g2s(bDV2, p.DV2 + g * CH128, 32768, &ld1);
            bulk_g2s(bHs, p.Hs + g * CH128, 32768, &ld1);
            bulk_g2s(bM, p.M + g * CH128, 32768, &ld1);
            mbar_expect_tx(&ld2, 81920);
            bulk_g2s(bVc, p.Vc + g * CH64, 16384, &ld2);
            bulk_g2s(bP, p.P + g * CH128, 32768, &ld2);
            bulk_g2s(bAh, p.Ah + g * CH128, 32768, &ld2);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const Tile tM = t8::tile(bM, 128), tDV2 = t8::tile(bDV2, 128), tHs = t8::tile(bHs, 128), tP = t8::tile(bP, 128),
               tAh = t8::tile(bAh, 128), tdP = t8::tile(bdP, 128), tVc = t8::tile(bVc, 64);
    const int r = tid;
    float f[64];
    uint32_t it = 0;
    for (long long g = blockIdx.x; g < p.G; g += gridDim.x, ++it) {
        const uint32_t ph = it & 1;
        const long long gn = g + gridDim.x;              // next tile of this CTA
        const bool more = gn < p.G;
        // ---- phase 1: dWh = dv2 St^T (cols 0..127), dP = M^T dv2 (cols 128..255)
        wait_or_flag(&ld1, ph, p.status, 30);
        if (tid == 0) {
            tc_fence_after();
            t8::mma_chain<false, false>(tmem, tDV2, 0, 0, tHs, 0, 0, 128, 128, false);
            t8::mma_chain<true, true>(tmem + 128, tM, 0, 0, tDV2, 0, 0, 128, 128, false);
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, 0, p.status, 31);
        tc_fence_after();
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
            tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                const uint4 c = t8::pack8(f + c8 * 8);
                bHs[(hh * 8 + c8) * 128 + r] = c;                       // dWh replaces St
                p.dW[g * CH128 + (hh * 8 + c8) * 128 + r] = c;
            }
            tmem_row64(t8::taddr(tmem, warp, 128 + hh * 64), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                const uint4 c = t8::pack8(f + c8 * 8);
                bdP[(hh * 8 + c8) * 128 + r] = c;
                p.dP[g * CH128 + (hh * 8 + c8) * 128 + r] = c;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- phase 2: dAak = dP v^T (cols 0..63), dM = dv2 P^T + dWh Ah^T (cols 128..255)
        wait_or_flag(&ld2, ph, p.status, 32);
        if (tid == 0) {
            tc_fence_after();
            t8::mma_chain<false, false>(tmem, tdP, 0, 0, tVc, 0, 0, 64, 128, false);
            t8::mma_chain<false, false>(tmem + 128, tDV2, 0, 0, tP, 0, 0, 128, 128, false);
            t8::mma_chain<false, false>(tmem + 128, tHs, 0, 0, tAh, 0, 0, 128, 128, true);
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, 1, p.status, 33);
        tc_fence_after();
        if (tid == 0 && more) {                          // St, v, Ah slots have been read for the last time
            mbar_expect_tx(&ld1, 98304);
            bulk_g2s(bHs, p.Hs + gn * CH128, 32768, &ld1);
            mbar_expect_tx(&ld2, 81920);
            bulk_g2s(bVc, p.Vc + gn * CH64, 16384, &ld2);
            bulk_g2s(bAh, p.Ah + gn * CH128, 32768, &ld2);
        }
        {
            const int i = r >> 1;
            tmem_row64(t8::taddr(tmem, warp, 0), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) if (!((c8 * 8 + j) < i)) f[c8 * 8 + j] = 0.f;
                p.dAak[g * CH64 + c8 * 128 + r] = t8::pack8(f + c8 * 8);
            }
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {
                tmem_row64(t8::taddr(tmem, warp, 128 + hh * 64), f);
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) bDV2[(hh * 8 + c8) * 128 + r] = t8::pack8(f + c8 * 8);   // dM replaces dv2
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- phase 3: tmp = M^T dM
        if (tid == 0) {
            tc_fence_after();
            t8::mma_chain<true, true>(tmem, tM, 0, 0, tDV2, 0, 0, 128, 128, false);
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, 0, p.status, 34);
        tc_fence_after();
        if (tid == 0 && more) bulk_g2s(bDV2, p.DV2 + gn * CH128, 32768, &ld1);     // dM has been consumed
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
            tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) bP[(hh * 8 + c8) * 128 + r] = t8::pack8(f + c8 * 8);         // tmp replaces P
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- phase 4: dAab = smask(tmp M^T)
        if (tid == 0) {
            tc_fence_after();
            t8::mma_chain<false, false>(tmem + 128, tP, 0, 0, tM, 0, 0, 128, 128, false);
            umma_commit(&mma_bar);
        }
        wait_or_flag(&mma_bar, 1, p.status, 35);
        tc_fence_after();
        if (tid == 0 && more) {                          // M and tmp have been consumed
            bulk_g2s(bM, p.M + gn * CH128, 32768, &ld1);
            bulk_g2s(bP, p.P + gn * CH128, 32768, &ld2);
        }
        {
            const int i = r >> 1;
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {
                tmem_row64(t8::taddr(tmem, warp, 128 + hh * 64), f);
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) if (!(((hh * 64 + c8 * 8 + j) >> 1) < i)) f[c8 * 8 + j] = 0.f;
                    p.dAab[g * CH128 + (hh * 8 + c8) * 128 + r] = t8::pack8(f + c8 * 8);
                }
            }
        }
        // the accumulators are read; the next tile's first products overwrite them
        tc_fence_before();
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------
// backward, first stage (HRDPLR/bwd_triton.py:17-105), one kernel per chunk:
//   dAqk = tril(dO v^T), dAqb = mask(dO v2^T), dv2_intra = Aqb^T dO
// dO is read from the public [B,T,H,V] tensor, laid out as a C8 tile in shared memory (and stored
// for the later stages); v, v2 and Aqb arrive by bulk copy.
// ------------------------------------------------------------------------------------------
struct DauP {
    const __nv_bfloat16* d_o;
    const uint4 *Vc, *V2, *Aqb;
    uint4 *dOc, *dAqk, *dAqb, *DV2;
    int T, H, NT;
    int* status;
    int Vd;
    const int2* chunk_tab;
};

__global__ void __launch_bounds__(128) dau_tc_kernel(DauP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sdO = reinterpret_cast<uint4*>(smem);     // 16 KB [64 x 128]
    uint4* sAqb = sdO + CH64;                        // 16 KB [64 x 128]
    uint4* sVc = sAqb + CH64;                        // 16 KB [64 x 128]
    uint4* sV2 = sVc + CH64;                         // 32 KB [128 x 128]
    __shared__ __align__(8) uint64_t ld_bar, mma_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (warp == 0) { tmem_alloc(&tmem_s, 256); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&mma_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 65536);
        bulk_g2s(sAqb, p.Aqb + g * CH64, 16384, &ld_bar);
        bulk_g2s(sVc, p.Vc + g * CH64, 16384, &ld_bar);
        bulk_g2s(sV2, p.V2 + g * CH128, 32768, &ld_bar);
    }
    {
        const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
        const int b = bh / p.H, h = bh % p.H;
        int t0, valid;
        chunk_tokens(p.chunk_tab, n, p.T, t0, valid);
        uint4 c[8];                                    // all eight loads in flight before the first store
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int blk = warp * 8 + it;
            const int r = (blk >> 2) * 8 + (lane & 7);
            const int kc = (blk & 3) * 4 + (lane >> 3);
            const int t = t0 + r;
            c[it] = make_uint4(0, 0, 0, 0);
            if (r < valid && kc * 8 < p.Vd)
                c[it] = __ldg(reinterpret_cast<const uint4*>(p.d_o + (((size_t)b * p.T + t) * p.H + h) * p.Vd + kc * 8));
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int blk = warp * 8 + it;
            const int r = (blk >> 2) * 8 + (lane & 7);
            const int kc = (blk & 3) * 4 + (lane >> 3);
            sdO[kc * 64 + r] = c[it];
            p.dOc[g * CH64 + kc * 64 + r] = c[it];
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const Tile tdO = t8::tile(sdO, 64), tAqb = t8::tile(sAqb, 64), tVc = t8::tile(sVc, 64), tV2 = t8::tile(sV2, 128);
    wait_or_flag(&ld_bar, 0, p.status, 50);
    if (tid == 0) {
        t8::mma_chain<false, false>(tmem, tdO, 0, 0, tV2, 0, 0, 128, 128, false);        // dO v2^T
        t8::mma_chain<true, true>(tmem + 128, tAqb, 0, 0, tdO, 0, 0, 128, 64, false);    // Aqb^T dO
        umma_commit(&mma_bar);
    }
    wait_or_flag(&mma_bar, 0, p.status, 51);
    tc_fence_after();
    float f[64];
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        if (warp < 2) {
            tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) if (!(((hh * 64 + c8 * 8 + j) >> 1) <= tid)) f[c8 * 8 + j] = 0.f;
                p.dAqb[g * CH64 + (hh * 8 + c8) * 64 + tid] = t8::pack8(f + c8 * 8);
            }
        }
        tmem_row64(t8::taddr(tmem, warp, 128 + hh * 64), f);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) p.DV2[g * CH128 + (hh * 8 + c8) * 128 + tid] = t8::pack8(f + c8 * 8);
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after();
        t8::mma_chain<false, false>(tmem, tdO, 0, 0, tVc, 0, 0, 64, 128, false);         // dO v^T
        umma_commit(&mma_bar);
    }
    wait_or_flag(&mma_bar, 1, p.status, 52);
    tc_fence_after();
    if (warp < 2) {
        tmem_row64(t8::taddr(tmem, warp, 0), f);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) if (!((c8 * 8 + j) <= tid)) f[c8 * 8 + j] = 0.f;
            p.dAqk[g * 512 + c8 * 64 + tid] = t8::pack8(f + c8 * 8);
        }
    }
    tc_fence_before();
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
    int Vd;
    const int2* chunk_tab;
};

__global__ void __launch_bounds__(128) out_tc_kernel(OutP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // 72 KB, three CTAs per SM: the operands of the last product (Aqb, v2) take the place of the first
    // product's (Qh, St) once that has completed; the other CTAs on the SM cover the extra round trip.
    uint4* sQ = reinterpret_cast<uint4*>(smem);      // 16 KB [64 x 128]  Qh, then Aqb
    uint4* sH = sQ + CH64;                           // 32 KB [128 x 128] St, then v2
    uint4* sAqk = sH + CH128;                        //  8 KB [64 x 64]
    uint4* sV = sAqk + 512;                          // 16 KB [64 x 128]
    __shared__ __align__(8) uint64_t ld_bar, ld2_bar, mma_bar, mma2_bar;
    __shared__ uint32_t tmem_s;
    const long long g = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (warp == 0) { tmem_alloc(&tmem_s, 128); tmem_relinquish(); }
    if (tid == 0) {
        mbar_init(&ld_bar, 1); mbar_init(&ld2_bar, 1); mbar_init(&mma_bar, 1); mbar_init(&mma2_bar, 1); fence_mbar_init();
        mbar_expect_tx(&ld_bar, 16384 + 32768 + 8192 + 16384);
        bulk_g2s(sQ, p.Qh + g * CH64, 16384, &ld_bar);
        bulk_g2s(sH, p.Hs + g * CH128, 32768, &ld_bar);
        bulk_g2s(sAqk, p.Aqk + g * 512, 8192, &ld_bar);
        bulk_g2s(sV, p.Vc + g * CH64, 16384, &ld_bar);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    if (tid == 0) {
        // the three A operands have 64 rows; lanes 64..127 of the accumulator are never read
        wait_or_flag(&ld_bar, 0, p.status, 16);
        t8::mma_chain<false, true>(tmem, t8::tile(sQ, 64), 0, 0, t8::tile(sH, 128), 0, 0, 128, 128, false);
        t8::mma_chain<false, true>(tmem, t8::tile(sAqk, 64), 0, 0, t8::tile(sV, 64), 0, 0, 128, 64, true);
        umma_commit(&mma_bar);
        wait_or_flag(&mma_bar, 0, p.status, 17);
        mbar_expect_tx(&ld2_bar, 16384 + 32768);
        bulk_g2s(sQ, p.Aqb + g * CH64, 16384, &ld2_bar);
        bulk_g2s(sH, p.V2 + g * CH128, 32768, &ld2_bar);
        wait_or_flag(&ld2_bar, 0, p.status, 18);
        tc_fence_after();
        t8::mma_chain<false, true>(tmem, t8::tile(sQ, 64), 0, 0, t8::tile(sH, 128), 0, 0, 128, 128, true);
        umma_commit(&mma2_bar);
    }
    if (warp < 2) wait_idle_or_flag(&mma2_bar, 0, p.status, 19);
    tc_fence_after();
    if (warp < 2) {
        const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
        const int b = bh / p.H, h = bh % p.H;
        int t0, valid;
        chunk_tokens(p.chunk_tab, n, p.T, t0, valid);
        const int t = t0 + tid;
        uint4* dst = reinterpret_cast<uint4*>(p.o + (((size_t)b * p.T + t) * p.H + h) * p.Vd);
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
            float f[64];
            tmem_row64(t8::taddr(tmem, warp, hh * 64), f);
            if (tid < valid) {
                // whole 32-byte sectors per lane (lanes are 4 KB apart) where the rows of o start on 32-byte
                // boundaries, i.e. V is a multiple of 16; rows of V = 8, 24, 40, ... elements start on odd multiples
                // of 16 bytes and take 16-byte stores
                const bool rows_32B = p.Vd % 16 == 0;
#pragma unroll
                for (int cg = 0; cg < 8; cg += 2) {
                    const int col = (hh * 8 + cg) * 8;
                    if (rows_32B && col + 16 <= p.Vd) {
                        sm100::st_global_32B(dst + hh * 8 + cg, t8::pack8(f + cg * 8), t8::pack8(f + cg * 8 + 8));
                    } else {
                        if (col < p.Vd) dst[hh * 8 + cg] = t8::pack8(f + cg * 8);
                        if (col + 8 < p.Vd) dst[hh * 8 + cg + 1] = t8::pack8(f + cg * 8 + 8);
                    }
                }
            }
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

// ------------------------------------------------------------------------------------------
// backward, last stage: gradients of the hat operands, dv, un-gating and dgk in one kernel
//   (HRDPLR/bwd_triton.py: dv 227-290, bwd_o 295-487, score-gradient applications of intra 761-827,
//    un-gating 854-880, dgk 885-947)
// Five products, all evaluated transposed so that the accumulator lane is the channel k (or v):
//   P1 dQh^T = St dO^T   + Kh^T dAqk^T + Bh^T dAqb^T        [k x 64 tokens]
//   P2 dv^T  = dSt^T Kh^T + dO^T Aqk   + dP^T Aak           [v x 64 tokens]
//   P3 dAh^T = dWh^T M   + Kh^T dAak^T + Bh^T dAab^T        [k x 128 rows]
//   P4 dBh^T = dSt V2^T  + Qh^T dAqb   + Ah^T dAab          [k x 128 rows]
//   P5 dKh^T = dSt v^T   + Qh^T dAqk   + Ah^T dAak          [k x 64 tokens]
// They read 18 distinct tiles (416 KB) -- more than shared memory holds -- so the tiles go through
// a fixed slot schedule: five 32 KB slots A..E, three 16 KB slots a..c, two 8 KB slots x, y; a tile
// is loaded (bulk copy) as soon as the product that last read its slot has completed:
//   at the start: St->A dO->a Aqk->y dP->D Aak->E Kh->b dAqk->x Bh->B dAqb->c dSt->C
//   dWh->A once St dO^T is complete, dAak->a once dO^T Aqk is, M->D and dAab->E once dP^T Aak is;
//   Ah->B once Bh^T dAab^T is complete, V2->A, Qh->D.lo, v->D.hi once dWh^T M is.
// Every group of tiles has its own load barrier, and a chain is issued when its own operands have landed.
// All five accumulators stay in TMEM (448 columns). Sixteen epilogue warps un-gate them (dq = scale e^{gi-half}
// dQh, ...) and write every gradient in the public layout (a warp writes 32 adjacent channels of one token)
// as soon as the product is complete -- dv and dq after P1/P2, da after P3, overlapping the later loads --
// and after P4/P5 walk their tokens backwards for dk, db and the running sum of dgk.
// ------------------------------------------------------------------------------------------
struct GradP {
    const uint4 *Hs, *Bh, *dOc, *Kh, *dAqb, *dAqk, *DE, *dP, *Aak, *Aqk, *dW, *M, *dAab, *dAak, *V2, *Ah, *Qh, *Vc;
    const __nv_bfloat16* ghat;            // e^{gi - half}, bf16 [64][128] per tile
    const float *E, *dgl;                 // e^{half} per (tile, channel); dgL from the reverse scan
    __nv_bfloat16 *dq, *dk, *dv, *da, *db;
    void* dgk;
    float scale;
    int T, H, NT, gdt;
    int* status;
    long long G;           // number of tiles; the grid is persistent
    int Kd, Vd;            // head dims of the public tensors (channels beyond them are padding and are not written)
    const int2* chunk_tab;
};

template <bool A_MN, bool B_MN>
__device__ __forceinline__ void chain0(uint32_t tm, Tile A, Tile B, int N, int kdim, bool acc) {
    t8::mma_chain<A_MN, B_MN>(tm, A, 0, 0, B, 0, 0, N, kdim, acc);
}

__global__ void __launch_bounds__(544) grad_tc_kernel(GradP p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint4* sA = reinterpret_cast<uint4*>(smem);          // 32 KB slots
    uint4* sB = sA + CH128;
    uint4* sC = sB + CH128;
    uint4* sD = sC + CH128;
    uint4* sE = sD + CH128;
    uint4* sa = sE + CH128;                              // 16 KB slots
    uint4* sb = sa + CH64;
    uint4* sc = sb + CH64;
    uint4* sx = sc + CH64;                               // 8 KB slots
    uint4* sy = sx + 512;
    // load barriers (one per group of tiles that a chain waits for) and commit barriers (chains or whole products)
    __shared__ __align__(8) uint64_t ld[13], mc1, mc5, mc6, mc7, mc9, m1, m2, m3, m4;
    enum { T_StdO, T_Aqk, T_dPAak, T_KhdAqk, T_BhdAqb, T_dSt, T_dW, T_dAak, T_M, T_dAab, T_V2, T_QhVc, T_Ah };
    __shared__ uint32_t tmem_s;
    const int tid = threadIdx.x, warp = tid >> 5;
    const bool producer = tid == 512;                   // lane 0 of the seventeenth warp loads tiles and issues MMAs
    if (warp == 0) { tmem_alloc(&tmem_s, 512); tmem_relinquish(); }
    if (producer) {
#pragma unroll
        for (int i = 0; i < 13; ++i) mbar_init(&ld[i], 1);
        mbar_init(&mc1, 1); mbar_init(&mc5, 1); mbar_init(&mc6, 1); mbar_init(&mc7, 1); mbar_init(&mc9, 1);
        mbar_init(&m1, 1); mbar_init(&m2, 1); mbar_init(&m3, 1); mbar_init(&m4, 1);
        fence_mbar_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    // TMEM columns: dQh^T 0..63, dv^T 64..127, dAh^T 128..255, dBh^T 256..383, dKh^T 384..447
    uint32_t it = 0;
#pragma unroll 1
    for (long long g = blockIdx.x; g < p.G; g += gridDim.x, ++it) {
    const uint32_t ph = it & 1;
    if (producer) {
        TL(0);
        // first loads, in the order the chains need them (the chain that frees two slots for the next
        // generation of tiles comes first)
        mbar_expect_tx(&ld[T_dPAak], 32768 + 16384);
        bulk_g2s(sD, p.dP + g * CH128, 32768, &ld[T_dPAak]);
        bulk_g2s(sE, p.Aak + g * CH64, 16384, &ld[T_dPAak]);
        mbar_expect_tx(&ld[T_StdO], 32768 + 16384);
        bulk_g2s(sA, p.Hs + g * CH128, 32768, &ld[T_StdO]);
        bulk_g2s(sa, p.dOc + g * CH64, 16384, &ld[T_StdO]);
        mbar_expect_tx(&ld[T_Aqk], 8192);
        bulk_g2s(sy, p.Aqk + g * 512, 8192, &ld[T_Aqk]);
        mbar_expect_tx(&ld[T_KhdAqk], 16384 + 8192);
        bulk_g2s(sb, p.Kh + g * CH64, 16384, &ld[T_KhdAqk]);
        bulk_g2s(sx, p.dAqk + g * 512, 8192, &ld[T_KhdAqk]);
        mbar_expect_tx(&ld[T_BhdAqb], 32768 + 16384);
        bulk_g2s(sB, p.Bh + g * CH128, 32768, &ld[T_BhdAqb]);
        bulk_g2s(sc, p.dAqb + g * CH64, 16384, &ld[T_BhdAqb]);
        mbar_expect_tx(&ld[T_dSt], 32768);
        bulk_g2s(sC, p.DE + g * CH128, 32768, &ld[T_dSt]);
        // Chains are issued as soon as their own tiles have landed, and the chains that read a slot for the last
        // time are issued first and committed on their own, so that the slot is refilled while the rest of the
        // product still runs.
        wait_or_flag(&ld[T_dPAak], ph, p.status, 72);
        chain0<true, true>(tmem + 64, t8::tile(sD, 128), t8::tile(sE, 128), 64, 128, false);      // P2: dP^T Aak
        umma_commit(&mc6);                                                                        // slots D, E free
        wait_or_flag(&ld[T_StdO], ph, p.status, 70);
        chain0<false, false>(tmem, t8::tile(sA, 128), t8::tile(sa, 64), 64, 128, false);          // P1: St dO^T
        umma_commit(&mc1);                                                                        // slot A free
        wait_or_flag(&ld[T_Aqk], ph, p.status, 71);
        chain0<true, true>(tmem + 64, t8::tile(sa, 64), t8::tile(sy, 64), 64, 64, true);          // P2: dO^T Aqk
        umma_commit(&mc5);                                                                        // slots a, y free
        wait_or_flag(&mc6, ph, p.status, 77);
        mbar_expect_tx(&ld[T_M], 32768);
        bulk_g2s(sD, p.M + g * CH128, 32768, &ld[T_M]);
        mbar_expect_tx(&ld[T_dAab], 32768);
        bulk_g2s(sE, p.dAab + g * CH128, 32768, &ld[T_dAab]);
        wait_or_flag(&mc1, ph, p.status, 73);
        mbar_expect_tx(&ld[T_dW], 32768);
        bulk_g2s(sA, p.dW + g * CH128, 32768, &ld[T_dW]);
        wait_or_flag(&ld[T_KhdAqk], ph, p.status, 74);
        chain0<true, false>(tmem, t8::tile(sb, 64), t8::tile(sx, 64), 64, 64, true);              // P1: Kh^T dAqk^T
        wait_or_flag(&mc5, ph, p.status, 75);
        mbar_expect_tx(&ld[T_dAak], 16384);
        bulk_g2s(sa, p.dAak + g * CH64, 16384, &ld[T_dAak]);
        wait_or_flag(&ld[T_BhdAqb], ph, p.status, 76);
        chain0<true, false>(tmem, t8::tile(sB, 128), t8::tile(sc, 64), 64, 128, true);            // P1: Bh^T dAqb^T
        umma_commit(&m1);
        wait_or_flag(&ld[T_dSt], ph, p.status, 78);
        chain0<true, false>(tmem + 64, t8::tile(sC, 128), t8::tile(sb, 64), 64, 128, true);       // P2: dSt^T Kh^T
        umma_commit(&m2);
        TL(4);
        wait_or_flag(&ld[T_dAab], ph, p.status, 79);
        chain0<true, false>(tmem + 128, t8::tile(sB, 128), t8::tile(sE, 128), 128, 128, false);   // P3: Bh^T dAab^T
        umma_commit(&mc9);                                                                        // slot B free
        wait_or_flag(&ld[T_dW], ph, p.status, 80);
        wait_or_flag(&ld[T_M], ph, p.status, 81);
        chain0<true, true>(tmem + 128, t8::tile(sA, 128), t8::tile(sD, 128), 128, 128, true);     // P3: dWh^T M
        umma_commit(&mc7);                                                                        // slots A, D free
        wait_or_flag(&ld[T_dAak], ph, p.status, 82);
        chain0<true, false>(tmem + 128, t8::tile(sb, 64), t8::tile(sa, 128), 128, 64, true);      // P3: Kh^T dAak^T
        umma_commit(&m3);
        wait_or_flag(&mc9, ph, p.status, 83);
        mbar_expect_tx(&ld[T_Ah], 32768);
        bulk_g2s(sB, p.Ah + g * CH128, 32768, &ld[T_Ah]);
        wait_or_flag(&mc7, ph, p.status, 84);
        TL(6);
        mbar_expect_tx(&ld[T_V2], 32768);
        bulk_g2s(sA, p.V2 + g * CH128, 32768, &ld[T_V2]);
        mbar_expect_tx(&ld[T_QhVc], 16384 + 16384);
        bulk_g2s(sD, p.Qh + g * CH64, 16384, &ld[T_QhVc]);
        bulk_g2s(sD + CH64, p.Vc + g * CH64, 16384, &ld[T_QhVc]);
        wait_or_flag(&ld[T_V2], ph, p.status, 85);
        chain0<false, false>(tmem + 256, t8::tile(sC, 128), t8::tile(sA, 128), 128, 128, false);  // P4: dSt V2^T
        wait_or_flag(&ld[T_QhVc], ph, p.status, 86);
        chain0<false, false>(tmem + 384, t8::tile(sC, 128), t8::tile(sD + CH64, 64), 64, 128, false);  // P5: dSt v^T
        chain0<true, true>(tmem + 256, t8::tile(sD, 64), t8::tile(sc, 64), 128, 64, true);        // P4: Qh^T dAqb
        chain0<true, true>(tmem + 384, t8::tile(sD, 64), t8::tile(sx, 64), 64, 64, true);         // P5: Qh^T dAqk
        wait_or_flag(&ld[T_Ah], ph, p.status, 87);
        TL(7);
        chain0<true, true>(tmem + 256, t8::tile(sB, 128), t8::tile(sE, 128), 128, 128, true);     // P4: Ah^T dAab
        chain0<true, true>(tmem + 384, t8::tile(sB, 128), t8::tile(sa, 128), 64, 128, true);      // P5: Ah^T dAak
        umma_commit(&m4);
        wait_or_flag(&m4, ph, p.status, 88);
        TL(8);
    }
    if (warp < 16) {
        // Sixteen epilogue warps in four token groups: group w owns tokens 48-16w .. 63-16w of the chunk and
        // thread k of a group the channel k.  Everything that does not need the last products runs while the
        // producer is still loading: the decay factors and this thread's Bh elements are fetched from global
        // memory into registers at once, dv and dq are written as soon as P1 and P2 are complete, da after P3;
        // only dk, db and the dgk sums wait for P4 and P5.
        float (*group_total)[K] = reinterpret_cast<float (*)[K]>(sy);      // 2 KB in the (consumed) Aqk slot
        const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
        const int b = bh / p.H, h = bh % p.H;
        const int k = tid & 127, wg = tid >> 7;
        const int i_lo = 48 - 16 * wg;
        int t0, t_left;                                               // first token / tokens of this chunk that exist
        chunk_tokens(p.chunk_tab, n, p.T, t0, t_left);
        const size_t tok_stride = (size_t)p.H * p.Kd;                 // elements between tokens in [B,T,H,K]
        const size_t base_qk = (((size_t)b * p.T + (size_t)t0 + i_lo) * p.H + h) * p.Kd + k;
        const size_t base_ab = (((size_t)b * p.T + (size_t)t0 + i_lo) * R * p.H + h) * p.Kd + k;
        const bool k_ok = k < p.Kd;                                   // this thread's channel exists in the public tensors
        // eg[j] = e^{gi - half} of token i_lo + j - 1 (the token before the chunk has e^{ge - half} = e^{-half})
        float eg[17];
        uint32_t bhp[16];                                             // Bh rows 2i, 2i+1 of this thread's tokens
        {
            const unsigned short* egp = reinterpret_cast<const unsigned short*>(p.ghat + (size_t)g * C * K) + k;
            const float e_half = __ldg(p.E + (size_t)g * K + k);
#pragma unroll
            for (int j = 0; j < 17; ++j)
                eg[j] = (i_lo + j - 1 >= 0) ? __uint_as_float((uint32_t)__ldg(egp + (size_t)(i_lo + j - 1) * K) << 16) : 0.f;
            if (i_lo == 0) eg[0] = __frcp_rn(e_half);        // e^{ge - half} of the chunk's first token
        }
        const float dgl = __ldg(p.dgl + (size_t)g * K + k);
        // ---- after P1: dq
        wait_idle_or_flag(&m1, ph, p.status, 89);
        tc_fence_after();
        {
            uint32_t u[16];
            tmem_ld_x16(t8::taddr(tmem, warp, i_lo), u);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (i_lo + j < t_left && k_ok) p.dq[base_qk + (size_t)j * tok_stride] = __float2bfloat16_rn(p.scale * eg[j + 1] * __uint_as_float(u[j]));
        }
        // ---- after P2: dv (lane = value channel; group w writes tokens 16w..16w+15)
        wait_idle_or_flag(&m2, ph, p.status, 90);
        tc_fence_after();
        {
            uint32_t v[16];
            tmem_ld_x16(t8::taddr(tmem, warp, 64 + wg * 16), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int t = t0 + wg * 16 + j;
                if (wg * 16 + j < t_left && k < p.Vd) p.dv[(((size_t)b * p.T + t) * p.H + h) * p.Vd + k] = __float2bfloat16_rn(__uint_as_float(v[j]));
            }
        }
        // ---- after P3: da = e^{ge-half} dAh
        wait_idle_or_flag(&m3, ph, p.status, 91);
        tc_fence_after();
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            uint32_t v[16];
            tmem_ld_x16(t8::taddr(tmem, warp, 128 + 2 * i_lo + hb * 16), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int jt = hb * 8 + j;
                if (i_lo + jt < t_left && k_ok) {
                    p.da[base_ab + (size_t)(2 * jt) * tok_stride] = __float2bfloat16_rn(eg[jt] * __uint_as_float(v[2 * j]));
                    p.da[base_ab + (size_t)(2 * jt + 1) * tok_stride] = __float2bfloat16_rn(eg[jt] * __uint_as_float(v[2 * j + 1]));
                }
            }
        }
        {   // this thread's Bh elements (L2-resident: the tile was loaded for P1), requested before the wait below
            const unsigned short* bg = reinterpret_cast<const unsigned short*>(p.Bh + g * CH128 + (k >> 3) * 128) + (k & 7);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t lo = __ldg(bg + (size_t)(2 * (i_lo + j)) * 8), hi = __ldg(bg + (size_t)(2 * (i_lo + j) + 1) * 8);
                bhp[j] = lo | (hi << 16);
            }
        }
        // ---- after P4, P5: dk, db and the reverse running sum for dgk
        wait_idle_or_flag(&m4, ph, p.status, 92);
        tc_fence_after();
        if (tid == 0) TL(9);
        // per-thread element pointers into the hat tiles still in shared memory (token i sits 16 bytes after token i-1)
        const __nv_bfloat16* eq = reinterpret_cast<const __nv_bfloat16*>(sD + (k >> 3) * 64) + (k & 7) + i_lo * 8;
        const __nv_bfloat16* ek = reinterpret_cast<const __nv_bfloat16*>(sb + (k >> 3) * 64) + (k & 7) + i_lo * 8;
        const __nv_bfloat16* ea = reinterpret_cast<const __nv_bfloat16*>(sB + (k >> 3) * 128) + (k & 7) + i_lo * 16;
        float run = 0.f;
        float loc[16];                                    // this thread's dgk values before the other groups' totals
#pragma unroll
        for (int hb = 3; hb >= 0; --hb) {                 // four tokens per accumulator read: fewer live registers
            uint32_t vq[4], vk[4], va[8], vb[8];
            tmem_ld_x4(t8::taddr(tmem, warp, i_lo + hb * 4), vq);
            tmem_ld_x4(t8::taddr(tmem, warp, 384 + i_lo + hb * 4), vk);
            tmem_ld_x8(t8::taddr(tmem, warp, 128 + 2 * i_lo + hb * 8), va);
            tmem_ld_x8(t8::taddr(tmem, warp, 256 + 2 * i_lo + hb * 8), vb);
            tmem_wait_ld();
#pragma unroll
            for (int j = 3; j >= 0; --j) {
                const int jt = hb * 4 + j;
                const bool ok = i_lo + jt < t_left && k_ok;
                const float em = __frcp_rn(eg[jt + 1]);
                const float dqh = __uint_as_float(vq[j]), dkh = __uint_as_float(vk[j]);
                const float db0 = __uint_as_float(vb[2 * j]), db1 = __uint_as_float(vb[2 * j + 1]);
                float d_gi = __bfloat162float(eq[jt * 8]) * dqh - __bfloat162float(ek[jt * 8]) * dkh;
                d_gi = fmaf(-__uint_as_float(bhp[jt] << 16), db0, d_gi);
                d_gi = fmaf(-__uint_as_float(bhp[jt] & 0xffff0000u), db1, d_gi);
                float d_ge = __bfloat162float(ea[(2 * jt) * 8]) * __uint_as_float(va[2 * j]);
                d_ge = fmaf(__bfloat162float(ea[(2 * jt + 1) * 8]), __uint_as_float(va[2 * j + 1]), d_ge);
                if (ok) {
                    p.dk[base_qk + (size_t)jt * tok_stride] = __float2bfloat16_rn(em * dkh);
                    p.db[base_ab + (size_t)(2 * jt) * tok_stride] = __float2bfloat16_rn(em * db0);
                    p.db[base_ab + (size_t)(2 * jt + 1) * tok_stride] = __float2bfloat16_rn(em * db1);
                }
                run += d_gi + d_ge;
                loc[jt] = run - d_ge + dgl;
            }
        }
        if (tid == 0) TL(10);
        group_total[wg][k] = run;
        asm volatile("bar.sync 1, 512;" ::: "memory");     // the sixteen epilogue warps only
        if (tid == 0) TL(11);
        float add = 0.f;
        for (int w = 0; w < wg; ++w) add += group_total[w][k];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj)
            if (i_lo + jj < t_left && k_ok) st_elem(p.dgk, base_qk + (size_t)jj * tok_stride, p.gdt, loc[jj] + add);
    }
    // every thread is done with this tile's slots and accumulators before the next tile's first loads and products
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) TL(12);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------
// two-level scan, composition step: the state entering each segment from the per-segment affine maps
//   forward:  Sin[0] = S0,            Sin[s+1] = T[s] Sin[s] + F[s]
//   reverse:  Sin[P-1] = D (dht),     Sin[s-1] = T[s]^T Sin[s] + F[s]        (F = per-segment gradient from zero)
// fp32 CUDA-core products, one CTA per (batch*head, 32 columns); the chain over segments is serial but short.
// ------------------------------------------------------------------------------------------
// With s0_identity the start is the identity and F is ignored (composition of the transitions themselves); `fin`
// (optional) receives the state after the last segment.  With lead_final the first segment in scan order was scanned
// for real: F of that segment is the state entering the next one, and the chain starts there.
// The maps of (pair bh, segment s) are matrix number bh * bh_stride + s * seg_stride of F, Sin (K x V) and matrix
// number bh * t_bh_stride + s * t_seg_stride of T (K x K).
// `pre` (optional, indexed like F) is added to the running state before a segment's map is applied, `post` (optional,
// one K x V matrix per pair) to the final value: with them the same chain serves the gradient of a sequence that is
// cut over ranks, where every rank contributes the gradient of its own final state.
// Layout of the work: one CTA of 256 threads per (pair, 16 state columns) -- 8 CTAs per pair, so even 16 pairs fill
// most SMs -- thread = (state row k, 8 of the 16 columns), its columns in registers.  The K x K transition of a
// segment is staged in shared memory in the orientation the product reads it (element (j, k) at [j][k], pitch 129
// words: conflict-free both for the transposing store of the forward case and for the reads) by coalesced scalar
// loads, all 64 of a thread in flight at once together with its loads of F, so a segment costs one round trip to L2
// plus 128 x 8 fused multiply-adds per thread.
constexpr int kComposeCols = 16;
constexpr int kComposeSmem = (K * 129 + K * (kComposeCols + 4)) * 4;

__global__ void __launch_bounds__(256) compose_segments_kernel(const float* T, const float* F, const float* S0,
                                                               float* Sin, float* fin, int nseg, int reverse,
                                                               int s0_identity, int lead_final, long long bh_stride,
                                                               long long seg_stride, long long t_bh_stride,
                                                               long long t_seg_stride, const float* pre,
                                                               const float* post) {
    constexpr int CB = kComposeCols, CT = 8;                                     // columns per CTA / per thread
    extern __shared__ __align__(16) float csm[];
    float (*sT)[129] = reinterpret_cast<float (*)[129]>(csm);                    // sT[j][k] = factor of cur[j] in row k
    float (*cur)[CB + 4] = reinterpret_cast<float (*)[CB + 4]>(csm + K * 129);   // 16-byte aligned rows: read as float4
    const int bh = blockIdx.x, tid = threadIdx.x;
    const int k = tid & (K - 1), ch = tid >> 7;                                  // row, column half
    const int c0 = blockIdx.y * CB + ch * CT;                                    // first state column of this thread
    const int lane = tid & 31, warp = tid >> 5;
    auto ld8 = [&](const float* base, float* dst) {                              // 8 consecutive floats (32-byte aligned)
        const float4 a = *reinterpret_cast<const float4*>(base), b = *reinterpret_cast<const float4*>(base + 4);
        dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w; dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
    };
    auto st8 = [&](float* base, const float* src) {
        *reinterpret_cast<float4*>(base) = make_float4(src[0], src[1], src[2], src[3]);
        *reinterpret_cast<float4*>(base + 4) = make_float4(src[4], src[5], src[6], src[7]);
    };
    float x[CT];
#pragma unroll
    for (int c = 0; c < CT; ++c) x[c] = s0_identity ? (c0 + c == k ? 1.f : 0.f) : 0.f;
    if (!s0_identity && S0) ld8(S0 + ((size_t)bh * K + k) * V + c0, x);
    const int first = reverse ? nseg - 1 : 0, step = reverse ? -1 : 1;
    if (lead_final) {          // F of the first segment in scan order IS the state leaving it (it was scanned for real)
        const size_t slot = (size_t)(bh * bh_stride + first * seg_stride);
        ld8(F + (slot * K + k) * V + c0, x);
    }
    for (int i = lead_final ? 1 : 0; i < nseg; ++i) {
        const int sgm = first + i * step;
        const size_t slot = (size_t)(bh * bh_stride + sgm * seg_stride);
        const bool apply = i + 1 < nseg || fin;
        float acc[CT];
#pragma unroll
        for (int c = 0; c < CT; ++c) acc[c] = 0.f;
        if (apply) {
            // stage the transition: forward needs T[k][j] at sT[j][k] (transposed), reverse T[j][k] at sT[j][k].
            // Warp w reads rows w, w + 8, ...; a lane reads elements lane, lane + 32, ... of the row.
            const float* Tm = T + (size_t)(bh * t_bh_stride + sgm * t_seg_stride) * K * K;
            float buf[64];
#pragma unroll
            for (int u = 0; u < 16; ++u)
#pragma unroll
                for (int q = 0; q < 4; ++q) buf[u * 4 + q] = __ldg(Tm + (size_t)(warp + 8 * u) * K + q * 32 + lane);
            if (!s0_identity) ld8(F + (slot * K + k) * V + c0, acc);
#pragma unroll
            for (int u = 0; u < 16; ++u)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int r = warp + 8 * u, c = q * 32 + lane;
                    if (reverse) sT[r][c] = buf[u * 4 + q];
                    else sT[c][r] = buf[u * 4 + q];
                }
        }
        if (pre) {
            float pv[CT];
            ld8(pre + (slot * K + k) * V + c0, pv);
#pragma unroll
            for (int c = 0; c < CT; ++c) x[c] += pv[c];
        }
        if (Sin) st8(Sin + (slot * K + k) * V + c0, x);
        st8(&cur[k][ch * CT], x);
        __syncthreads();
        if (apply) {
#pragma unroll 4
            for (int j = 0; j < K; ++j) {
                const float t = sT[j][k];
                const float4 v0 = *reinterpret_cast<const float4*>(&cur[j][ch * CT]);        // the same address for a
                const float4 v1 = *reinterpret_cast<const float4*>(&cur[j][ch * CT + 4]);    // whole warp: a broadcast
                acc[0] = fmaf(t, v0.x, acc[0]); acc[1] = fmaf(t, v0.y, acc[1]);
                acc[2] = fmaf(t, v0.z, acc[2]); acc[3] = fmaf(t, v0.w, acc[3]);
                acc[4] = fmaf(t, v1.x, acc[4]); acc[5] = fmaf(t, v1.y, acc[5]);
                acc[6] = fmaf(t, v1.z, acc[6]); acc[7] = fmaf(t, v1.w, acc[7]);
            }
#pragma unroll
            for (int c = 0; c < CT; ++c) x[c] = acc[c];
        }
        __syncthreads();
    }
    if (fin) {
        if (post) {
            float pv[CT];
            ld8(post + ((size_t)bh * K + k) * V + c0, pv);
#pragma unroll
            for (int c = 0; c < CT; ++c) x[c] += pv[c];
        }
        st8(fin + ((size_t)bh * K + k) * V + c0, x);
    }
}

// A kernel whose only act is a wait that cannot succeed: one CTA waits on an mbarrier nobody arrives at, with a
// budget of `budget_ns`, and records the failure in the status word like every other kernel of the pipeline.
// It exists so that the path from a device-side timeout to the host-side error can be tested without a fault.
__global__ void wait_timeout_probe_kernel(int* status, unsigned long long budget_ns) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(&bar, 0, budget_ns)) atomicExch(status + kStatusWait, 99);
}

constexpr int kGradSmem = 5 * 32768 + 3 * 16384 + 2 * 8192;
constexpr int kWySmem = 6 * 32768 + 16384;

template <typename Kern>
int set_smem(Kern kern, int bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return HDLA_OK;
}

// number of SMs of the current device (grid size of the persistent kernels), cached per host thread and device
int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cached_dev != dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

}  // namespace

int tc_compose_states(const float* T, const float* F, const float* S0, const float* pre, const float* post,
                      float* out, int BH, int count, long long f_stride, long long t_stride, int reverse,
                      cudaStream_t st) {
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        int rc = set_smem(compose_segments_kernel, kComposeSmem);
        if (rc != HDLA_OK) return rc;
        attr_dev = dev;
    }
    launch(compose_segments_kernel, dim3(dim3(BH, V / kComposeCols)), dim3(256), kComposeSmem, st, T, F, S0, nullptr, out, count, reverse,
                                                                                 0, 0, 1, f_stride, 1, t_stride, pre, post);
    HDLA_CHECK_LAUNCH("compose_segments_kernel");
    return HDLA_OK;
}

int tc_wait_timeout_probe(int* status, unsigned long long budget_ns, cudaStream_t st) {
    wait_timeout_probe_kernel<<<1, 32, 0, st>>>(status, budget_ns);
    HDLA_CHECK_LAUNCH("wait_timeout_probe_kernel");
    return HDLA_OK;
}

bool tc_supported(const HdlaDims& d) {
    // head dims below 128 run on the same 128-wide tiles, padded with zeros (multiples of 8: whole 16-byte chunks);
    // phased calls (context parallelism) exchange K x V states between devices and need the full 128 x 128
    const bool dims_ok = d.K % 8 == 0 && d.V % 8 == 0 && d.K >= 8 && d.V >= 8 && d.K <= K && d.V <= V;
    const bool full = d.K == K && d.V == V;
    if ((d.flags & HDLA_PHASE_MASK) != HDLA_PHASE_ALL && (!full || d.cu_seqlens)) return false;
    return d.dtype == HDLA_BF16 && !(d.flags & HDLA_FLAG_FORCE_SIMT) && effective_chunk(d.T, d.C) == C && d.R == R &&
           dims_ok && (long long)d.B * d.H * ((d.T + C - 1) / C) < 0x7fffffffLL;
}

size_t tc_workspace_bytes(const HdlaDims& d, int with_backward) {
    TcPlan pl = make_tc_plan(d);
    return with_backward ? pl.total : pl.total_fwd;
}

#define TRY(x) do { int rc__ = (x); if (rc__ != HDLA_OK) return rc__; } while (0)

int tc_chunk_fwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                 const void* gk, float scale, const float* h0, void* o, float* ht, unsigned char* ws, size_t ws_bytes,
                 bool need_o, cudaStream_t st) {
    const TcPlan pl = make_tc_plan(d);
    // a workspace sized for the backward pass also receives what only the backward kernels read
    const bool save_bwd = ws_bytes >= pl.total;
    const bool param_ab = (d.flags & HDLA_FLAG_PARAM_AB) != 0;
    // the one-kernel form needs full head dims and reads a and b as tensors
    const bool unfused = !(d.flags & HDLA_FLAG_FUSED_PREP) || d.K != K || d.V != V || param_ab;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        TRY(set_smem(gram_tc_kernel, 98304 + 1024));
        TRY(set_smem(inverse_tc_kernel, 32768));
        TRY(set_smem(wu_tc_kernel, 98304));
        TRY(set_smem(scan_tc_kernel, 196608));
        TRY(set_smem(out_tc_kernel, 73728));
        TRY(set_smem(wy_bwd_tc_kernel, kWySmem));
        TRY(set_smem(grad_tc_kernel, kGradSmem));
        TRY(set_smem(dau_tc_kernel, 81920));
        TRY(set_smem(compose_segments_kernel, kComposeSmem));
        attr_dev = dev;
    }
    auto U4 = [&](size_t off) { return reinterpret_cast<uint4*>(ws + off); };
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    int* status = reinterpret_cast<int*>(ws + pl.status);
    const unsigned G = (unsigned)pl.G;
    typedef const __nv_bfloat16* bp;
    const int phase = d.flags & HDLA_PHASE_MASK;
    const int2* chunk_tab = pl.nseq ? reinterpret_cast<const int2*>(ws + pl.chunk_tab) : nullptr;
    const int2* seq_tab = pl.nseq ? reinterpret_cast<const int2*>(ws + pl.seq_tab) : nullptr;
    if (phase == HDLA_PHASE_ALL || phase == HDLA_PHASE_PRE) {
        cudaError_t e = cudaMemsetAsync(ws + pl.status, 0, 256, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(ws + pl.zero, 0, 32768, st);
        if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "workspace clear: %s", cudaGetErrorString(e));
        if (pl.nseq) {
            // packed variable-length batch: which tokens every chunk covers and which chunks every sequence owns.
            // (The source is pageable host memory, which cudaMemcpyAsync stages before it returns.)
            std::vector<int2> chunks, seqs;
            chunks.reserve(pl.NT); seqs.reserve(pl.nseq);
            for (int s_ = 0; s_ < pl.nseq; ++s_) {
                const long long lo = d.cu_seqlens[s_], hi = d.cu_seqlens[s_ + 1];
                seqs.push_back(make_int2((int)chunks.size(), (int)((hi - lo + C - 1) / C)));
                for (long long t = lo; t < hi; t += C) chunks.push_back(make_int2((int)t, (int)(hi - t < C ? hi - t : C)));
            }
            if (!chunks.empty()) e = cudaMemcpyAsync(ws + pl.chunk_tab, chunks.data(), chunks.size() * sizeof(int2), cudaMemcpyHostToDevice, st);
            if (e == cudaSuccess) e = cudaMemcpyAsync(ws + pl.seq_tab, seqs.data(), seqs.size() * sizeof(int2), cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "chunk tables: %s", cudaGetErrorString(e));
            if (pl.G == 0) return HDLA_OK;
        }
        if (!unfused) {
            TRY(tc_launch_chunk_prep(pl, d, q, k, v, a, b, gk, scale, ws, save_bwd, st));
        } else {
            PrepP pp{(bp)q, (bp)k, (bp)v, (bp)a, (bp)b, gk, U4(pl.Qh), U4(pl.Kh), U4(pl.Ah), U4(pl.Bh), U4(pl.Vc),
                     F(pl.E), (__nv_bfloat16*)(ws + pl.ghat), scale, d.T, d.H, pl.NT, d.gk_dtype, status, d.K, d.V, chunk_tab,
                     param_ab ? (bp)a : nullptr, (d.flags & HDLA_FLAG_NORM_K) ? 1 : 0};
            if (param_ab) launch(prep_hat_kernel<true>, dim3(G), dim3(128), 0, st, pp);
            else launch(prep_hat_kernel<false>, dim3(G), dim3(128), 0, st, pp);
            HDLA_CHECK_LAUNCH("prep_hat_kernel");
            GramP gp{U4(pl.Qh), U4(pl.Kh), U4(pl.Ah), U4(pl.Bh), U4(pl.Aqk), U4(pl.Aqb), U4(pl.Aak), U4(pl.Aab), status};
            launch(gram_tc_kernel, dim3(G), dim3(128), 98304 + 1024, st, gp);
            HDLA_CHECK_LAUNCH("gram_tc_kernel");
            InvP ivp{U4(pl.Aab), U4(pl.M), status};
            launch(inverse_tc_kernel, dim3(G), dim3(128), 32768, st, ivp);
            HDLA_CHECK_LAUNCH("inverse_tc_kernel");
            WuP wp{U4(pl.M), U4(pl.Ah), U4(pl.Aak), U4(pl.Vc), U4(pl.P), U4(pl.U), U4(pl.W), status};
            launch(wu_tc_kernel, dim3(G), dim3(128), 98304, st, wp);
            HDLA_CHECK_LAUNCH("wu_tc_kernel");
        }
        if (phase == HDLA_PHASE_PRE) return HDLA_OK;
    }
    auto scan_params = [&](const float* init, uint4* ck, uint4* y, float* fin, float* fin2, int no_store) {
        ScanTcP sp{};
        sp.A1 = U4(pl.W); sp.ADD = U4(pl.U); sp.L1 = U4(pl.Kh); sp.R1 = U4(pl.Vc); sp.L2 = U4(pl.Bh); sp.E = F(pl.E);
        sp.init = init; sp.CK = ck; sp.Y = y; sp.fin = fin; sp.fin2 = fin2;
        sp.NT = pl.NT; sp.reverse = 0; sp.status = status; sp.add_stride = 1; sp.r1_stride = 1; sp.no_store = no_store;
        sp.nseg = 1; sp.seg_len = pl.NT; sp.zero_tile = U4(pl.zero);
        sp.Kd = d.K; sp.Vd = d.V; sp.seq_tab = seq_tab; sp.H = d.H;
        return sp;
    };
    if (phase == HDLA_PHASE_TRANSITION) {
        // chunk transition matrices composed over this call's chunks: state K x K from the identity,
        // no inputs (u = 0, v = 0):  X <- E (.) (I + Bh^T Wh) (E (.) X)
        if (!ht) return fail(HDLA_ERR_INVALID, "transition pass needs the output pointer (ht)");
        if (pl.nseg > 1) {
            // per-segment transitions and states-from-zero side by side, then the product of the transitions;
            // both stay in the workspace for the STATE and POST phases of this sequence slice
            ScanTcP s1 = scan_params(nullptr, nullptr, nullptr, F(pl.Fseg), nullptr, 1);
            s1.nseg = pl.nseg; s1.seg_len = pl.seg_len; s1.fin_by_slot = 1; s1.fin_transition = F(pl.Tseg);
            launch(scan_tc_kernel, dim3(dim3(pl.BH * pl.nseg, 2)), dim3(256), 196608, st, s1);
            HDLA_CHECK_LAUNCH("scan_tc_kernel");
            launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), nullptr, nullptr, ht,
                                                                         pl.nseg, 0, 1, 0, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
            HDLA_CHECK_LAUNCH("compose_segments_kernel");
            return HDLA_OK;
        }
        ScanTcP sp = scan_params(nullptr, nullptr, nullptr, ht, nullptr, 1);
        sp.ADD = U4(pl.zero); sp.R1 = U4(pl.zero); sp.L1 = U4(pl.zero); sp.add_stride = 0; sp.r1_stride = 0;
        sp.init_identity = 1;
        launch(scan_tc_kernel, dim3(pl.BH), dim3(256), 196608, st, sp);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
        return HDLA_OK;
    }
    if (phase == HDLA_PHASE_STATE) {
        if (!ht) return fail(HDLA_ERR_INVALID, "state pass needs the output pointer (ht)");
        if (pl.nseg > 1) {                    // affine maps of the segments are in the workspace (TRANSITION phase)
            launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), h0, nullptr, ht,
                                                                         pl.nseg, 0, 0, 0, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
            HDLA_CHECK_LAUNCH("compose_segments_kernel");
            return HDLA_OK;
        }
        ScanTcP sp = scan_params(h0, nullptr, nullptr, ht, nullptr, 1);
        launch(scan_tc_kernel, dim3(pl.BH), dim3(256), 196608, st, sp);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
        return HDLA_OK;
    }
    if (pl.nseg > 1 && pl.lead_real) {
        // two-level scan of a complete call: the first segment is scanned for real from h0 (checkpoints and v2
        // stored), next to the transition and state-from-zero twins of the segments between it and the last ...
        ScanTcP s1 = scan_params(nullptr, U4(pl.Hs), U4(pl.V2), F(pl.Fseg), nullptr, 1);
        s1.nseg = pl.nseg; s1.seg_len = pl.seg_len; s1.fin_by_slot = 1; s1.fin_transition = F(pl.Tseg);
        s1.seg_off = 0; s1.seg_cnt = pl.nseg - 1; s1.lead_real = 1; s1.lead_init = h0;
        launch(scan_tc_kernel, dim3(dim3(pl.BH * (pl.nseg - 1), 2)), dim3(256), 196608, st, s1);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
        // ... the state entering every later segment follows from the first segment's final state ...
        launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), nullptr, F(pl.Sin), nullptr,
                                                                     pl.nseg, 0, 0, 1, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
        HDLA_CHECK_LAUNCH("compose_segments_kernel");
        // ... and the remaining segments are scanned for real at once
        ScanTcP s2 = scan_params(F(pl.Sin), U4(pl.Hs), U4(pl.V2), ht, F(pl.HT), 0);
        s2.nseg = pl.nseg; s2.seg_len = pl.seg_len; s2.init_by_slot = 1; s2.fin_last_only = 1;
        s2.seg_off = 1; s2.seg_cnt = pl.nseg - 1;
        launch(scan_tc_kernel, dim3(pl.BH * (pl.nseg - 1)), dim3(256), 196608, st, s2);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
    } else     if (pl.nseg > 1) {
        // two-level scan: per segment, transition and state-from-zero side by side (grid.y = 2) ...
        if (phase == HDLA_PHASE_ALL) {        // (a phased POST call finds them in the workspace)
            ScanTcP s1 = scan_params(nullptr, nullptr, nullptr, F(pl.Fseg), nullptr, 1);
            s1.nseg = pl.nseg; s1.seg_len = pl.seg_len; s1.fin_by_slot = 1; s1.fin_transition = F(pl.Tseg);
            launch(scan_tc_kernel, dim3(dim3(pl.BH * pl.nseg, 2)), dim3(256), 196608, st, s1);
            HDLA_CHECK_LAUNCH("scan_tc_kernel");
        }
        // ... composed into the state entering every segment ...
        launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), h0, F(pl.Sin), nullptr, pl.nseg, 0, 0, 0, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
        HDLA_CHECK_LAUNCH("compose_segments_kernel");
        // ... and the real scan of all segments at once
        ScanTcP s2 = scan_params(F(pl.Sin), U4(pl.Hs), U4(pl.V2), ht, F(pl.HT), 0);
        s2.nseg = pl.nseg; s2.seg_len = pl.seg_len; s2.init_by_slot = 1; s2.fin_last_only = 1;
        launch(scan_tc_kernel, dim3(pl.BH * pl.nseg), dim3(256), 196608, st, s2);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
    } else {
        ScanTcP sp = scan_params(h0, U4(pl.Hs), U4(pl.V2), ht, F(pl.HT), 0);
        launch(scan_tc_kernel, dim3(pl.BH), dim3(256), 196608, st, sp);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
    }
    if (need_o) {
        OutP op{U4(pl.Qh), U4(pl.Aqk), U4(pl.Aqb), U4(pl.Vc), U4(pl.Hs), U4(pl.V2), (__nv_bfloat16*)o, d.T, d.H,
                pl.NT, status, d.V, chunk_tab};
        launch(out_tc_kernel, dim3(G), dim3(128), 73728, st, op);
        HDLA_CHECK_LAUNCH("out_tc_kernel");
    }
    return HDLA_OK;
}

int tc_chunk_bwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                 const void* gk, float scale, const float* h0, const void* d_o, const float* dht, void* dq, void* dk,
                 void* dv, void* da, void* db, void* dgk, float* dh0, unsigned char* ws, cudaStream_t st) {
    const int phase = d.flags & HDLA_PHASE_MASK;
    if (phase != HDLA_PHASE_ALL && !(d.flags & HDLA_FLAG_WS_HOLDS_FWD))
        return fail(HDLA_ERR_INVALID, "phased backward calls need HDLA_FLAG_WS_HOLDS_FWD");
    if (!(d.flags & HDLA_FLAG_WS_HOLDS_FWD)) {
        HdlaDims df = d;
        df.flags &= ~HDLA_PHASE_MASK;
        TRY(tc_chunk_fwd(df, q, k, v, a, b, gk, scale, h0, nullptr, nullptr, ws, make_tc_plan(df).total, false, st));
    }
    const TcPlan pl = make_tc_plan(d);
    const bool param_ab = (d.flags & HDLA_FLAG_PARAM_AB) != 0;
    auto U4 = [&](size_t off) { return reinterpret_cast<uint4*>(ws + off); };
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    int* status = reinterpret_cast<int*>(ws + pl.status);
    const unsigned G = (unsigned)pl.G;
    typedef __nv_bfloat16* bp;
    const int2* chunk_tab = pl.nseq ? reinterpret_cast<const int2*>(ws + pl.chunk_tab) : nullptr;
    const int2* seq_tab = pl.nseq ? reinterpret_cast<const int2*>(ws + pl.seq_tab) : nullptr;
    if (pl.nseq && pl.G == 0) return HDLA_OK;

    if (phase == HDLA_PHASE_ALL || phase == HDLA_PHASE_PRE) {
        DauP dp{(const __nv_bfloat16*)d_o, U4(pl.Vc), U4(pl.V2), U4(pl.Aqb), U4(pl.dOc), U4(pl.dAqk), U4(pl.dAqb),
                U4(pl.DV2), d.T, d.H, pl.NT, status, d.V, chunk_tab};
        launch(dau_tc_kernel, dim3(G), dim3(128), 81920, st, dp);
        HDLA_CHECK_LAUNCH("dau_tc_kernel");
        if (phase == HDLA_PHASE_PRE) return HDLA_OK;
    }
    if (phase == HDLA_PHASE_TRANSITION) return fail(HDLA_ERR_INVALID, "the transition pass belongs to the forward call");
    auto rscan_params = [&](const float* init, uint4* ck, uint4* y, float* fin, float* dgl, int no_store) {
        ScanTcP sp{};
        sp.A1 = U4(pl.Bh); sp.ADD = U4(pl.DV2); sp.L1 = U4(pl.Qh); sp.R1 = U4(pl.dOc); sp.L2 = U4(pl.W); sp.E = F(pl.E);
        sp.init = init; sp.CK = ck; sp.Y = y; sp.fin = fin; sp.fin2 = nullptr;
        sp.Hs = U4(pl.Hs); sp.HT = F(pl.HT); sp.dgl = dgl;
        sp.NT = pl.NT; sp.reverse = 1; sp.status = status; sp.add_stride = 1; sp.r1_stride = 1; sp.no_store = no_store;
        sp.nseg = 1; sp.seg_len = pl.NT; sp.zero_tile = U4(pl.zero);
        sp.Kd = d.K; sp.Vd = d.V; sp.seq_tab = seq_tab; sp.H = d.H;
        return sp;
    };
    if (phase == HDLA_PHASE_STATE) {
        // state gradient leaving this call's first chunk for the given incoming dht; nothing is stored
        if (!dh0) return fail(HDLA_ERR_INVALID, "state pass needs the output pointer (dh0)");
        if (pl.nseg > 1) {                    // per-segment gradients from zero, then composed with T^T
            ScanTcP s1 = rscan_params(nullptr, nullptr, nullptr, F(pl.Fseg), nullptr, 1);
            s1.nseg = pl.nseg; s1.seg_len = pl.seg_len; s1.fin_by_slot = 1;
            launch(scan_tc_kernel, dim3(pl.BH * pl.nseg), dim3(256), 196608, st, s1);
            HDLA_CHECK_LAUNCH("scan_tc_kernel");
            launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), dht, nullptr, dh0,
                                                                         pl.nseg, 1, 0, 0, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
            HDLA_CHECK_LAUNCH("compose_segments_kernel");
            return HDLA_OK;
        }
        ScanTcP sp = rscan_params(dht, nullptr, nullptr, dh0, nullptr, 1);
        launch(scan_tc_kernel, dim3(pl.BH), dim3(256), 196608, st, sp);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
        return HDLA_OK;
    }
    // --- dhu: reverse scan (dv2 is accumulated in place over dv2_intra)
    if (pl.nseg > 1 && pl.lead_real) {
        // mirror image of the forward pass of a complete call: the last segment is scanned for real from dht next to
        // the gradient-from-zero twins of the segments 1 .. nseg-2 (their transitions are in the workspace) ...
        ScanTcP s1 = rscan_params(nullptr, U4(pl.DE), U4(pl.DV2), F(pl.Fseg), F(pl.dgl), 1);
        s1.nseg = pl.nseg; s1.seg_len = pl.seg_len; s1.fin_by_slot = 1;
        s1.seg_off = 1; s1.seg_cnt = pl.nseg - 1; s1.lead_real = 1; s1.lead_init = dht;
        launch(scan_tc_kernel, dim3(pl.BH * (pl.nseg - 1)), dim3(256), 196608, st, s1);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
        launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), nullptr, F(pl.Sin), nullptr,
                                                                     pl.nseg, 1, 0, 1, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
        HDLA_CHECK_LAUNCH("compose_segments_kernel");
        ScanTcP s2 = rscan_params(F(pl.Sin), U4(pl.DE), U4(pl.DV2), dh0, F(pl.dgl), 0);
        s2.nseg = pl.nseg; s2.seg_len = pl.seg_len; s2.init_by_slot = 1; s2.fin_last_only = 1;
        s2.seg_off = 0; s2.seg_cnt = pl.nseg - 1;
        launch(scan_tc_kernel, dim3(pl.BH * (pl.nseg - 1)), dim3(256), 196608, st, s2);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
    } else     if (pl.nseg > 1) {
        // two-level reverse scan; the segment transitions were left in the workspace by the forward pass
        if (phase == HDLA_PHASE_ALL) {        // (a phased POST call finds the per-segment gradients in the workspace)
            ScanTcP s1 = rscan_params(nullptr, nullptr, nullptr, F(pl.Fseg), nullptr, 1);
            s1.nseg = pl.nseg; s1.seg_len = pl.seg_len; s1.fin_by_slot = 1;
            launch(scan_tc_kernel, dim3(pl.BH * pl.nseg), dim3(256), 196608, st, s1);
            HDLA_CHECK_LAUNCH("scan_tc_kernel");
        }
        launch(compose_segments_kernel, dim3(dim3(pl.BH, V / kComposeCols)), dim3(256), kComposeSmem, st, F(pl.Tseg), F(pl.Fseg), dht, F(pl.Sin), nullptr, pl.nseg, 1, 0, 0, pl.nseg, 1, pl.nseg, 1, nullptr, nullptr);
        HDLA_CHECK_LAUNCH("compose_segments_kernel");
        ScanTcP s2 = rscan_params(F(pl.Sin), U4(pl.DE), U4(pl.DV2), dh0, F(pl.dgl), 0);
        s2.nseg = pl.nseg; s2.seg_len = pl.seg_len; s2.init_by_slot = 1; s2.fin_last_only = 1;
        launch(scan_tc_kernel, dim3(pl.BH * pl.nseg), dim3(256), 196608, st, s2);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
    } else {
        ScanTcP sp = rscan_params(dht, U4(pl.DE), U4(pl.DV2), dh0, F(pl.dgl), 0);
        launch(scan_tc_kernel, dim3(pl.BH), dim3(256), 196608, st, sp);
        HDLA_CHECK_LAUNCH("scan_tc_kernel");
    }
    // --- wy: dWh, dP, dAak, dAab in one kernel
    WyBwdP wyp{U4(pl.M), U4(pl.DV2), U4(pl.Hs), U4(pl.Vc), U4(pl.P), U4(pl.Ah), U4(pl.dW), U4(pl.dP), U4(pl.dAak),
               U4(pl.dAab), status, (long long)G};
    const unsigned wy_grid = G < (unsigned)sm_count() ? G : (unsigned)sm_count();      // one persistent CTA per SM
    launch(wy_bwd_tc_kernel, dim3(wy_grid), dim3(128), kWySmem, st, wyp);
    HDLA_CHECK_LAUNCH("wy_bwd_tc_kernel");
    // --- everything else: hat-operand gradients, dv, un-gating, dgk
    GradP gp{U4(pl.Hs), U4(pl.Bh), U4(pl.dOc), U4(pl.Kh), U4(pl.dAqb), U4(pl.dAqk), U4(pl.DE), U4(pl.dP), U4(pl.Aak),
             U4(pl.Aqk), U4(pl.dW), U4(pl.M), U4(pl.dAab), U4(pl.dAak), U4(pl.V2), U4(pl.Ah), U4(pl.Qh), U4(pl.Vc),
             (bp)(ws + pl.ghat), F(pl.E), F(pl.dgl), (bp)dq, (bp)dk, (bp)dv, param_ab ? (bp)(ws + pl.dab) : (bp)da,
             param_ab ? (bp)(ws + pl.dab + pl.dab_half) : (bp)db, dgk, scale, d.T, d.H, pl.NT, d.gk_dtype,
             status, (long long)G, d.K, d.V, chunk_tab};
    const unsigned grad_grid = G < (unsigned)sm_count() ? G : (unsigned)sm_count();    // one persistent CTA per SM
    launch(grad_tc_kernel, dim3(grad_grid), dim3(544), kGradSmem, st, gp);
    HDLA_CHECK_LAUNCH("grad_tc_kernel");
    if (param_ab)      // da, db -> dbeta (through the `da` argument), and their shares of dk and dgk = dlog_f added in place
        return param_ab_launch(true, a, k, gk, ws + pl.dab, ws + pl.dab + pl.dab_half, da, dk, dgk, d.B, d.T, d.H, d.K,
                               d.dtype, d.gk_dtype, 1, (d.flags & HDLA_FLAG_NORM_K) ? 1 : 0, st);
    return HDLA_OK;
}

// debugging aid: named bf16 tile buffer of the tensor-core workspace -> fp32 row-major [G][rows][cols]
int tc_debug_buffer(const HdlaDims& d, const unsigned char* ws, const char* name, float* out, cudaStream_t st) {
    const TcPlan pl = make_tc_plan(d);
    struct Ent { const char* n; size_t off; int rows, cols; };
    const Ent tab[] = {{"Qh", pl.Qh, 64, 128}, {"Kh", pl.Kh, 64, 128}, {"Ah", pl.Ah, 128, 128}, {"Bh", pl.Bh, 128, 128},
                       {"Vc", pl.Vc, 64, 128}, {"Aqk", pl.Aqk, 64, 64}, {"Aqb", pl.Aqb, 64, 128},
                       {"Aak", pl.Aak, 128, 64}, {"M", pl.M, 128, 128},
                       {"W", pl.W, 128, 128}, {"P", pl.P, 128, 128}, {"U", pl.U, 128, 128}, {"Hs", pl.Hs, 128, 128},
                       {"V2", pl.V2, 128, 128},
                       {"dOc", pl.dOc, 64, 128}, {"dAqk", pl.dAqk, 64, 64}, {"dAqb", pl.dAqb, 64, 128},
                       {"DV2", pl.DV2, 128, 128}, {"DE", pl.DE, 128, 128}, {"dW", pl.dW, 128, 128},
                       {"dP", pl.dP, 128, 128}, {"dAak", pl.dAak, 128, 64}, {"dAab", pl.dAab, 128, 128}};
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
    if (!strcmp(name, "dgl")) {
        cudaMemcpyAsync(out, ws + pl.dgl, (size_t)pl.G * K * 4, cudaMemcpyDeviceToDevice, st);
        return HDLA_OK;
    }
    if (!strcmp(name, "status")) {
        cudaMemcpyAsync(out, ws + pl.status, 4, cudaMemcpyDeviceToDevice, st);
        return HDLA_OK;
    }
    return fail(HDLA_ERR_INVALID, "unknown debug buffer '%s'", name);
}

}  // namespace hdla

#ifdef HDLA_TIMELINE
extern "C" __attribute__((visibility("default"))) int hdla_debug_timeline_scan(unsigned long long* host_dst, size_t count) {
    return (int)cudaMemcpyFromSymbol(host_dst, hdla::tc::g_timeline_scan, count * sizeof(unsigned long long));
}
extern "C" __attribute__((visibility("default"))) int hdla_debug_timeline(unsigned long long* host_dst, size_t count) {
    return (int)cudaMemcpyFromSymbol(host_dst, hdla::g_timeline, count * sizeof(unsigned long long));
}
#endif
