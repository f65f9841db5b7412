// fp32 CUDA-core pipeline of the chunked HDLA operator (forward and backward).
//
// This is the full-precision path: it serves fp32 inputs (tensor-core operand rounding cannot
// meet a 1e-4 tolerance) and is the on-device reference every tensor-core stage is compared
// with.  It mirrors the reference's stage sequence one to one
//   forward  (HRDPLR/hrdplr.py:25-99):   cumsum+gating -> A matrices -> (I-Aab)^-1 -> w,u -> state scan -> o
//   backward (HRDPLR/hrdplr.py:146-284): dAu -> dhu (reverse scan) -> dv -> bwd_o -> wy -> intra -> dgk
// but keeps every intermediate in fp32, chunk-major and zero padded to whole chunks:
// buffer[(bh*NT + n)][rows][cols] with bh = b*H + h.  Decay-weighted products are evaluated
// with the exponent difference taken per element (exp(g_i - g_j) with g_i <= g_j on the causal
// mask), so no operand is ever scaled by exp(-g) and nothing can overflow however strong the
// decay is.  All dense products go through one batched tile-GEMM routine.
#include "common.cuh"

namespace hdla {
namespace {

// ------------------------------------------------------------------------------------------
// workspace plan
// ------------------------------------------------------------------------------------------
struct Plan {
    int B, T, H, K, V, R, C, m, NT, BH;
    long long G;
    // per chunk-head sizes
    long long CK, CV, mK, mV, CC, Cm, mm, KV;
    // offsets (floats)
    long long qs, kc, vc, ac, bc, g, gi, qg, kg, ag, bg, decay, Aqk, Aqb, Aak, Aab, M, w, P, u, h, v2, oc;
    long long doc, dAqk, dAqb, dv2, dhs, dv, dqg, dkg, dbg, dw, dgl, dP, dAak, dM, tmp, dAab, dag, dqs, dk, da, db;
    long long total_fwd, total;
};

Plan make_plan(const HdlaDims& d) {
    Plan p{};
    p.B = d.B; p.T = d.T; p.H = d.H; p.K = d.K; p.V = d.V; p.R = d.R;
    p.C = effective_chunk(d.T, d.C);
    p.m = p.C * p.R;
    p.NT = (d.T + p.C - 1) / p.C;
    p.BH = d.B * d.H;
    p.G = (long long)p.BH * p.NT;
    p.CK = (long long)p.C * p.K; p.CV = (long long)p.C * p.V; p.mK = (long long)p.m * p.K;
    p.mV = (long long)p.m * p.V; p.CC = (long long)p.C * p.C; p.Cm = (long long)p.C * p.m;
    p.mm = (long long)p.m * p.m; p.KV = (long long)p.K * p.V;
    long long off = 0;
    auto take = [&](long long per_chunk, long long count) {
        long long o = off;
        off += ((per_chunk * count + 63) / 64) * 64;     // keep every buffer 256-byte aligned
        return o;
    };
    const long long G = p.G;
    p.qs = take(p.CK, G); p.kc = take(p.CK, G); p.vc = take(p.CV, G); p.ac = take(p.mK, G); p.bc = take(p.mK, G);
    p.g = take(p.CK, G); p.gi = take(p.CK, G); p.qg = take(p.CK, G); p.kg = take(p.CK, G); p.ag = take(p.mK, G);
    p.bg = take(p.mK, G); p.decay = take(p.K, G); p.Aqk = take(p.CC, G); p.Aqb = take(p.Cm, G);
    p.Aak = take(p.Cm, G); p.Aab = take(p.mm, G); p.M = take(p.mm, G); p.w = take(p.mK, G); p.P = take(p.mV, G);
    p.u = take(p.mV, G); p.h = take(p.KV, (long long)p.BH * (p.NT + 1)); p.v2 = take(p.mV, G);
    p.oc = take(p.CV, G);
    p.total_fwd = off;
    p.doc = take(p.CV, G); p.dAqk = take(p.CC, G); p.dAqb = take(p.Cm, G); p.dv2 = take(p.mV, G);
    p.dhs = take(p.KV, (long long)p.BH * (p.NT + 1)); p.dv = take(p.CV, G); p.dqg = take(p.CK, G);
    p.dkg = take(p.CK, G); p.dbg = take(p.mK, G); p.dw = take(p.mK, G); p.dgl = take(p.K, G);
    p.dP = take(p.mV, G); p.dAak = take(p.Cm, G); p.dM = take(p.mm, G); p.tmp = take(p.mm, G);
    p.dAab = take(p.mm, G); p.dag = take(p.mK, G); p.dqs = take(p.CK, G); p.dk = take(p.CK, G);
    p.da = take(p.mK, G); p.db = take(p.mK, G);
    p.total = off;
    return p;
}

// ------------------------------------------------------------------------------------------
// ingest: inputs -> fp32 chunk-major, chunk-local cumulative log decay, gated operands
//   gi = inclusive cumsum of gk within the chunk, ge = gi - gk (the reference takes both from
//   fla's chunk_rwkv6_fwd_cumsum, call site HRDPLR/hrdplr.py:44; restated in HRDPLR/naive.py:107-108)
//   qg = scale q e^{gi}, kg = k e^{g_last-gi}, ag = a e^{ge}, bg = b e^{g_last-gi}
//   (HRDPLR/fwd_triton.py:222-245)
// ------------------------------------------------------------------------------------------
struct IngestP {
    const void *q, *k, *v, *a, *b, *gk;
    float *qs, *kc, *vc, *ac, *bc, *g, *gi, *qg, *kg, *ag, *bg, *decay;
    float scale;
    int T, H, K, V, R, C, NT, dt, gdt;
};

__global__ void __launch_bounds__(256) ingest_fwd_kernel(IngestP p) {
    const long long g = blockIdx.x;
    const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
    const int b = bh / p.H, h = bh % p.H;
    const int C = p.C, K = p.K, V = p.V, R = p.R;
    const int t0 = n * C;
    const int valid = min(C, p.T - t0);
    for (int col = threadIdx.x; col < K; col += blockDim.x) {
        float run = 0.f;
        for (int i = 0; i < C; ++i) {
            float gv = 0.f, qv = 0.f, kv = 0.f;
            if (i < valid) {
                const size_t src = (((size_t)b * p.T + t0 + i) * p.H + h) * K + col;
                gv = ld_elem(p.gk, src, p.gdt);
                qv = ld_elem(p.q, src, p.dt) * p.scale;
                kv = ld_elem(p.k, src, p.dt);
            }
            run += gv;
            const size_t dst = (size_t)g * C * K + (size_t)i * K + col;
            p.g[dst] = gv; p.gi[dst] = run; p.qs[dst] = qv; p.kc[dst] = kv;
            p.qg[dst] = qv * __expf(run);
            for (int r = 0; r < R; ++r) {
                float av = 0.f, bv = 0.f;
                if (i < valid) {
                    const size_t sa = (((size_t)b * p.T * R + (size_t)(t0 + i) * R + r) * p.H + h) * K + col;
                    av = ld_elem(p.a, sa, p.dt);
                    bv = ld_elem(p.b, sa, p.dt);
                }
                const size_t da = (size_t)g * C * R * K + (size_t)(i * R + r) * K + col;
                p.ac[da] = av; p.bc[da] = bv;
                p.ag[da] = av * __expf(run - gv);
            }
        }
        const float glast = run;
        p.decay[(size_t)g * K + col] = __expf(glast);
        for (int i = 0; i < C; ++i) {
            const size_t dst = (size_t)g * C * K + (size_t)i * K + col;
            const float e = __expf(glast - p.gi[dst]);
            p.kg[dst] = p.kc[dst] * e;
            for (int r = 0; r < R; ++r) {
                const size_t da = (size_t)g * C * R * K + (size_t)(i * R + r) * K + col;
                p.bg[da] = p.bc[da] * e;
            }
        }
    }
    for (int col = threadIdx.x; col < V; col += blockDim.x)
        for (int i = 0; i < C; ++i) {
            float x = 0.f;
            if (i < valid) x = ld_elem(p.v, (((size_t)b * p.T + t0 + i) * p.H + h) * V + col, p.dt);
            p.vc[(size_t)g * C * V + (size_t)i * V + col] = x;
        }
}

// [B,T,H,D] (any dtype) -> chunk-major fp32 (used for dO), and back (used for o)
__global__ void to_chunk_major_kernel(const void* src, float* dst, int T, int H, int D, int C, int NT, int dt) {
    const long long g = blockIdx.x;
    const int bh = (int)(g / NT), n = (int)(g % NT);
    const int b = bh / H, h = bh % H;
    for (int e = threadIdx.x; e < C * D; e += blockDim.x) {
        const int i = e / D, col = e % D;
        const int t = n * C + i;
        dst[(size_t)g * C * D + e] = t < T ? ld_elem(src, (((size_t)b * T + t) * H + h) * D + col, dt) : 0.f;
    }
}
__global__ void from_chunk_major_kernel(const float* src, void* dst, int T, int H, int D, int C, int NT, int dt,
                                        float alpha) {
    const long long g = blockIdx.x;
    const int bh = (int)(g / NT), n = (int)(g % NT);
    const int b = bh / H, h = bh % H;
    for (int e = threadIdx.x; e < C * D; e += blockDim.x) {
        const int i = e / D, col = e % D;
        const int t = n * C + i;
        if (t < T) st_elem(dst, (((size_t)b * T + t) * H + h) * D + col, dt, alpha * src[(size_t)g * C * D + e]);
    }
}

// ------------------------------------------------------------------------------------------
// gated Gram matrices:  A[i,j] = sum_k x[i,k] y[j,k] exp(gx[i,k] - gy[j,k]) on the causal mask
//   Aqk/Aqb use gx = gi (mask j <= i), Aak/Aab use gx = ge (mask j < i)
//   (HRDPLR/naive.py:136-184; reference kernels HRDPLR/fwd_triton.py:13-290 and :295-514)
// ------------------------------------------------------------------------------------------
struct GramP {
    const float *x, *y, *gi, *g;
    float* out;
    int mx, ny, rx, ry, K, C, excl;      // excl: row gate is ge (strict mask) instead of gi
};

__global__ void __launch_bounds__(256) gated_gram_kernel(GramP p) {
    constexpr int KB = 64;
    __shared__ float xs[16][KB + 1], gxs[16][KB + 1], ys[16][KB + 1], gys[16][KB + 1];
    const long long g = blockIdx.z;
    const int i0 = blockIdx.y * 16, j0 = blockIdx.x * 16;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int i = i0 + ty, j = j0 + tx;
    const bool in = i < p.mx && j < p.ny;
    const int ti = i / p.rx, tj = j / p.ry;
    const bool keep = in && (p.excl ? (tj < ti) : (tj <= ti));
    // the whole tile is masked when its largest row token is below its smallest column token
    const int ti_max = min(i0 + 15, p.mx - 1) / p.rx, tj_min = j0 / p.ry;
    const bool tile_live = p.excl ? (tj_min < ti_max) : (tj_min <= ti_max);
    float acc = 0.f;
    if (tile_live) {
        const float* X = p.x + (size_t)g * p.mx * p.K;
        const float* Y = p.y + (size_t)g * p.ny * p.K;
        const float* GI = p.gi + (size_t)g * p.C * p.K;
        const float* GG = p.g + (size_t)g * p.C * p.K;
        for (int k0 = 0; k0 < p.K; k0 += KB) {
            for (int e = threadIdx.x; e < 16 * KB; e += 256) {
                const int rr = e / KB, kk = e % KB;
                const int k = k0 + kk;
                float xv = 0.f, gxv = 0.f, yv = 0.f, gyv = 0.f;
                if (k < p.K) {
                    if (i0 + rr < p.mx) {
                        const int tok = (i0 + rr) / p.rx;
                        xv = X[(size_t)(i0 + rr) * p.K + k];
                        gxv = GI[(size_t)tok * p.K + k] - (p.excl ? GG[(size_t)tok * p.K + k] : 0.f);
                    }
                    if (j0 + rr < p.ny) {
                        const int tok = (j0 + rr) / p.ry;
                        yv = Y[(size_t)(j0 + rr) * p.K + k];
                        gyv = GI[(size_t)tok * p.K + k];
                    }
                }
                xs[rr][kk] = xv; gxs[rr][kk] = gxv; ys[rr][kk] = yv; gys[rr][kk] = gyv;
            }
            __syncthreads();
            if (keep) {
#pragma unroll 8
                for (int kk = 0; kk < KB; ++kk)
                    acc = fmaf(xs[ty][kk] * ys[tx][kk], __expf(gxs[ty][kk] - gys[tx][kk]), acc);
            }
            __syncthreads();
        }
    }
    if (in) p.out[(size_t)g * p.mx * p.ny + (size_t)i * p.ny + j] = keep ? acc : 0.f;
}

// ------------------------------------------------------------------------------------------
// M = (I - Aab)^-1 by forward substitution (HRDPLR/naive.py:189-192; reference kernel
// HRDPLR/fwd_triton.py:588-667).  One CTA per chunk, one thread per column of M.
// ------------------------------------------------------------------------------------------
__global__ void tri_inverse_kernel(const float* Aab, float* Mout, int m) {
    extern __shared__ float Ms[];          // [m][m]
    const long long g = blockIdx.x;
    const float* L = Aab + (size_t)g * m * m;
    const int c = threadIdx.x;
    for (int i = 0; i < m; ++i) {
        float val = (c == i) ? 1.f : 0.f;
        if (c < i) {
            const float* Li = L + (size_t)i * m;
            float s = 0.f;
            for (int j = c; j < i; ++j) s = fmaf(Li[j], Ms[j * m + c], s);
            val = s;
        }
        Ms[i * m + c] = val;
        __syncthreads();
    }
    float* out = Mout + (size_t)g * m * m;
    for (int e = threadIdx.x; e < m * m; e += blockDim.x) out[e] = Ms[e];
}

// ------------------------------------------------------------------------------------------
// tile GEMM: a 256-thread CTA accumulates a 64x64 tile, 4x4 per thread, arbitrary strides
// ------------------------------------------------------------------------------------------
constexpr int TM = 64, TN = 64, TL = 16;
struct TileSmem {
    float As[TL][TM + 4];
    float Bs[TL][TN + 4];
};

// acc += A[0:mrem, 0:L] * B[0:L, 0:nrem];  A(i,l) = A[i*rsA + l*csA], B(l,j) = B[l*rsB + j*csB].
// The operands may have been written earlier by this CTA (plain loads, no read-only path).
__device__ __forceinline__ void tile_gemm(float (&acc)[4][4], const float* A, long long rsA, long long csA, int mrem,
                                          const float* B, long long rsB, long long csB, int nrem, int L,
                                          TileSmem& sm) {
    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    for (int l0 = 0; l0 < L; l0 += TL) {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const int idx = tid + 256 * s;
            int r, l;
            if (csA == 1) { l = idx & 15; r = idx >> 4; } else { r = idx & 63; l = idx >> 6; }
            float x = 0.f;
            if (r < mrem && l0 + l < L) x = A[r * rsA + (l0 + l) * csA];
            sm.As[l][r] = x;
        }
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const int idx = tid + 256 * s;
            int c, l;
            if (csB == 1) { c = idx & 63; l = idx >> 6; } else { l = idx & 15; c = idx >> 4; }
            float x = 0.f;
            if (c < nrem && l0 + l < L) x = B[(l0 + l) * rsB + c * csB];
            sm.Bs[l][c] = x;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < TL; ++l) {
            const float4 a4 = *reinterpret_cast<const float4*>(&sm.As[l][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&sm.Bs[l][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w};
            const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
}

struct Mat {
    const float* p;
    long long sbh, sn;      // strides over (batch*head) and chunk
    long long rs, cs;       // row / column stride of the logical operand
};
struct GemmP {
    Mat A, B;               // C[M,N] = alpha * A[M,L] * B[L,N]
    float* C;
    long long cbh, cn, rsC, csC;
    int M, N, L, NT;
    float alpha;
    int accumulate;         // C += ...
    int mask;               // 0 none, 1 keep (i/ri) >= (j/rj), 2 keep (i/ri) > (j/rj); masked entries are written as 0
    int ri, rj;
};

__global__ void __launch_bounds__(256) bgemm_kernel(GemmP p) {
    __shared__ TileSmem sm;
    const long long g = blockIdx.x;
    const long long bh = g / p.NT, n = g % p.NT;
    const int row0 = blockIdx.z * TM, col0 = blockIdx.y * TN;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    bool live = true;
    if (p.mask) {
        const int ti_max = min(row0 + TM - 1, p.M - 1) / p.ri, tj_min = col0 / p.rj;
        live = p.mask == 1 ? (ti_max >= tj_min) : (ti_max > tj_min);
    }
    if (live)
        tile_gemm(acc, p.A.p + bh * p.A.sbh + n * p.A.sn + row0 * p.A.rs, p.A.rs, p.A.cs, p.M - row0,
                  p.B.p + bh * p.B.sbh + n * p.B.sn + col0 * p.B.cs, p.B.rs, p.B.cs, p.N - col0, p.L, sm);
    float* Cb = p.C + bh * p.cbh + n * p.cn;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
            if (r < p.M && c < p.N) {
                float* dst = Cb + r * p.rsC + c * p.csC;
                bool keep = true;
                if (p.mask == 1) keep = (r / p.ri) >= (c / p.rj);
                else if (p.mask == 2) keep = (r / p.ri) > (c / p.rj);
                float val = 0.f;
                if (keep) {
                    val = p.alpha * acc[i][j];
                    if (p.accumulate) val += *dst;
                }
                *dst = val;
            }
        }
}

// ------------------------------------------------------------------------------------------
// inter-chunk state scan (HRDPLR/fwd_triton.py:795-968; HRDPLR/naive.py:232-255)
//   v2_n = w_n S_n + u_n ;  S_{n+1} = decay_n (.) S_n + kg_n^T v_n + bg_n^T v2_n
// One CTA per (batch*head, 64 state columns); the state lives in the h buffer, whose slot n is the
// state entering chunk n (slot NT = final state).
// ------------------------------------------------------------------------------------------
struct ScanP {
    const float *w, *u, *kg, *bg, *vc, *decay;
    float *h, *v2;
    int NT, C, m, K, V;
};

__global__ void __launch_bounds__(256) scan_fwd_kernel(ScanP p) {
    __shared__ TileSmem sm;
    const int bh = blockIdx.y, col0 = blockIdx.x * TN;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int K = p.K, V = p.V, m = p.m, C = p.C;
    for (int n = 0; n < p.NT; ++n) {
        const long long g = (long long)bh * p.NT + n;
        float* hn = p.h + ((long long)bh * (p.NT + 1) + n) * K * V;
        float* hn1 = hn + (long long)K * V;
        const float* w = p.w + g * m * K;
        const float* u = p.u + g * m * V;
        float* v2 = p.v2 + g * m * V;
        for (int row0 = 0; row0 < m; row0 += TM) {
            float acc[4][4] = {};
            tile_gemm(acc, w + (long long)row0 * K, K, 1, m - row0, hn + col0, V, 1, V - col0, K, sm);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
                    if (r < m && c < V) v2[(long long)r * V + c] = acc[i][j] + u[(long long)r * V + c];
                }
        }
        __syncthreads();
        const float* kg = p.kg + g * C * K;
        const float* bg = p.bg + g * m * K;
        const float* vc = p.vc + g * C * V;
        const float* dec = p.decay + g * K;
        for (int row0 = 0; row0 < K; row0 += TM) {
            float acc[4][4] = {};
            tile_gemm(acc, kg + row0, 1, K, K - row0, vc + col0, V, 1, V - col0, C, sm);
            tile_gemm(acc, bg + row0, 1, K, K - row0, v2 + col0, V, 1, V - col0, m, sm);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
                    if (r < K && c < V) hn1[(long long)r * V + c] = acc[i][j] + dec[r] * hn[(long long)r * V + c];
                }
        }
        __syncthreads();
    }
}

// reverse scan of the state gradient (HRDPLR/bwd_triton.py:110-222)
//   dE = gradient of the state at the end of chunk n (slot n+1 of dhs)
//   dv2_n = dv2_intra_n + bg_n dE ;  dS_n = decay_n (.) dE + qg_n^T dO_n + w_n^T dv2_n  (slot n)
struct ScanBP {
    const float *w, *qg, *bg, *doc, *decay;
    float *dhs, *dv2;
    int NT, C, m, K, V;
};

__global__ void __launch_bounds__(256) scan_bwd_kernel(ScanBP p) {
    __shared__ TileSmem sm;
    const int bh = blockIdx.y, col0 = blockIdx.x * TN;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const int K = p.K, V = p.V, m = p.m, C = p.C;
    for (int n = p.NT - 1; n >= 0; --n) {
        const long long g = (long long)bh * p.NT + n;
        float* dS = p.dhs + ((long long)bh * (p.NT + 1) + n) * K * V;
        const float* dE = dS + (long long)K * V;
        const float* bg = p.bg + g * m * K;
        float* dv2 = p.dv2 + g * m * V;
        for (int row0 = 0; row0 < m; row0 += TM) {
            float acc[4][4] = {};
            tile_gemm(acc, bg + (long long)row0 * K, K, 1, m - row0, dE + col0, V, 1, V - col0, K, sm);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
                    if (r < m && c < V) dv2[(long long)r * V + c] += acc[i][j];
                }
        }
        __syncthreads();
        const float* qg = p.qg + g * C * K;
        const float* w = p.w + g * m * K;
        const float* doc = p.doc + g * C * V;
        const float* dec = p.decay + g * K;
        for (int row0 = 0; row0 < K; row0 += TM) {
            float acc[4][4] = {};
            tile_gemm(acc, qg + row0, 1, K, K - row0, doc + col0, V, 1, V - col0, C, sm);
            tile_gemm(acc, w + row0, 1, K, K - row0, dv2 + col0, V, 1, V - col0, m, sm);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
                    if (r < K && c < V) dS[(long long)r * V + c] = acc[i][j] + dec[r] * dE[(long long)r * V + c];
                }
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// gradient of the chunk-end log decay (HRDPLR/bwd_triton.py:400,442,457-459)
//   dgl[k] = decay[k] sum_v S_n[k,v] dE[k,v] + sum_i kg[i,k] dkg[i,k] + sum_{i,r} bg dbg
// ------------------------------------------------------------------------------------------
struct DglP {
    const float *h, *dhs, *kg, *dkg, *bg, *dbg, *decay;
    float* dgl;
    int NT, C, m, K, V;
};
__global__ void __launch_bounds__(256) dgl_kernel(DglP p) {
    __shared__ float red[256];
    const long long g = blockIdx.x;
    const long long bh = g / p.NT, n = g % p.NT;
    const int K = p.K, V = p.V;
    const float* S = p.h + (bh * (p.NT + 1) + n) * K * V;
    const float* dE = p.dhs + (bh * (p.NT + 1) + n + 1) * K * V;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int k = warp; k < K; k += 8) {
        float s = 0.f;
        for (int v = lane; v < V; v += 32) s = fmaf(S[(long long)k * V + v], dE[(long long)k * V + v], s);
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) red[k] = s;
    }
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        float s = p.decay[g * K + k] * red[k];
        const float* kg = p.kg + g * p.C * K;
        const float* dkg = p.dkg + g * p.C * K;
        for (int i = 0; i < p.C; ++i) s = fmaf(kg[i * K + k], dkg[i * K + k], s);
        const float* bg = p.bg + g * p.m * K;
        const float* dbg = p.dbg + g * p.m * K;
        for (int i = 0; i < p.m; ++i) s = fmaf(bg[i * K + k], dbg[i * K + k], s);
        p.dgl[g * K + k] = s;
    }
}

// ------------------------------------------------------------------------------------------
// decay-weighted application of a score-gradient matrix (HRDPLR/bwd_triton.py:761-827):
//   out[i,k] (+)= sum_j coef(i,j) z[j,k] exp(sgn * (go[i,k] - gz[j,k]))      for coef(i,j) != 0
// Row side (dq, da): out rows are the score rows, sgn = +1.  Column side (dk, db): out rows are the
// score columns, coef is addressed transposed and sgn = -1.  Masked scores are exact zeros and are
// skipped, so every exponent that is evaluated is <= 0.
// ------------------------------------------------------------------------------------------
struct ApplyP {
    const float *coef, *z, *gi, *g;
    float* out;
    long long coef_sg, coef_rs, coef_cs;
    int n_out, n_z, ro, rz, K, C;
    int out_excl, z_excl;      // gate is ge (= gi - g) instead of gi
    float sgn;
    int accumulate;
};

__global__ void __launch_bounds__(256) gated_apply_kernel(ApplyP p) {
    constexpr int RB = 32, JB = 32, KB = 64;
    __shared__ float zs[JB][KB], gzs[JB][KB], cs[RB][JB + 1];
    const long long g = blockIdx.y;
    const int i0 = blockIdx.x * RB;
    const int kc = threadIdx.x & 63, rg = threadIdx.x >> 6;       // 64 columns x 4 row groups of 8
    const float* GI = p.gi + (size_t)g * p.C * p.K;
    const float* GG = p.g + (size_t)g * p.C * p.K;
    const float* Z = p.z + (size_t)g * p.n_z * p.K;
    const float* CF = p.coef + (size_t)g * p.coef_sg;
    for (int k0 = 0; k0 < p.K; k0 += KB) {
        const int k = k0 + kc;
        float acc[8], go[8];
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            acc[rr] = 0.f;
            const int i = i0 + rg * 8 + rr;
            go[rr] = 0.f;
            if (i < p.n_out && k < p.K) {
                const int tok = i / p.ro;
                go[rr] = GI[(size_t)tok * p.K + k] - (p.out_excl ? GG[(size_t)tok * p.K + k] : 0.f);
            }
        }
        for (int j0 = 0; j0 < p.n_z; j0 += JB) {
            int nz = 0;
            for (int e = threadIdx.x; e < RB * JB; e += 256) {
                const int rr = e / JB, jj = e % JB;
                float c = 0.f;
                if (i0 + rr < p.n_out && j0 + jj < p.n_z) c = CF[(i0 + rr) * p.coef_rs + (j0 + jj) * p.coef_cs];
                cs[rr][jj] = c;
                nz |= (c != 0.f);
            }
            for (int e = threadIdx.x; e < JB * KB; e += 256) {
                const int jj = e / KB, kk = e % KB;
                float zv = 0.f, gv = 0.f;
                if (j0 + jj < p.n_z && k0 + kk < p.K) {
                    const int tok = (j0 + jj) / p.rz;
                    zv = Z[(size_t)(j0 + jj) * p.K + k0 + kk];
                    gv = GI[(size_t)tok * p.K + k0 + kk] - (p.z_excl ? GG[(size_t)tok * p.K + k0 + kk] : 0.f);
                }
                zs[jj][kk] = zv; gzs[jj][kk] = gv;
            }
            const int any = __syncthreads_or(nz);
            if (any) {
                for (int jj = 0; jj < JB; ++jj) {
                    const float zv = zs[jj][kc], gv = gzs[jj][kc];
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        const float c = cs[rg * 8 + rr][jj];
                        if (c != 0.f) acc[rr] = fmaf(c * zv, __expf(p.sgn * (go[rr] - gv)), acc[rr]);
                    }
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
            const int i = i0 + rg * 8 + rr;
            if (i < p.n_out && k < p.K) {
                float* dst = p.out + (size_t)g * p.n_out * p.K + (size_t)i * p.K + k;
                *dst = p.accumulate ? (*dst + acc[rr]) : acc[rr];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// backward egress: un-gate, log-decay gradient, write gradients in the public layout
//   dq~ += dqg e^{gi}, dk += dkg e^{gl-gi}, da += dag e^{ge}, db += dbg e^{gl-gi}   (HRDPLR/bwd_triton.py:854-861)
//   dgk = revcumsum(q dq - k dk - sum_r b db + sum_r a da) - sum_r a da + dgl        (HRDPLR/bwd_triton.py:868-880,944-946)
// ------------------------------------------------------------------------------------------
struct EgressP {
    const float *qs, *kc, *ac, *bc, *g, *gi, *dqs, *dk, *da, *db, *dqg, *dkg, *dag, *dbg, *dgl, *dv;
    void *o_dq, *o_dk, *o_dv, *o_da, *o_db, *o_dgk;
    float scale;
    int T, H, K, V, R, C, NT, dt, gdt;
};

__global__ void __launch_bounds__(256) egress_bwd_kernel(EgressP p) {
    const long long g = blockIdx.x;
    const int bh = (int)(g / p.NT), n = (int)(g % p.NT);
    const int b = bh / p.H, h = bh % p.H;
    const int C = p.C, K = p.K, V = p.V, R = p.R;
    const int t0 = n * C;
    for (int col = threadIdx.x; col < K; col += blockDim.x) {
        const float glast = p.gi[(size_t)g * C * K + (size_t)(C - 1) * K + col];
        const float dgl = p.dgl[(size_t)g * K + col];
        float run = 0.f;
        for (int i = C - 1; i >= 0; --i) {
            const size_t e = (size_t)g * C * K + (size_t)i * K + col;
            const float gi = p.gi[e], gv = p.g[e];
            const float el = __expf(glast - gi);
            const float dq = p.dqs[e] + p.dqg[e] * __expf(gi);
            const float dk = p.dk[e] + p.dkg[e] * el;
            float d_gi = p.qs[e] * dq - p.kc[e] * dk;
            float d_ge = 0.f;
            const int t = t0 + i;
            for (int r = 0; r < R; ++r) {
                const size_t ea = (size_t)g * C * R * K + (size_t)(i * R + r) * K + col;
                const float da = p.da[ea] + p.dag[ea] * __expf(gi - gv);
                const float db = p.db[ea] + p.dbg[ea] * el;
                d_ge = fmaf(p.ac[ea], da, d_ge);
                d_gi = fmaf(-p.bc[ea], db, d_gi);
                if (t < p.T) {
                    const size_t oa = (((size_t)b * p.T * R + (size_t)t * R + r) * p.H + h) * K + col;
                    st_elem(p.o_da, oa, p.dt, da);
                    st_elem(p.o_db, oa, p.dt, db);
                }
            }
            run += d_gi + d_ge;
            if (t < p.T) {
                const size_t o = (((size_t)b * p.T + t) * p.H + h) * K + col;
                st_elem(p.o_dq, o, p.dt, dq * p.scale);
                st_elem(p.o_dk, o, p.dt, dk);
                st_elem(p.o_dgk, o, p.gdt, run - d_ge + dgl);
            }
        }
    }
    for (int e = threadIdx.x; e < C * V; e += blockDim.x) {
        const int i = e / V, col = e % V;
        const int t = t0 + i;
        if (t < p.T) st_elem(p.o_dv, (((size_t)b * p.T + t) * p.H + h) * V + col, p.dt, p.dv[(size_t)g * C * V + e]);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct Ctx {
    Plan pl;
    float* ws;
    cudaStream_t st;
    float* at(long long off) const { return ws + off; }
    Mat mat(long long off, long long per_chunk, long long rs, long long cs) const {
        return Mat{ws + off, per_chunk * pl.NT, per_chunk, rs, cs};
    }
    Mat state(long long off, int slot_shift, long long rs, long long cs) const {   // h / dhs: NT+1 slots per bh
        return Mat{ws + off + (long long)slot_shift * pl.KV, pl.KV * (pl.NT + 1), pl.KV, rs, cs};
    }
};

int gemm(const Ctx& c, Mat A, Mat B, long long Coff, long long c_per_chunk, long long rsC, long long csC, int M,
         int N, int L, float alpha = 1.f, int accumulate = 0, int mask = 0, int ri = 1, int rj = 1) {
    GemmP p{A, B, c.ws + Coff, c_per_chunk * c.pl.NT, c_per_chunk, rsC, csC, M, N, L, c.pl.NT,
            alpha, accumulate, mask, ri, rj};
    dim3 grid((unsigned)c.pl.G, (N + TN - 1) / TN, (M + TM - 1) / TM);
    bgemm_kernel<<<grid, 256, 0, c.st>>>(p);
    HDLA_CHECK_LAUNCH("bgemm_kernel");
    return HDLA_OK;
}

#define TRY(x) do { int rc__ = (x); if (rc__ != HDLA_OK) return rc__; } while (0)

int check_dims(const HdlaDims& d, const Plan& pl) {
    if (pl.m > 128) return fail(HDLA_ERR_UNSUPPORTED, "chunk: R*chunk = %d exceeds 128", pl.m);
    if (d.K > 256 || d.V > 4096) return fail(HDLA_ERR_UNSUPPORTED, "chunk: K=%d (max 256) / V=%d", d.K, d.V);
    if (pl.G > 0x7fffffffLL) return fail(HDLA_ERR_UNSUPPORTED, "chunk: too many chunks");
    return HDLA_OK;
}

}  // namespace

size_t simt_workspace_floats(const HdlaDims& d, int with_backward) {
    Plan pl = make_plan(d);
    if (check_dims(d, pl) != HDLA_OK) return 0;
    return (size_t)(with_backward ? pl.total : pl.total_fwd);
}

int simt_chunk_fwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, void* o, float* ht, float* ws, bool need_o,
                   cudaStream_t st) {
    Ctx c{make_plan(d), ws, st};
    const Plan& pl = c.pl;
    TRY(check_dims(d, pl));
    const int C = pl.C, m = pl.m, K = pl.K, V = pl.V, R = pl.R;
    const unsigned G = (unsigned)pl.G;

    IngestP ip{q, k, v, a, b, gk, c.at(pl.qs), c.at(pl.kc), c.at(pl.vc), c.at(pl.ac), c.at(pl.bc), c.at(pl.g),
               c.at(pl.gi), c.at(pl.qg), c.at(pl.kg), c.at(pl.ag), c.at(pl.bg), c.at(pl.decay), scale,
               d.T, d.H, K, V, R, C, pl.NT, d.dtype, d.gk_dtype};
    ingest_fwd_kernel<<<G, 256, 0, st>>>(ip);
    HDLA_CHECK_LAUNCH("ingest_fwd_kernel");

    auto gram = [&](long long x, int mx, int rx, int excl, long long y, int ny, int ry, long long out) -> int {
        GramP gp{c.at(x), c.at(y), c.at(pl.gi), c.at(pl.g), c.at(out), mx, ny, rx, ry, K, C, excl};
        dim3 grid((ny + 15) / 16, (mx + 15) / 16, G);
        if (G > 65535) return fail(HDLA_ERR_UNSUPPORTED, "chunk: more than 65535 chunk-heads in one call");
        gated_gram_kernel<<<grid, 256, 0, st>>>(gp);
        HDLA_CHECK_LAUNCH("gated_gram_kernel");
        return HDLA_OK;
    };
    TRY(gram(pl.qs, C, 1, 0, pl.kc, C, 1, pl.Aqk));
    TRY(gram(pl.qs, C, 1, 0, pl.bc, m, R, pl.Aqb));
    TRY(gram(pl.ac, m, R, 1, pl.kc, C, 1, pl.Aak));
    TRY(gram(pl.ac, m, R, 1, pl.bc, m, R, pl.Aab));

    {
        const size_t smem = (size_t)m * m * sizeof(float);
        static thread_local int attr_dev = -1;
        int dev = 0;
        cudaGetDevice(&dev);
        if (attr_dev != dev) {
            cudaFuncSetAttribute(tri_inverse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 128 * 4);
            attr_dev = dev;
        }
        tri_inverse_kernel<<<G, m, smem, st>>>(c.at(pl.Aab), c.at(pl.M), m);
        HDLA_CHECK_LAUNCH("tri_inverse_kernel");
    }
    // P = Aak v ; w = M ag ; u = M P           (HRDPLR/naive.py:195-196)
    TRY(gemm(c, c.mat(pl.Aak, pl.Cm, C, 1), c.mat(pl.vc, pl.CV, V, 1), pl.P, pl.mV, V, 1, m, V, C));
    TRY(gemm(c, c.mat(pl.M, pl.mm, m, 1), c.mat(pl.ag, pl.mK, K, 1), pl.w, pl.mK, K, 1, m, K, m));
    TRY(gemm(c, c.mat(pl.M, pl.mm, m, 1), c.mat(pl.P, pl.mV, V, 1), pl.u, pl.mV, V, 1, m, V, m));

    // state slots: slot 0 <- h0 (or zero)
    const size_t pitch = (size_t)(pl.NT + 1) * pl.KV * sizeof(float), width = (size_t)pl.KV * sizeof(float);
    cudaError_t e;
    if (h0) e = cudaMemcpy2DAsync(c.at(pl.h), pitch, h0, width, width, pl.BH, cudaMemcpyDeviceToDevice, st);
    else e = cudaMemset2DAsync(c.at(pl.h), pitch, 0, width, pl.BH, st);
    if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "state init: %s", cudaGetErrorString(e));

    ScanP sp{c.at(pl.w), c.at(pl.u), c.at(pl.kg), c.at(pl.bg), c.at(pl.vc), c.at(pl.decay), c.at(pl.h), c.at(pl.v2),
             pl.NT, C, m, K, V};
    scan_fwd_kernel<<<dim3((V + TN - 1) / TN, pl.BH), 256, 0, st>>>(sp);
    HDLA_CHECK_LAUNCH("scan_fwd_kernel");
    if (ht) {
        e = cudaMemcpy2DAsync(ht, width, c.at(pl.h) + (long long)pl.NT * pl.KV, pitch, width, pl.BH,
                              cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "final state copy: %s", cudaGetErrorString(e));
    }
    if (need_o) {
        // o = qg S + Aqk v + Aqb v2      (HRDPLR/fwd_triton.py:1031,1094)
        TRY(gemm(c, c.mat(pl.qg, pl.CK, K, 1), c.state(pl.h, 0, V, 1), pl.oc, pl.CV, V, 1, C, V, K));
        TRY(gemm(c, c.mat(pl.Aqk, pl.CC, C, 1), c.mat(pl.vc, pl.CV, V, 1), pl.oc, pl.CV, V, 1, C, V, C, 1.f, 1));
        TRY(gemm(c, c.mat(pl.Aqb, pl.Cm, m, 1), c.mat(pl.v2, pl.mV, V, 1), pl.oc, pl.CV, V, 1, C, V, m, 1.f, 1));
        from_chunk_major_kernel<<<G, 256, 0, st>>>(c.at(pl.oc), o, d.T, d.H, V, C, pl.NT, d.dtype, 1.f);
        HDLA_CHECK_LAUNCH("from_chunk_major_kernel");
    }
    return HDLA_OK;
}

int simt_chunk_bwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, const void* d_o, const float* dht, void* dq,
                   void* dk, void* dv, void* da, void* db, void* dgk, float* dh0, float* ws, cudaStream_t st) {
    if (!(d.flags & HDLA_FLAG_WS_HOLDS_FWD))
        TRY(simt_chunk_fwd(d, q, k, v, a, b, gk, scale, h0, nullptr, nullptr, ws, false, st));
    Ctx c{make_plan(d), ws, st};
    const Plan& pl = c.pl;
    TRY(check_dims(d, pl));
    const int C = pl.C, m = pl.m, K = pl.K, V = pl.V, R = pl.R;
    const unsigned G = (unsigned)pl.G;

    to_chunk_major_kernel<<<G, 256, 0, st>>>(d_o, c.at(pl.doc), d.T, d.H, V, C, pl.NT, d.dtype);
    HDLA_CHECK_LAUNCH("to_chunk_major_kernel");
    // --- dAu
    TRY(gemm(c, c.mat(pl.doc, pl.CV, V, 1), c.mat(pl.vc, pl.CV, 1, V), pl.dAqk, pl.CC, C, 1, C, C, V, 1.f, 0, 1, 1, 1));
    TRY(gemm(c, c.mat(pl.doc, pl.CV, V, 1), c.mat(pl.v2, pl.mV, 1, V), pl.dAqb, pl.Cm, m, 1, C, m, V, 1.f, 0, 1, 1, R));
    TRY(gemm(c, c.mat(pl.Aqb, pl.Cm, 1, m), c.mat(pl.doc, pl.CV, V, 1), pl.dv2, pl.mV, V, 1, m, V, C));
    // --- dhu: slot NT <- dht (or zero), reverse scan
    const size_t pitch = (size_t)(pl.NT + 1) * pl.KV * sizeof(float), width = (size_t)pl.KV * sizeof(float);
    cudaError_t e;
    float* last = c.at(pl.dhs) + (long long)pl.NT * pl.KV;
    if (dht) e = cudaMemcpy2DAsync(last, pitch, dht, width, width, pl.BH, cudaMemcpyDeviceToDevice, st);
    else e = cudaMemset2DAsync(last, pitch, 0, width, pl.BH, st);
    if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "dht init: %s", cudaGetErrorString(e));
    ScanBP sp{c.at(pl.w), c.at(pl.qg), c.at(pl.bg), c.at(pl.doc), c.at(pl.decay), c.at(pl.dhs), c.at(pl.dv2),
              pl.NT, C, m, K, V};
    scan_bwd_kernel<<<dim3((V + TN - 1) / TN, pl.BH), 256, 0, st>>>(sp);
    HDLA_CHECK_LAUNCH("scan_bwd_kernel");
    if (dh0) {
        e = cudaMemcpy2DAsync(dh0, width, c.at(pl.dhs), pitch, width, pl.BH, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "dh0 copy: %s", cudaGetErrorString(e));
    }
    Mat S = c.state(pl.h, 0, V, 1), St = c.state(pl.h, 0, 1, V);            // S_n and its transpose
    Mat dE = c.state(pl.dhs, 1, V, 1), dEt = c.state(pl.dhs, 1, 1, V);      // gradient at chunk end
    // --- dv (direct): kg dE + Aqk^T dO
    TRY(gemm(c, c.mat(pl.kg, pl.CK, K, 1), dE, pl.dv, pl.CV, V, 1, C, V, K));
    TRY(gemm(c, c.mat(pl.Aqk, pl.CC, 1, C), c.mat(pl.doc, pl.CV, V, 1), pl.dv, pl.CV, V, 1, C, V, C, 1.f, 1));
    // --- bwd_o
    TRY(gemm(c, c.mat(pl.doc, pl.CV, V, 1), St, pl.dqg, pl.CK, K, 1, C, K, V));
    TRY(gemm(c, c.mat(pl.vc, pl.CV, V, 1), dEt, pl.dkg, pl.CK, K, 1, C, K, V));
    TRY(gemm(c, c.mat(pl.v2, pl.mV, V, 1), dEt, pl.dbg, pl.mK, K, 1, m, K, V));
    TRY(gemm(c, c.mat(pl.dv2, pl.mV, V, 1), St, pl.dw, pl.mK, K, 1, m, K, V));
    DglP gp{c.at(pl.h), c.at(pl.dhs), c.at(pl.kg), c.at(pl.dkg), c.at(pl.bg), c.at(pl.dbg), c.at(pl.decay),
            c.at(pl.dgl), pl.NT, C, m, K, V};
    dgl_kernel<<<G, 256, 0, st>>>(gp);
    HDLA_CHECK_LAUNCH("dgl_kernel");
    // --- wy
    Mat Mt = c.mat(pl.M, pl.mm, 1, m);
    TRY(gemm(c, Mt, c.mat(pl.dv2, pl.mV, V, 1), pl.dP, pl.mV, V, 1, m, V, m));
    TRY(gemm(c, c.mat(pl.dP, pl.mV, V, 1), c.mat(pl.vc, pl.CV, 1, V), pl.dAak, pl.Cm, C, 1, m, C, V, 1.f, 0, 2, R, 1));
    TRY(gemm(c, c.mat(pl.Aak, pl.Cm, 1, C), c.mat(pl.dP, pl.mV, V, 1), pl.dv, pl.CV, V, 1, C, V, m, 1.f, 1));
    TRY(gemm(c, c.mat(pl.dv2, pl.mV, V, 1), c.mat(pl.P, pl.mV, 1, V), pl.dM, pl.mm, m, 1, m, m, V));
    TRY(gemm(c, c.mat(pl.dw, pl.mK, K, 1), c.mat(pl.ag, pl.mK, 1, K), pl.dM, pl.mm, m, 1, m, m, K, 1.f, 1));
    TRY(gemm(c, Mt, c.mat(pl.dM, pl.mm, m, 1), pl.tmp, pl.mm, m, 1, m, m, m));
    TRY(gemm(c, c.mat(pl.tmp, pl.mm, m, 1), Mt, pl.dAab, pl.mm, m, 1, m, m, m, 1.f, 0, 2, R, R));
    TRY(gemm(c, Mt, c.mat(pl.dw, pl.mK, K, 1), pl.dag, pl.mK, K, 1, m, K, m));
    // --- intra
    if (G > 65535) return fail(HDLA_ERR_UNSUPPORTED, "chunk: more than 65535 chunk-heads in one call");
    auto apply = [&](long long coef, long long coef_sg, long long crs, long long ccs, long long z, int n_z, int rz,
                     int z_excl, long long out, int n_out, int ro, int out_excl, float sgn, int accumulate) -> int {
        ApplyP ap{c.at(coef), c.at(z), c.at(pl.gi), c.at(pl.g), c.at(out), coef_sg, crs, ccs, n_out, n_z, ro, rz,
                  K, C, out_excl, z_excl, sgn, accumulate};
        gated_apply_kernel<<<dim3((n_out + 31) / 32, G), 256, 0, st>>>(ap);
        HDLA_CHECK_LAUNCH("gated_apply_kernel");
        return HDLA_OK;
    };
    // row side
    TRY(apply(pl.dAqk, pl.CC, C, 1, pl.kc, C, 1, 0, pl.dqs, C, 1, 0, 1.f, 0));
    TRY(apply(pl.dAqb, pl.Cm, m, 1, pl.bc, m, R, 0, pl.dqs, C, 1, 0, 1.f, 1));
    TRY(apply(pl.dAak, pl.Cm, C, 1, pl.kc, C, 1, 0, pl.da, m, R, 1, 1.f, 0));
    TRY(apply(pl.dAab, pl.mm, m, 1, pl.bc, m, R, 0, pl.da, m, R, 1, 1.f, 1));
    // column side (coef addressed transposed)
    TRY(apply(pl.dAqk, pl.CC, 1, C, pl.qs, C, 1, 0, pl.dk, C, 1, 0, -1.f, 0));
    TRY(apply(pl.dAak, pl.Cm, 1, C, pl.ac, m, R, 1, pl.dk, C, 1, 0, -1.f, 1));
    TRY(apply(pl.dAqb, pl.Cm, 1, m, pl.qs, C, 1, 0, pl.db, m, R, 0, -1.f, 0));
    TRY(apply(pl.dAab, pl.mm, 1, m, pl.ac, m, R, 1, pl.db, m, R, 0, -1.f, 1));
    // --- egress (+ dgk)
    EgressP ep{c.at(pl.qs), c.at(pl.kc), c.at(pl.ac), c.at(pl.bc), c.at(pl.g), c.at(pl.gi), c.at(pl.dqs), c.at(pl.dk),
               c.at(pl.da), c.at(pl.db), c.at(pl.dqg), c.at(pl.dkg), c.at(pl.dag), c.at(pl.dbg), c.at(pl.dgl),
               c.at(pl.dv), dq, dk, dv, da, db, dgk, scale, d.T, d.H, K, V, R, C, pl.NT, d.dtype, d.gk_dtype};
    egress_bwd_kernel<<<G, 256, 0, st>>>(ep);
    HDLA_CHECK_LAUNCH("egress_bwd_kernel");
    return HDLA_OK;
}

}  // namespace hdla
