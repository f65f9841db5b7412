// a/b parametrisation of the HDLA layer (reference: parameterize_a_b, HRDPLR/hdla_custom.py:19-43):
//   ef = exp(log_f);  a1 = -beta k;  at2 = -beta ef k;  s = sum_K(k at2);  a2 = at2 + a1 s
//   b1 = ef k;  b2 = k;   a, b interleaved time-major / rank-minor: row 2t + r of [B, 2T, H, K]
// Forward and backward, bandwidth bound.  Head dims that are multiples of 8 up to 256 (the operator's own) take the
// vector kernels: 16 lanes per (b, t, h) row, 16-byte loads and stores, the row held in registers between the
// K-reduction (a shuffle tree over the 16 lanes) and the stores.  Other head dims take the scalar kernels, one warp
// per row.
#include "common.cuh"

namespace hdla {
namespace {

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

struct AbP {
    const void *beta, *k, *log_f;
    void *a, *b;                       // forward outputs / backward: incoming da, db
    void *dbeta, *dk, *dlog_f;         // backward outputs
    long long rows;                    // B*T*H
    int T, H, K, dt;
    int gdt;                           // dtype of log_f and dlog_f (the operator's gk may be fp32 next to bf16 tensors)
    int accumulate;                    // backward: add to what dk and dlog_f already hold (the operator's own shares)
    int norm_k;                        // backward (vector kernel): k was normalised on the way in, k / sqrt(sum k^2 + eps);
                                       // everything is taken at the normalised k and dk goes back through the norm
};

__device__ __forceinline__ void row_index(const AbP& p, long long row, size_t& in_off, size_t& o1, size_t& o2) {
    const int h = (int)(row % p.H);
    const long long bt = row / p.H;
    const long long b = bt / p.T, t = bt % p.T;
    in_off = (size_t)row * p.K;
    o1 = (((size_t)b * 2 * p.T + 2 * t) * p.H + h) * p.K;
    o2 = o1 + (size_t)p.H * p.K;
}

__global__ void __launch_bounds__(256) param_ab_fwd_kernel(AbP p) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= p.rows) return;
    const int lane = threadIdx.x & 31;
    size_t in, o1, o2;
    row_index(p, row, in, o1, o2);
    const float beta = ld_elem(p.beta, (size_t)row, p.dt);
    float s = 0.f;
    for (int c = lane; c < p.K; c += 32) {
        const float kv = ld_elem(p.k, in + c, p.dt);
        s += kv * (-beta * __expf(ld_elem(p.log_f, in + c, p.gdt)) * kv);
    }
    s = warp_sum(s);
    for (int c = lane; c < p.K; c += 32) {
        const float kv = ld_elem(p.k, in + c, p.dt);
        const float ef = __expf(ld_elem(p.log_f, in + c, p.gdt));
        const float a1 = -beta * kv, at2 = -beta * ef * kv;
        st_elem(p.a, o1 + c, p.dt, a1);
        st_elem(p.a, o2 + c, p.dt, at2 + a1 * s);
        st_elem(p.b, o1 + c, p.dt, ef * kv);
        st_elem(p.b, o2 + c, p.dt, kv);
    }
}

__global__ void __launch_bounds__(256) param_ab_bwd_kernel(AbP p) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= p.rows) return;
    const int lane = threadIdx.x & 31;
    size_t in, o1, o2;
    row_index(p, row, in, o1, o2);
    const float beta = ld_elem(p.beta, (size_t)row, p.dt);
    // pass 1: s = sum k at2 ; ds = sum a1 da2
    float s = 0.f, ds = 0.f;
    for (int c = lane; c < p.K; c += 32) {
        const float kv = ld_elem(p.k, in + c, p.dt);
        const float ef = __expf(ld_elem(p.log_f, in + c, p.gdt));
        s += kv * (-beta * ef * kv);
        ds += (-beta * kv) * ld_elem(p.a, o2 + c, p.dt);
    }
    s = warp_sum(s);
    ds = warp_sum(ds);
    float dbeta = 0.f;
    for (int c = lane; c < p.K; c += 32) {
        const float kv = ld_elem(p.k, in + c, p.dt);
        const float ef = __expf(ld_elem(p.log_f, in + c, p.gdt));
        const float da1 = ld_elem(p.a, o1 + c, p.dt), da2 = ld_elem(p.a, o2 + c, p.dt);
        const float db1 = ld_elem(p.b, o1 + c, p.dt), db2 = ld_elem(p.b, o2 + c, p.dt);
        const float at2 = -beta * ef * kv;
        const float dat2 = da2 + kv * ds;            // a2 = at2 + a1 s,  s = sum k at2
        const float da1t = da1 + s * da2;
        float dk = at2 * ds;                         // through s (the factor k)
        dk += -beta * ef * dat2;                     // at2 = -beta ef k
        dk += -beta * da1t;                          // a1 = -beta k
        dk += ef * db1 + db2;                        // b1 = ef k, b2 = k
        const float def = -beta * kv * dat2 + kv * db1;
        dbeta += -ef * kv * dat2 - kv * da1t;
        float dlf = def * ef;
        if (p.accumulate) {
            dk += ld_elem(p.dk, in + c, p.dt);
            dlf += ld_elem(p.dlog_f, in + c, p.gdt);
        }
        st_elem(p.dk, in + c, p.dt, dk);
        st_elem(p.dlog_f, in + c, p.gdt, dlf);
    }
    dbeta = warp_sum(dbeta);
    if (lane == 0) st_elem(p.dbeta, (size_t)row, p.dt, dbeta);
}

// ---- vector kernels: 16 lanes per row, lane l owns the 8-column pieces l and l + 16
constexpr int kAbLanes = 16;

__device__ __forceinline__ float sub_sum(float x) {
#pragma unroll
    for (int o = kAbLanes / 2; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

template <int PIECES>
__global__ void __launch_bounds__(256) param_ab_fwd_vec_kernel(AbP p) {
    const long long row = (long long)blockIdx.x * (256 / kAbLanes) + (threadIdx.x / kAbLanes);
    const bool live = row < p.rows;                          // whole warps stay for the shuffles
    const int l = threadIdx.x % kAbLanes, npiece = p.K / 8;
    size_t in = 0, o1 = 0, o2 = 0;
    if (live) row_index(p, row, in, o1, o2);
    const float beta = live ? ld_elem(p.beta, (size_t)row, p.dt) : 0.f;
    float kv[PIECES][8], ef[PIECES][8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int pc = l + j * kAbLanes;
        if (live && pc < npiece) {
            ld_elem8(p.k, in + pc * 8, p.dt, kv[j]);
            ld_elem8(p.log_f, in + pc * 8, p.gdt, ef[j]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ef[j][e] = __expf(ef[j][e]);
                s += kv[j][e] * (-beta * ef[j][e] * kv[j][e]);
            }
        }
    }
    s = sub_sum(s);
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int pc = l + j * kAbLanes;
        if (live && pc < npiece) {
            float a1[8], a2[8], b1[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a1[e] = -beta * kv[j][e];
                a2[e] = -beta * ef[j][e] * kv[j][e] + a1[e] * s;
                b1[e] = ef[j][e] * kv[j][e];
            }
            st_elem8(p.a, o1 + pc * 8, p.dt, a1);
            st_elem8(p.a, o2 + pc * 8, p.dt, a2);
            st_elem8(p.b, o1 + pc * 8, p.dt, b1);
            st_elem8(p.b, o2 + pc * 8, p.dt, kv[j]);
        }
    }
}

// Every load of a row's piece sits in ONE conditional block together with the first use of its data, so that all of
// them are in flight at once (a load whose result is merged with a default after its condition is waited for right
// there, which would put the round trips to memory one behind the other).  The sums that need the normalised k are
// taken at the raw k inside that block and scaled after the reductions: s = rn^2 s_raw, ds = rn ds_raw.
template <int PIECES, bool ACC, int DT>
__global__ void __launch_bounds__(256) param_ab_bwd_vec_kernel(AbP p) {
    const long long row = (long long)blockIdx.x * (256 / kAbLanes) + (threadIdx.x / kAbLanes);
    const bool live = row < p.rows;
    const int l = threadIdx.x % kAbLanes, npiece = p.K / 8;
    size_t in = 0, o1 = 0, o2 = 0;
    if (live) row_index(p, row, in, o1, o2);
    const float beta = live ? ld_elem(p.beta, (size_t)row, DT) : 0.f;
    float kv[PIECES][8], ef[PIECES][8], da1[PIECES][8], da2[PIECES][8], db1[PIECES][8], db2[PIECES][8];
    float dk0[PIECES][8], dlf0[PIECES][8];
    float s = 0.f, ds = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int pc = l + j * kAbLanes;
        if (live && pc < npiece) {
            ld_elem8(p.k, in + pc * 8, DT, kv[j]);
            ld_elem8(p.log_f, in + pc * 8, p.gdt, ef[j]);
            ld_elem8(p.a, o1 + pc * 8, DT, da1[j]);
            ld_elem8(p.a, o2 + pc * 8, DT, da2[j]);
            ld_elem8(p.b, o1 + pc * 8, DT, db1[j]);
            ld_elem8(p.b, o2 + pc * 8, DT, db2[j]);
            if (ACC) {
                ld_elem8(p.dk, in + pc * 8, DT, dk0[j]);
                ld_elem8(p.dlog_f, in + pc * 8, p.gdt, dlf0[j]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ef[j][e] = __expf(ef[j][e]);
                s += kv[j][e] * (-beta * ef[j][e] * kv[j][e]);
                ds += (-beta * kv[j][e]) * da2[j][e];
                ss = fmaf(kv[j][e], kv[j][e], ss);
            }
        }
    }
    s = sub_sum(s);
    ds = sub_sum(ds);
    float rn = 1.f;
    if (p.norm_k) {
        rn = rsqrtf(sub_sum(ss) + kNormEps);
        s *= rn * rn;
        ds *= rn;
    }
    float dbeta = 0.f, kdk = 0.f;
    float dk[PIECES][8];
#pragma unroll
    for (int j = 0; j < PIECES; ++j) {
        const int pc = l + j * kAbLanes;
        if (live && pc < npiece) {
            float dlf[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float k = kv[j][e] * rn, f = ef[j][e];
                kv[j][e] = k;
                const float at2 = -beta * f * k;
                const float dat2 = da2[j][e] + k * ds;       // a2 = at2 + a1 s,  s = sum k at2
                const float da1t = da1[j][e] + s * da2[j][e];
                float g = at2 * ds;                          // through s (the factor k)
                g += -beta * f * dat2;                       // at2 = -beta ef k
                g += -beta * da1t;                           // a1 = -beta k
                g += f * db1[j][e] + db2[j][e];              // b1 = ef k, b2 = k
                dk[j][e] = ACC ? g + dk0[j][e] : g;
                kdk = fmaf(k, dk[j][e], kdk);
                dlf[e] = (-beta * k * dat2 + k * db1[j][e]) * f + (ACC ? dlf0[j][e] : 0.f);
                dbeta += -f * k * dat2 - k * da1t;
            }
            st_elem8(p.dlog_f, in + pc * 8, p.gdt, dlf);
            if (!p.norm_k) st_elem8(p.dk, in + pc * 8, DT, dk[j]);
        }
    }
    if (p.norm_k) {                                          // k_n = k rn:  dk = rn (dk_n - k_n (k_n . dk_n))
        kdk = sub_sum(kdk);
#pragma unroll
        for (int j = 0; j < PIECES; ++j) {
            const int pc = l + j * kAbLanes;
            if (live && pc < npiece) {
#pragma unroll
                for (int e = 0; e < 8; ++e) dk[j][e] = rn * (dk[j][e] - kv[j][e] * kdk);
                st_elem8(p.dk, in + pc * 8, DT, dk[j]);
            }
        }
    }
    dbeta = sub_sum(dbeta);
    if (live && l == 0) st_elem(p.dbeta, (size_t)row, DT, dbeta);
}

}  // namespace

int param_ab_launch(bool backward, const void* beta, const void* k, const void* log_f, void* a, void* b, void* dbeta,
                    void* dk, void* dlog_f, int B, int T, int H, int K, int dt, int gdt, int accumulate, int norm_k,
                    cudaStream_t st) {
    AbP p{beta, k, log_f, a, b, dbeta, dk, dlog_f, (long long)B * T * H, T, H, K, dt, gdt, accumulate, norm_k};
    bool aligned = true;
    for (const void* q : {k, log_f, (const void*)a, (const void*)b, (const void*)dk, (const void*)dlog_f})
        aligned = aligned && reinterpret_cast<uintptr_t>(q) % 16 == 0;
    if (aligned && K % 8 == 0 && K <= kAbLanes * 16) {
        const unsigned blocks = (unsigned)((p.rows + 15) / 16);
        const bool wide = K > kAbLanes * 8;
        if (backward) {
            void (*kern)(AbP) = nullptr;
            if (dt == HDLA_BF16)
                kern = wide ? (accumulate ? param_ab_bwd_vec_kernel<2, true, HDLA_BF16> : param_ab_bwd_vec_kernel<2, false, HDLA_BF16>)
                            : (accumulate ? param_ab_bwd_vec_kernel<1, true, HDLA_BF16> : param_ab_bwd_vec_kernel<1, false, HDLA_BF16>);
            else
                kern = wide ? (accumulate ? param_ab_bwd_vec_kernel<2, true, HDLA_F32> : param_ab_bwd_vec_kernel<2, false, HDLA_F32>)
                            : (accumulate ? param_ab_bwd_vec_kernel<1, true, HDLA_F32> : param_ab_bwd_vec_kernel<1, false, HDLA_F32>);
            kern<<<blocks, 256, 0, st>>>(p);
        } else {
            if (wide) param_ab_fwd_vec_kernel<2><<<blocks, 256, 0, st>>>(p);
            else param_ab_fwd_vec_kernel<1><<<blocks, 256, 0, st>>>(p);
        }
        HDLA_CHECK_LAUNCH(backward ? "param_ab_bwd_vec_kernel" : "param_ab_fwd_vec_kernel");
        return HDLA_OK;
    }
    if (norm_k) return fail(HDLA_ERR_INVALID, "param_ab: the normalised-k form needs 16-byte aligned tensors and K a multiple of 8");
    const unsigned blocks = (unsigned)((p.rows + 7) / 8);
    if (backward) param_ab_bwd_kernel<<<blocks, 256, 0, st>>>(p);
    else param_ab_fwd_kernel<<<blocks, 256, 0, st>>>(p);
    HDLA_CHECK_LAUNCH(backward ? "param_ab_bwd_kernel" : "param_ab_fwd_kernel");
    return HDLA_OK;
}

}  // namespace hdla
