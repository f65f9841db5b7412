// a/b parametrisation of the HDLA layer (reference: parameterize_a_b, HRDPLR/hdla_custom.py:19-43):
//   ef = exp(log_f);  a1 = -beta k;  at2 = -beta ef k;  s = sum_K(k at2);  a2 = at2 + a1 s
//   b1 = ef k;  b2 = k;   a, b interleaved time-major / rank-minor: row 2t + r of [B, 2T, H, K]
// One warp per (b, t, h) row; the K-reduction is a shuffle tree.  Forward and backward.
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
        s += kv * (-beta * __expf(ld_elem(p.log_f, in + c, p.dt)) * kv);
    }
    s = warp_sum(s);
    for (int c = lane; c < p.K; c += 32) {
        const float kv = ld_elem(p.k, in + c, p.dt);
        const float ef = __expf(ld_elem(p.log_f, in + c, p.dt));
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
        const float ef = __expf(ld_elem(p.log_f, in + c, p.dt));
        s += kv * (-beta * ef * kv);
        ds += (-beta * kv) * ld_elem(p.a, o2 + c, p.dt);
    }
    s = warp_sum(s);
    ds = warp_sum(ds);
    float dbeta = 0.f;
    for (int c = lane; c < p.K; c += 32) {
        const float kv = ld_elem(p.k, in + c, p.dt);
        const float ef = __expf(ld_elem(p.log_f, in + c, p.dt));
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
        st_elem(p.dk, in + c, p.dt, dk);
        st_elem(p.dlog_f, in + c, p.dt, def * ef);
    }
    dbeta = warp_sum(dbeta);
    if (lane == 0) st_elem(p.dbeta, (size_t)row, p.dt, dbeta);
}

}  // namespace

int param_ab_launch(bool backward, const void* beta, const void* k, const void* log_f, void* a, void* b, void* dbeta,
                    void* dk, void* dlog_f, int B, int T, int H, int K, int dt, cudaStream_t st) {
    AbP p{beta, k, log_f, a, b, dbeta, dk, dlog_f, (long long)B * T * H, T, H, K, dt};
    const unsigned blocks = (unsigned)((p.rows + 7) / 8);
    if (backward) param_ab_bwd_kernel<<<blocks, 256, 0, st>>>(p);
    else param_ab_fwd_kernel<<<blocks, 256, 0, st>>>(p);
    HDLA_CHECK_LAUNCH(backward ? "param_ab_bwd_kernel" : "param_ab_fwd_kernel");
    return HDLA_OK;
}

}  // namespace hdla
