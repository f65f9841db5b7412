// Fused recurrent forward of the rank-R DPLR delta rule (decode and short prefill).
//
// Follows the per-token recurrence of the reference kernel (HRDPLR/recurrent.py:75-115):
//     sa_r  = a_r^T S_{t-1}                          (one V-vector per rank)
//     S_t   = exp(g_t) (.) S_{t-1} + sum_r b_r sa_r^T + k_t v_t^T
//     o_t   = (scale q_t)^T S_t
//
// The kernel is bound by HBM traffic: with one token per call the fp32 state [K,V] of every
// (sequence, head) is read once and written once.  Layout of the work:
//   * one CTA per (sequence, head); one warp per 32 state columns;
//   * a lane owns rows k = (lane/8) + 4 s, s = 0..KT-1, of 4 adjacent columns, so every state
//     access is a 128-bit load/store and 8 lanes cover one full 128-byte line of a row;
//   * the two K-reductions per token (a^T S and q^T S) are register sums over the lane's rows
//     followed by two warp shuffles (xor 8, 16) -- no shared-memory reduction, no block barrier
//     on the reduction path;
//   * the per-token K-vectors (q, k, exp(g), a_r, b_r) and v are staged once per CTA in shared
//     memory (double buffered, one barrier per token) and broadcast from there.
#include "common.cuh"
#include "sm100.cuh"

namespace hdla {
namespace {

// Set to 1 by the decode kernel when its (time-bounded) wait for the state tile ran out: the call's
// outputs are invalid and the final state was not written.  Read with hdla_recurrent_read_status().
__device__ int g_recurrent_status;

struct RecParams {
    const void *q, *k, *v, *a, *b, *gk;
    const float* h0;
    void* o;
    float* ht;
    const int64_t* cu;
    float scale;
    int T, H, K, V, dt, gdt, reverse;
};

template <int KT, int R>
__global__ void __launch_bounds__(256) recurrent_fwd_kernel(RecParams p) {
    const int nh = blockIdx.x;
    const int n = nh / p.H, h = nh % p.H;
    const int K = p.K, V = p.V, H = p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 3;
    const int c4 = (warp * 8 + (lane & 7)) * 4;
    const bool col_ok = c4 < V;

    long long bos, len;
    if (p.cu) { bos = p.cu[n]; len = p.cu[n + 1] - bos; }
    else      { bos = (long long)n * p.T; len = p.T; }

    extern __shared__ float sm[];
    const int vec_floats = (3 + 2 * R) * K + V;       // q k eg a[R] b[R] v

    float S[KT][4];
#pragma unroll
    for (int s = 0; s < KT; ++s) {
        const int kk = r + 4 * s;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.h0 && col_ok && kk < K)
            x = __ldcs(reinterpret_cast<const float4*>(p.h0 + ((size_t)nh * K + kk) * V + c4));
        S[s][0] = x.x; S[s][1] = x.y; S[s][2] = x.z; S[s][3] = x.w;
    }

    for (long long step = 0; step < len; ++step) {
        const long long t = p.reverse ? (bos + len - 1 - step) : (bos + step);
        float* buf = sm + (step & 1) * vec_floats;
        float* s_q = buf;
        float* s_k = buf + K;
        float* s_e = buf + 2 * K;
        float* s_a = buf + 3 * K;
        float* s_b = buf + (3 + R) * K;
        float* s_v = buf + (3 + 2 * R) * K;
        const size_t tk = ((size_t)t * H + h) * K;
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            s_q[i] = ld_elem(p.q, tk + i, p.dt) * p.scale;
            s_k[i] = ld_elem(p.k, tk + i, p.dt);
            s_e[i] = __expf(ld_elem(p.gk, tk + i, p.gdt));
#pragma unroll
            for (int rr = 0; rr < R; ++rr) {
                const size_t ta = (((size_t)t * R + rr) * H + h) * K;
                s_a[rr * K + i] = ld_elem(p.a, ta + i, p.dt);
                s_b[rr * K + i] = ld_elem(p.b, ta + i, p.dt);
            }
        }
        for (int i = threadIdx.x; i < V; i += blockDim.x)
            s_v[i] = ld_elem(p.v, ((size_t)t * H + h) * V + i, p.dt);
        __syncthreads();

        float sa[R][4];
#pragma unroll
        for (int rr = 0; rr < R; ++rr) { sa[rr][0] = sa[rr][1] = sa[rr][2] = sa[rr][3] = 0.f; }
#pragma unroll
        for (int s = 0; s < KT; ++s) {
            const int kk = r + 4 * s;
            if (kk < K) {
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const float av = s_a[rr * K + kk];
#pragma unroll
                    for (int j = 0; j < 4; ++j) sa[rr][j] = fmaf(av, S[s][j], sa[rr][j]);
                }
            }
        }
#pragma unroll
        for (int rr = 0; rr < R; ++rr)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sa[rr][j] += __shfl_xor_sync(0xffffffffu, sa[rr][j], 8);
                sa[rr][j] += __shfl_xor_sync(0xffffffffu, sa[rr][j], 16);
            }
        float vv[4] = {0.f, 0.f, 0.f, 0.f};
        if (col_ok) { vv[0] = s_v[c4]; vv[1] = s_v[c4 + 1]; vv[2] = s_v[c4 + 2]; vv[3] = s_v[c4 + 3]; }
        float oa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < KT; ++s) {
            const int kk = r + 4 * s;
            if (kk < K) {
                const float e = s_e[kk], kv = s_k[kk], qv = s_q[kk];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x = fmaf(kv, vv[j], e * S[s][j]);
#pragma unroll
                    for (int rr = 0; rr < R; ++rr) x = fmaf(s_b[rr * K + kk], sa[rr][j], x);
                    S[s][j] = x;
                    oa[j] = fmaf(qv, x, oa[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            oa[j] += __shfl_xor_sync(0xffffffffu, oa[j], 8);
            oa[j] += __shfl_xor_sync(0xffffffffu, oa[j], 16);
        }
        if (r == 0 && col_ok) {
            const size_t to = ((size_t)t * H + h) * V + c4;
            if (p.dt == HDLA_F32) {
                *reinterpret_cast<float4*>(static_cast<float*>(p.o) + to) = make_float4(oa[0], oa[1], oa[2], oa[3]);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(oa[0], oa[1]);
                __nv_bfloat162 hi = __floats2bfloat162_rn(oa[2], oa[3]);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.o) + to) = pk;
            }
        }
    }

    if (p.ht && col_ok) {
#pragma unroll
        for (int s = 0; s < KT; ++s) {
            const int kk = r + 4 * s;
            if (kk < K)
                __stcs(reinterpret_cast<float4*>(p.ht + ((size_t)nh * K + kk) * V + c4),
                       make_float4(S[s][0], S[s][1], S[s][2], S[s][3]));
        }
    }
}

// ------------------------------------------------------------------------------------------
// Decode variant (a few tokens per call): the state tile is staged in shared memory by the bulk
// asynchronous copy engine instead of through registers.
//   * one CTA per (sequence, head): ONE cp.async.bulk brings the whole contiguous fp32 [K,V] tile
//     (64 KB at K=V=128) into shared memory and one brings it back, so the bytes in flight per SM
//     are set by how many tiles fit in shared memory (three), not by the register file;
//   * the update runs in place in shared memory with the same ownership as above (lane owns rows
//     lane/8 + 4s of 4 adjacent columns: 128-bit, conflict-free accesses; reductions by register
//     sums and two shuffles);
//   * the CTA leaves as soon as the outgoing copy has read the tile (wait_group.read), the global
//     write itself drains asynchronously while the next CTA's load is already running.
// ------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(256) recurrent_bulk_kernel(RecParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    const int nh = blockIdx.x;
    const int n = nh / p.H, h = nh % p.H;
    const int K = p.K, V = p.V, H = p.H;
    float* sS = reinterpret_cast<float*>(smem_raw);             // [K][V]
    float* s_q = sS + (size_t)K * V;
    float* s_k = s_q + K;
    float* s_e = s_k + K;
    float* s_a = s_e + K;
    float* s_b = s_a + R * K;
    float* s_v = s_b + R * K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 3;
    const int c4 = (warp * 8 + (lane & 7)) * 4;
    const bool col_ok = c4 < V;
    const uint32_t tile_bytes = (uint32_t)K * V * 4u;

    long long bos, len;
    if (p.cu) { bos = p.cu[n]; len = p.cu[n + 1] - bos; }
    else      { bos = (long long)n * p.T; len = p.T; }
    bool state_ok = true;                                        // false once the wait for the state tile ran out

    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        sm100::fence_mbar_init();
        if (p.h0) {
            sm100::mbar_expect_tx(&bar, tile_bytes);
            sm100::bulk_g2s(sS, p.h0 + (size_t)nh * K * V, tile_bytes, &bar);
        }
    }
    if (!p.h0)
        for (int i = threadIdx.x; i < K * V / 4; i += blockDim.x)
            reinterpret_cast<float4*>(sS)[i] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (long long step = 0; step < len; ++step) {
        const long long t = p.reverse ? (bos + len - 1 - step) : (bos + step);
        const size_t tk = ((size_t)t * H + h) * K;
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            s_q[i] = ld_elem(p.q, tk + i, p.dt) * p.scale;
            s_k[i] = ld_elem(p.k, tk + i, p.dt);
            s_e[i] = __expf(ld_elem(p.gk, tk + i, p.gdt));
#pragma unroll
            for (int rr = 0; rr < R; ++rr) {
                const size_t ta = (((size_t)t * R + rr) * H + h) * K;
                s_a[rr * K + i] = ld_elem(p.a, ta + i, p.dt);
                s_b[rr * K + i] = ld_elem(p.b, ta + i, p.dt);
            }
        }
        for (int i = threadIdx.x; i < V; i += blockDim.x)
            s_v[i] = ld_elem(p.v, ((size_t)t * H + h) * V + i, p.dt);
        __syncthreads();
        if (step == 0 && p.h0) {                                 // bounded; the tile is in shared memory after it
            state_ok = __syncthreads_and(sm100::mbar_wait(&bar, 0) ? 1 : 0) != 0;
            if (!state_ok && threadIdx.x == 0) atomicExch(&g_recurrent_status, 1);
        }

        float sa[R][4];
#pragma unroll
        for (int rr = 0; rr < R; ++rr) { sa[rr][0] = sa[rr][1] = sa[rr][2] = sa[rr][3] = 0.f; }
        if (col_ok) {
            for (int kk = r; kk < K; kk += 4) {
                const float4 x = *reinterpret_cast<const float4*>(sS + (size_t)kk * V + c4);
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const float av = s_a[rr * K + kk];
                    sa[rr][0] = fmaf(av, x.x, sa[rr][0]); sa[rr][1] = fmaf(av, x.y, sa[rr][1]);
                    sa[rr][2] = fmaf(av, x.z, sa[rr][2]); sa[rr][3] = fmaf(av, x.w, sa[rr][3]);
                }
            }
        }
#pragma unroll
        for (int rr = 0; rr < R; ++rr)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sa[rr][j] += __shfl_xor_sync(0xffffffffu, sa[rr][j], 8);
                sa[rr][j] += __shfl_xor_sync(0xffffffffu, sa[rr][j], 16);
            }
        float oa[4] = {0.f, 0.f, 0.f, 0.f};
        if (col_ok) {
            const float vv[4] = {s_v[c4], s_v[c4 + 1], s_v[c4 + 2], s_v[c4 + 3]};
            for (int kk = r; kk < K; kk += 4) {
                float4* ps = reinterpret_cast<float4*>(sS + (size_t)kk * V + c4);
                const float4 x = *ps;
                const float e = s_e[kk], kv = s_k[kk], qv = s_q[kk];
                float y[4] = {fmaf(kv, vv[0], e * x.x), fmaf(kv, vv[1], e * x.y), fmaf(kv, vv[2], e * x.z),
                              fmaf(kv, vv[3], e * x.w)};
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const float bv = s_b[rr * K + kk];
#pragma unroll
                    for (int j = 0; j < 4; ++j) y[j] = fmaf(bv, sa[rr][j], y[j]);
                }
                *ps = make_float4(y[0], y[1], y[2], y[3]);
#pragma unroll
                for (int j = 0; j < 4; ++j) oa[j] = fmaf(qv, y[j], oa[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            oa[j] += __shfl_xor_sync(0xffffffffu, oa[j], 8);
            oa[j] += __shfl_xor_sync(0xffffffffu, oa[j], 16);
        }
        if (r == 0 && col_ok) {
            const size_t to = ((size_t)t * H + h) * V + c4;
            if (p.dt == HDLA_F32) {
                *reinterpret_cast<float4*>(static_cast<float*>(p.o) + to) = make_float4(oa[0], oa[1], oa[2], oa[3]);
            } else {
                uint2 pk;
                pk.x = sm100::pack_bf16(oa[0], oa[1]);
                pk.y = sm100::pack_bf16(oa[2], oa[3]);
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.o) + to) = pk;
            }
        }
        __syncthreads();                                         // vectors are single buffered
    }
    if (len == 0 && p.h0) {
        state_ok = __syncthreads_and(sm100::mbar_wait(&bar, 0) ? 1 : 0) != 0;
        if (!state_ok && threadIdx.x == 0) atomicExch(&g_recurrent_status, 1);
    }
    if (p.ht && state_ok) {                                      // a state that never arrived is not written back
        sm100::fence_proxy_async();
        __syncthreads();
        if (threadIdx.x == 0) {
            sm100::bulk_s2g(p.ht + (size_t)nh * K * V, sS, tile_bytes);
            sm100::bulk_commit();
            sm100::bulk_wait_read<0>();
        }
    }
}

template <int KT>
int launch_r(const RecParams& p, int R, int blocks, int threads, size_t smem, cudaStream_t st) {
    switch (R) {
        case 1: recurrent_fwd_kernel<KT, 1><<<blocks, threads, smem, st>>>(p); break;
        case 2: recurrent_fwd_kernel<KT, 2><<<blocks, threads, smem, st>>>(p); break;
        case 3: recurrent_fwd_kernel<KT, 3><<<blocks, threads, smem, st>>>(p); break;
        case 4: recurrent_fwd_kernel<KT, 4><<<blocks, threads, smem, st>>>(p); break;
        default: return fail(HDLA_ERR_UNSUPPORTED, "recurrent: rank R=%d not in 1..4", R);
    }
    return HDLA_OK;
}

}  // namespace

int recurrent_read_status(int* dst, cudaStream_t st) {
    void* sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_recurrent_status);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst, sym, sizeof(int), cudaMemcpyDefault, st);
    if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "recurrent status: %s", cudaGetErrorString(e));
    return HDLA_OK;
}

int recurrent_fwd_launch(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a,
                         const void* b, const void* gk, float scale, const float* h0, void* o, float* ht,
                         const int64_t* cu_seqlens, int n_seqs, int reverse, cudaStream_t st) {
    if (d.K > 256 || d.K < 1) return fail(HDLA_ERR_UNSUPPORTED, "recurrent: K=%d must be in 1..256", d.K);
    if (d.V % 4 != 0 || d.V > 256 || d.V < 4)
        return fail(HDLA_ERR_UNSUPPORTED, "recurrent: V=%d must be a multiple of 4 in 4..256", d.V);
    if (cu_seqlens && d.B != 1) return fail(HDLA_ERR_INVALID, "recurrent: cu_seqlens needs B == 1, got B=%d", d.B);
    const int N = cu_seqlens ? n_seqs : d.B;
    if (N <= 0) return fail(HDLA_ERR_INVALID, "recurrent: no sequences");
    RecParams p{q, k, v, a, b, gk, h0, o, ht, cu_seqlens, scale, d.T, d.H, d.K, d.V, d.dtype, d.gk_dtype, reverse};
    const int blocks = N * d.H;
    const int threads = 32 * ((d.V + 31) / 32);
    // few tokens per call: the bulk-copy staged kernel (state tile must fit in shared memory)
    const size_t tile = (size_t)d.K * d.V * 4;
    const long long tokens = cu_seqlens ? (long long)d.T : (long long)d.T;
    if (tokens <= 8 && tile <= 65536 && tile % 16 == 0 && d.R <= 4) {
        const size_t smem_b = tile + sizeof(float) * ((3 + 2 * d.R) * (size_t)d.K + d.V);
        static thread_local int attr_dev = -1;
        int dev = 0;
        cudaGetDevice(&dev);
        if (attr_dev != dev) {
            cudaError_t e = cudaFuncSetAttribute(recurrent_bulk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 + 16384);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(recurrent_bulk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 + 16384);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(recurrent_bulk_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 + 16384);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(recurrent_bulk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 + 16384);
            if (e != cudaSuccess) return fail(HDLA_ERR_CUDA, "recurrent: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            attr_dev = dev;
        }
        switch (d.R) {
            case 1: recurrent_bulk_kernel<1><<<blocks, threads, smem_b, st>>>(p); break;
            case 2: recurrent_bulk_kernel<2><<<blocks, threads, smem_b, st>>>(p); break;
            case 3: recurrent_bulk_kernel<3><<<blocks, threads, smem_b, st>>>(p); break;
            default: recurrent_bulk_kernel<4><<<blocks, threads, smem_b, st>>>(p); break;
        }
        HDLA_CHECK_LAUNCH("recurrent_bulk_kernel");
        return HDLA_OK;
    }
    const size_t smem = 2 * sizeof(float) * ((3 + 2 * d.R) * (size_t)d.K + d.V);
    int rc;
    if (d.K <= 32)       rc = launch_r<8>(p, d.R, blocks, threads, smem, st);
    else if (d.K <= 64)  rc = launch_r<16>(p, d.R, blocks, threads, smem, st);
    else if (d.K <= 128) rc = launch_r<32>(p, d.R, blocks, threads, smem, st);
    else                 rc = launch_r<64>(p, d.R, blocks, threads, smem, st);
    if (rc != HDLA_OK) return rc;
    HDLA_CHECK_LAUNCH("recurrent_fwd_kernel");
    return HDLA_OK;
}

}  // namespace hdla
