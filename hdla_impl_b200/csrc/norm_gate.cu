// Output epilogue of the HDLA layer: gated RMS norm over the hidden row,
//   y = x * sigmoid(gate);  o = sqrt(D) * y / sqrt(sum(y^2) + eps) * weight
// (reference: RMSNormFusedGate with gate_act="sigmoid", gate_pos="pre", HRDPLR/normalizations/rms_norm.py:48-91,
//  arithmetic as in HRDPLR/normalizations/normalize/normalize/normalize_torch.py:9-99 with c = sqrt(D), no mean,
//  one group).  The norm spans the whole hidden row (all heads of a token), so it is not local to a (chunk, head)
//  tile of the operator's output kernel and stays a kernel of its own.  Forward and backward; bandwidth bound:
//  x, gate (and do) are read once with 16-byte loads, o (dx, dgate) written once.
#include "common.cuh"

namespace hdla {
namespace {

struct NgP {
    const void *x, *gate, *weight, *d_o;
    void *o, *dx, *dgate;
    float* dweight;            // fp32, accumulated (caller zeroes it)
    long long rows;
    int D, dt;
    float eps;
};

// Two sums over the CTA at once (the second is ignored by the forward kernel).
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();                                   // the previous row's sums have been read
    if (lane == 0) red[warp] = make_float2(a, b);
    __syncthreads();
    float2 t = make_float2(0.f, 0.f);
    for (int w = 0; w < nw; ++w) { t.x += red[w].x; t.y += red[w].y; }
    return t;
}

// A CTA walks over rows (grid-stride); a thread owns the same 8-element column pieces in every row
// (piece j of thread t covers columns (t + j * 256) * 8 ..), so the row is read once with 16-byte loads, kept in
// registers between the reduction and the store, and -- in the backward kernel -- the thread's share of dweight is
// summed in registers over all the CTA's rows and added to global memory once per column and CTA.
// The number of pieces per thread is a template parameter so that a narrow row does not pay for the registers of a
// wide one (rows up to 2048 columns: one piece, 4 CTAs per SM in the backward kernel).
constexpr int kNgThreads = 256, kNgMaxPieces = 4;         // up to 256 * 4 * 8 = 8192 columns

template <int kNgPieces, int kDt>
__global__ void __launch_bounds__(kNgThreads) norm_gate_fwd_kernel(NgP p) {
    __shared__ float2 red[kNgThreads / 32];
    const int npiece = p.D / 8;
    float w[kNgPieces][8];
#pragma unroll
    for (int j = 0; j < kNgPieces; ++j) {
        const int pc = threadIdx.x + j * kNgThreads;
        if (pc < npiece) ld_elem8(p.weight, (size_t)pc * 8, kDt, w[j]);
    }
    const float cD = sqrtf((float)p.D);
    Raw8 nx[kNgPieces] = {}, ng[kNgPieces] = {};                       // the requests for the next row
    auto request = [&](long long row) {
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            const int pc = threadIdx.x + j * kNgThreads;
            if (pc < npiece && row < p.rows) {
                nx[j] = ld_raw8(p.x, (size_t)row * p.D + (size_t)pc * 8, kDt);
                ng[j] = ld_raw8(p.gate, (size_t)row * p.D + (size_t)pc * 8, kDt);
            }
        }
    };
    request(blockIdx.x);
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const size_t base = (size_t)row * p.D;
        float y[kNgPieces][8];
        float ss = 0.f;
        Raw8 cx[kNgPieces], cg[kNgPieces];
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) { cx[j] = nx[j]; cg[j] = ng[j]; }
        request(row + gridDim.x);
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            const int pc = threadIdx.x + j * kNgThreads;
            if (pc < npiece) {
                float g[8];
                raw8_to_float(cx[j], kDt, y[j]);
                raw8_to_float(cg[j], kDt, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    y[j][e] = y[j][e] / (1.f + __expf(-g[e]));
                    ss = fmaf(y[j][e], y[j][e], ss);
                }
            }
        }
        ss = block_sum2(ss, 0.f, red).x;
        const float r = cD * rsqrtf(ss + p.eps);
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            const int pc = threadIdx.x + j * kNgThreads;
            if (pc < npiece) {
                float out[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) out[e] = y[j][e] * r * w[j][e];
                st_elem8(p.o, base + (size_t)pc * 8, kDt, out);
            }
        }
    }
}

template <int kNgPieces, int kDt>
__global__ void __launch_bounds__(kNgThreads, (kNgPieces == 1 && kDt == HDLA_BF16) ? 4 : 1) norm_gate_bwd_kernel(NgP p) {
    __shared__ float2 red[kNgThreads / 32];
    const int npiece = p.D / 8;
    float w[kNgPieces][8], dw[kNgPieces][8];
#pragma unroll
    for (int j = 0; j < kNgPieces; ++j) {
        const int pc = threadIdx.x + j * kNgThreads;
        if (pc < npiece) ld_elem8(p.weight, (size_t)pc * 8, kDt, w[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) dw[j][e] = 0.f;
    }
    const float cD = sqrtf((float)p.D);
    Raw8 nx[kNgPieces] = {}, ng[kNgPieces] = {}, nd[kNgPieces] = {};        // the requests for the next row
    auto request = [&](long long row) {
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            const int pc = threadIdx.x + j * kNgThreads;
            if (pc < npiece && row < p.rows) {
                nx[j] = ld_raw8(p.x, (size_t)row * p.D + (size_t)pc * 8, kDt);
                ng[j] = ld_raw8(p.gate, (size_t)row * p.D + (size_t)pc * 8, kDt);
                nd[j] = ld_raw8(p.d_o, (size_t)row * p.D + (size_t)pc * 8, kDt);
            }
        }
    };
    request(blockIdx.x);
    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const size_t base = (size_t)row * p.D;
        float xv[kNgPieces][8], sg[kNgPieces][8], dov[kNgPieces][8];
        float ss = 0.f, uy = 0.f;
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            raw8_to_float(nx[j], kDt, xv[j]);
            raw8_to_float(ng[j], kDt, sg[j]);
            raw8_to_float(nd[j], kDt, dov[j]);
        }
        request(row + gridDim.x);
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            const int pc = threadIdx.x + j * kNgThreads;
            if (pc < npiece) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    sg[j][e] = 1.f / (1.f + __expf(-sg[j][e]));
                    const float y = xv[j][e] * sg[j][e];
                    ss = fmaf(y, y, ss);
                    uy = fmaf(w[j][e] * dov[j][e], y, uy);
                }
            }
        }
        const float2 t = block_sum2(ss, uy, red);
        const float r = rsqrtf(t.x + p.eps);
        const float k3 = cD * r * r * r * t.y;
#pragma unroll
        for (int j = 0; j < kNgPieces; ++j) {
            const int pc = threadIdx.x + j * kNgThreads;
            if (pc < npiece) {
                float dxo[8], dgo[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float s = sg[j][e], y = xv[j][e] * s;
                    const float dy = cD * r * w[j][e] * dov[j][e] - k3 * y;
                    dxo[e] = dy * s;
                    dgo[e] = dy * xv[j][e] * s * (1.f - s);
                    dw[j][e] = fmaf(cD * r * y, dov[j][e], dw[j][e]);
                }
                st_elem8(p.dx, base + (size_t)pc * 8, kDt, dxo);
                st_elem8(p.dgate, base + (size_t)pc * 8, kDt, dgo);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kNgPieces; ++j) {
        const int pc = threadIdx.x + j * kNgThreads;
        if (pc < npiece) {
            // two 16-byte vector reductions per piece instead of eight scalar ones (the grid's CTAs all arrive here
            // at about the same time, on the same D words)
            float* at = p.dweight + (size_t)pc * 8;
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                         ::"l"(at), "f"(dw[j][0]), "f"(dw[j][1]), "f"(dw[j][2]), "f"(dw[j][3]) : "memory");
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                         ::"l"(at + 4), "f"(dw[j][4]), "f"(dw[j][5]), "f"(dw[j][6]), "f"(dw[j][7]) : "memory");
        }
    }
}

}  // namespace

int norm_gate_launch(bool backward, const void* x, const void* gate, const void* weight, const void* d_o, void* o,
                     void* dx, void* dgate, float* dweight, long long rows, int D, float eps, int dt,
                     cudaStream_t st) {
    if (D % 8 != 0 || D > kNgThreads * kNgMaxPieces * 8)
        return fail(HDLA_ERR_UNSUPPORTED, "norm_gate: D=%d must be a multiple of 8 up to %d", D, kNgThreads * kNgMaxPieces * 8);
    for (const void* q : {x, gate, weight, d_o, (const void*)o, (const void*)dx, (const void*)dgate, (const void*)dweight})
        if (reinterpret_cast<uintptr_t>(q) % 16 != 0) return fail(HDLA_ERR_INVALID, "norm_gate: tensors must be 16-byte aligned");
    NgP p{x, gate, weight, d_o, o, dx, dgate, dweight, rows, D, dt, eps};
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const int pieces = (D / 8 + kNgThreads - 1) / kNgThreads;
    void (*kern)(NgP) = nullptr;
    if (dt == HDLA_F32)
        kern = backward ? (pieces <= 1 ? norm_gate_bwd_kernel<1, HDLA_F32> : pieces <= 2 ? norm_gate_bwd_kernel<2, HDLA_F32> : norm_gate_bwd_kernel<4, HDLA_F32>)
                        : (pieces <= 1 ? norm_gate_fwd_kernel<1, HDLA_F32> : pieces <= 2 ? norm_gate_fwd_kernel<2, HDLA_F32> : norm_gate_fwd_kernel<4, HDLA_F32>);
    else
        kern = backward ? (pieces <= 1 ? norm_gate_bwd_kernel<1, HDLA_BF16> : pieces <= 2 ? norm_gate_bwd_kernel<2, HDLA_BF16> : norm_gate_bwd_kernel<4, HDLA_BF16>)
                        : (pieces <= 1 ? norm_gate_fwd_kernel<1, HDLA_BF16> : pieces <= 2 ? norm_gate_fwd_kernel<2, HDLA_BF16> : norm_gate_fwd_kernel<4, HDLA_BF16>);
    // persistent: as many CTAs as are resident at once, every CTA walks over many rows
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kNgThreads, 0) != cudaSuccess || per_sm <= 0) per_sm = 1;
    const long long cap = (long long)sms * per_sm;
    const unsigned grid = (unsigned)(rows < cap ? rows : cap);
    kern<<<grid, kNgThreads, 0, st>>>(p);
    HDLA_CHECK_LAUNCH(backward ? "norm_gate_bwd_kernel" : "norm_gate_fwd_kernel");
    return HDLA_OK;
}

}  // namespace hdla
