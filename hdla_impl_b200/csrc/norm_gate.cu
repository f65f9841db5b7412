// Output epilogue of the HDLA layer: gated RMS norm over the hidden row,
//   y = x * sigmoid(gate);  o = sqrt(D) * y / sqrt(sum(y^2) + eps) * weight
// (reference: RMSNormFusedGate with gate_act="sigmoid", gate_pos="pre", HRDPLR/normalizations/rms_norm.py:48-91,
//  arithmetic as in HRDPLR/normalizations/normalize/normalize/normalize_torch.py:9-99 with c = sqrt(D), no mean,
//  one group).  One CTA per row; forward and backward.  Bandwidth bound: x, gate read once, o written once.
#include "common.cuh"

namespace hdla {
namespace {

__device__ __forceinline__ float block_sum(float x, float* red) {
#pragma unroll
    for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += red[w];
    return t;
}

struct NgP {
    const void *x, *gate, *weight, *d_o;
    void *o, *dx, *dgate;
    float* dweight;            // fp32, accumulated with atomics (caller zeroes it)
    long long rows;
    int D, dt;
    float eps;
};

__global__ void __launch_bounds__(256) norm_gate_fwd_kernel(NgP p) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * p.D;
    float ss = 0.f;
    for (int c = threadIdx.x; c < p.D; c += blockDim.x) {
        const float y = ld_elem(p.x, base + c, p.dt) / (1.f + __expf(-ld_elem(p.gate, base + c, p.dt)));
        ss = fmaf(y, y, ss);
    }
    ss = block_sum(ss, red);
    const float r = sqrtf((float)p.D) * rsqrtf(ss + p.eps);
    for (int c = threadIdx.x; c < p.D; c += blockDim.x) {
        const float y = ld_elem(p.x, base + c, p.dt) / (1.f + __expf(-ld_elem(p.gate, base + c, p.dt)));
        st_elem(p.o, base + c, p.dt, y * r * ld_elem(p.weight, c, p.dt));
    }
}

__global__ void __launch_bounds__(256) norm_gate_bwd_kernel(NgP p) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * p.D;
    float ss = 0.f, uy = 0.f;
    for (int c = threadIdx.x; c < p.D; c += blockDim.x) {
        const float s = 1.f / (1.f + __expf(-ld_elem(p.gate, base + c, p.dt)));
        const float y = ld_elem(p.x, base + c, p.dt) * s;
        ss = fmaf(y, y, ss);
        uy = fmaf(ld_elem(p.weight, c, p.dt) * ld_elem(p.d_o, base + c, p.dt), y, uy);
    }
    ss = block_sum(ss, red);
    uy = block_sum(uy, red);
    const float cD = sqrtf((float)p.D);
    const float r = rsqrtf(ss + p.eps);
    const float k3 = cD * r * r * r * uy;
    for (int c = threadIdx.x; c < p.D; c += blockDim.x) {
        const float xv = ld_elem(p.x, base + c, p.dt);
        const float s = 1.f / (1.f + __expf(-ld_elem(p.gate, base + c, p.dt)));
        const float y = xv * s;
        const float dov = ld_elem(p.d_o, base + c, p.dt);
        const float dy = cD * r * ld_elem(p.weight, c, p.dt) * dov - k3 * y;
        st_elem(p.dx, base + c, p.dt, dy * s);
        st_elem(p.dgate, base + c, p.dt, dy * xv * s * (1.f - s));
        atomicAdd(p.dweight + c, cD * r * y * dov);
    }
}

}  // namespace

int norm_gate_launch(bool backward, const void* x, const void* gate, const void* weight, const void* d_o, void* o,
                     void* dx, void* dgate, float* dweight, long long rows, int D, float eps, int dt,
                     cudaStream_t st) {
    NgP p{x, gate, weight, d_o, o, dx, dgate, dweight, rows, D, dt, eps};
    if (backward) norm_gate_bwd_kernel<<<(unsigned)rows, 256, 0, st>>>(p);
    else norm_gate_fwd_kernel<<<(unsigned)rows, 256, 0, st>>>(p);
    HDLA_CHECK_LAUNCH(backward ? "norm_gate_bwd_kernel" : "norm_gate_fwd_kernel");
    return HDLA_OK;
}

}  // namespace hdla
