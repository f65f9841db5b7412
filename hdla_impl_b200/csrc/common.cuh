// Shared helpers for libhdla: error reporting, element-type access.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/hdla.h"

namespace hdla {

// Records a message for hdla_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// Process-wide count of kernel launches (see hdla_kernel_launches()); when kernel timing is on
// (hdla_timing_enable) it also records a CUDA event after the launch on the call's stream.
void count_launch(const char* what);
// Tells the instrumentation which stream the calling thread's current entry point launches on.
void begin_call(cudaStream_t stream);
// Validation shared by all entry points (api.cu).
int check_common(const HdlaDims* d, bool chunked);

#define HDLA_CHECK_LAUNCH(what)                                                       \
    do {                                                                              \
        ::hdla::count_launch(what);                                                   \
        cudaError_t e__ = cudaGetLastError();                                         \
        if (e__ != cudaSuccess)                                                       \
            return ::hdla::fail(HDLA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e__)); \
    } while (0)

// Effective chunk size: min(C, max(next_pow2(T), 16)).
static inline int effective_chunk(int T, int C) {
    int p2 = 1;
    while (p2 < T) p2 <<= 1;
    int lo = p2 > 16 ? p2 : 16;
    return C < lo ? C : lo;
}

// Runtime-typed element access (dt: HDLA_F32 | HDLA_BF16). The branch is warp-uniform.
__device__ __forceinline__ float ld_elem(const void* p, size_t i, int dt) {
    return dt == HDLA_F32 ? static_cast<const float*>(p)[i]
                          : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_elem(void* p, size_t i, int dt, float x) {
    if (dt == HDLA_F32) static_cast<float*>(p)[i] = x;
    else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
}

// Eight consecutive elements of a row (the index is a multiple of 8 and the base 16-byte aligned): requested as raw
// 16-byte pieces (one for bf16, two for fp32) so that a kernel can hold the request for its next row while it works
// on the current one, and turned into floats where they are used.
struct Raw8 { uint4 lo, hi; };
__device__ __forceinline__ Raw8 ld_raw8(const void* base, size_t i, int dt) {
    Raw8 r;
    if (dt == HDLA_F32) {
        r.lo = *reinterpret_cast<const uint4*>(static_cast<const float*>(base) + i);
        r.hi = *reinterpret_cast<const uint4*>(static_cast<const float*>(base) + i + 4);
    } else {
        r.lo = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + i);
        r.hi = make_uint4(0, 0, 0, 0);
    }
    return r;
}
__device__ __forceinline__ void raw8_to_float(const Raw8& r, int dt, float* f) {
    if (dt == HDLA_F32) {
        f[0] = __uint_as_float(r.lo.x); f[1] = __uint_as_float(r.lo.y); f[2] = __uint_as_float(r.lo.z); f[3] = __uint_as_float(r.lo.w);
        f[4] = __uint_as_float(r.hi.x); f[5] = __uint_as_float(r.hi.y); f[6] = __uint_as_float(r.hi.z); f[7] = __uint_as_float(r.hi.w);
    } else {
        const uint32_t w[4] = {r.lo.x, r.lo.y, r.lo.z, r.lo.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[2 * j] = __uint_as_float(w[j] << 16);
            f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}
__device__ __forceinline__ void ld_elem8(const void* base, size_t i, int dt, float* f) {
    raw8_to_float(ld_raw8(base, i, dt), dt, f);
}
__device__ __forceinline__ void st_elem8(void* base, size_t i, int dt, const float* f) {
    if (dt == HDLA_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(base) + i) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(static_cast<float*>(base) + i + 4) = make_float4(f[4], f[5], f[6], f[7]);
    } else {
        uint4 c;
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(f[0], f[1]); c.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(f[2], f[3]); c.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(f[4], f[5]); c.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(f[6], f[7]); c.w = *reinterpret_cast<uint32_t*>(&h);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + i) = c;
    }
}

// pipelines implemented in the other translation units
int recurrent_fwd_launch(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a,
                         const void* b, const void* gk, float scale, const float* h0, void* o, float* ht,
                         const int64_t* cu_seqlens, int n_seqs, int reverse, cudaStream_t st);

size_t simt_workspace_floats(const HdlaDims& d, int with_backward);
int simt_chunk_fwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, void* o, float* ht, float* ws, bool need_o,
                   cudaStream_t st);
int simt_chunk_bwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, const void* d_o, const float* dht, void* dq,
                   void* dk, void* dv, void* da, void* db, void* dgk, float* dh0, float* ws, cudaStream_t st);

int param_ab_launch(bool backward, const void* beta, const void* k, const void* log_f, void* a, void* b, void* dbeta,
                    void* dk, void* dlog_f, int B, int T, int H, int K, int dt, int gdt, int accumulate, int norm_k,
                    cudaStream_t st);

// eps of the layer's l2_norm of k (HRDPLR/normalizations/l2_norm.py:4): k / sqrt(sum_K k^2 + eps)
constexpr float kNormEps = 1e-5f;

int norm_gate_launch(bool backward, const void* x, const void* gate, const void* weight, const void* d_o, void* o,
                     void* dx, void* dgate, float* dweight, long long rows, int D, float eps, int dt, cudaStream_t st);

// tensor-core (bf16) pipeline, chunk_tc.cu
bool tc_supported(const HdlaDims& d);
size_t tc_workspace_bytes(const HdlaDims& d, int with_backward);
int tc_chunk_fwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                 const void* gk, float scale, const float* h0, void* o, float* ht, unsigned char* ws, size_t ws_bytes,
                 bool need_o, cudaStream_t st);
int tc_chunk_bwd(const HdlaDims& d, const void* q, const void* k, const void* v, const void* a, const void* b,
                 const void* gk, float scale, const float* h0, const void* d_o, const float* dht, void* dq, void* dk,
                 void* dv, void* da, void* db, void* dgk, float* dh0, unsigned char* ws, cudaStream_t st);
int tc_compose_states(const float* T, const float* F, const float* S0, const float* pre, const float* post,
                      float* out, int BH, int count, long long f_stride, long long t_stride, int reverse,
                      cudaStream_t st);
int tc_wait_timeout_probe(int* status, unsigned long long budget_ns, cudaStream_t st);
int recurrent_read_status(int* dst, cudaStream_t st);
int tc_debug_buffer(const HdlaDims& d, const unsigned char* ws, const char* name, float* out, cudaStream_t st);

}  // namespace hdla
