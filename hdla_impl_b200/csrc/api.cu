// extern "C" boundary of libhdla (declared in include/hdla.h): argument validation, dispatch,
// thread-local error text.  Nothing here allocates, frees or synchronises device memory, and the only
// state kept between calls is the calling thread's last error text (instrumentation lives in debug.cu).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace hdla {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_common(const HdlaDims* d, bool chunked) {
    if (!d) return fail(HDLA_ERR_INVALID, "dims is null");
    if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->K <= 0 || d->V <= 0 || d->R <= 0)
        return fail(HDLA_ERR_INVALID, "non-positive dimension: B=%d T=%d H=%d K=%d V=%d R=%d", d->B, d->T, d->H,
                    d->K, d->V, d->R);
    if (chunked && d->C <= 0) return fail(HDLA_ERR_INVALID, "chunk size C=%d must be positive", d->C);
    if (chunked && (d->C & (d->C - 1))) return fail(HDLA_ERR_UNSUPPORTED, "chunk size C=%d must be a power of two", d->C);
    if (d->dtype != HDLA_F32 && d->dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "dtype %d", d->dtype);
    if (d->gk_dtype != HDLA_F32 && d->gk_dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "gk_dtype %d", d->gk_dtype);
    if (chunked && d->cu_seqlens) {
        if (d->B != 1) return fail(HDLA_ERR_INVALID, "cu_seqlens needs B == 1, got B=%d", d->B);
        if (d->n_seqs < 1) return fail(HDLA_ERR_INVALID, "cu_seqlens given with n_seqs=%d", d->n_seqs);
        if (d->cu_seqlens[0] != 0 || d->cu_seqlens[d->n_seqs] != d->T)
            return fail(HDLA_ERR_INVALID, "cu_seqlens must start at 0 and end at T=%d", d->T);
        for (int s = 0; s < d->n_seqs; ++s)
            if (d->cu_seqlens[s + 1] < d->cu_seqlens[s]) return fail(HDLA_ERR_INVALID, "cu_seqlens must not decrease");
    } else if (chunked && d->n_seqs != 0) {
        return fail(HDLA_ERR_INVALID, "n_seqs=%d without cu_seqlens", d->n_seqs);
    }
    return HDLA_OK;
}

static int check_ws(const HdlaDims* d, void* ws, size_t bytes, int with_backward) {
    const size_t need = hdla_chunk_workspace_bytes(d, with_backward);
    if (need == 0) return HDLA_ERR_UNSUPPORTED;      // message already set
    if (!ws) return fail(HDLA_ERR_WORKSPACE, "workspace is null");
    if (reinterpret_cast<uintptr_t>(ws) % 256) return fail(HDLA_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    if (bytes < need) return fail(HDLA_ERR_WORKSPACE, "workspace too small: %zu < %zu bytes", bytes, need);
    return HDLA_OK;
}

}  // namespace hdla

using namespace hdla;

extern "C" {

int hdla_version(void) { return HDLA_VERSION; }

const char* hdla_last_error(void) { return g_err; }

// bf16 problems the tensor-core pipeline supports use its workspace plan, everything else the fp32 one.
static size_t tc_region_bytes(const HdlaDims& d, int with_backward) {
    return tc_supported(d) ? tc_workspace_bytes(d, with_backward) : 0;
}

size_t hdla_chunk_workspace_bytes(const HdlaDims* dims, int with_backward) {
    if (check_common(dims, true) != HDLA_OK) return 0;
    if (dims->cu_seqlens && !tc_supported(*dims)) {
        fail(HDLA_ERR_UNSUPPORTED, "variable-length batches (cu_seqlens) need the bf16 tensor-core pipeline "
                                   "(bf16, chunk 64, R=2, K and V multiples of 8 up to 128)");
        return 0;
    }
    if ((dims->flags & HDLA_FLAG_NORM_K) && !(dims->flags & HDLA_FLAG_PARAM_AB)) {
        fail(HDLA_ERR_INVALID, "HDLA_FLAG_NORM_K needs HDLA_FLAG_PARAM_AB");
        return 0;
    }
    if ((dims->flags & HDLA_FLAG_PARAM_AB) && !tc_supported(*dims)) {
        fail(HDLA_ERR_UNSUPPORTED, "the in-operator a/b parametrisation (HDLA_FLAG_PARAM_AB) needs the bf16 tensor-core "
                                   "pipeline (bf16, chunk 64, R=2, K and V multiples of 8 up to 128)");
        return 0;
    }
    const size_t simt = simt_workspace_floats(*dims, with_backward) * sizeof(float);
    if (simt == 0) return 0;
    if (tc_supported(*dims)) return tc_region_bytes(*dims, with_backward);
    return simt;
}

int hdla_chunk_uses_tensor_cores(const HdlaDims* dims) {
    if (check_common(dims, true) != HDLA_OK) return 0;
    return tc_supported(*dims) ? 1 : 0;
}

int hdla_chunk_fwd(const HdlaDims* dims, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, void* o, float* ht, void* workspace,
                   size_t workspace_bytes, void* cuda_stream) {
    int rc = check_common(dims, true);
    if (rc != HDLA_OK) return rc;
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    const int phase = dims->flags & HDLA_PHASE_MASK;
    const bool needs_o = phase == HDLA_PHASE_ALL || phase == HDLA_PHASE_POST;
    const bool param_ab = (dims->flags & HDLA_FLAG_PARAM_AB) != 0;       // `a` is beta, `b` is not read
    if (!q || !k || !v || !a || (!b && !param_ab) || !gk || (needs_o && !o))
        return fail(HDLA_ERR_INVALID, "chunk_fwd: null tensor pointer");
    rc = check_ws(dims, workspace, workspace_bytes, phase == HDLA_PHASE_ALL ? 0 : 1);
    if (rc != HDLA_OK) return rc;
    if (phase != HDLA_PHASE_ALL && !tc_supported(*dims))
        return fail(HDLA_ERR_UNSUPPORTED, "phased calls need the bf16 tensor-core pipeline (bf16, chunk 64, R=2, K=V=128)");
    if (tc_supported(*dims))
        return tc_chunk_fwd(*dims, q, k, v, a, b, gk, scale, h0, o, ht, static_cast<unsigned char*>(workspace),
                            workspace_bytes, true, static_cast<cudaStream_t>(cuda_stream));
    return simt_chunk_fwd(*dims, q, k, v, a, b, gk, scale, h0, o, ht, static_cast<float*>(workspace), true,
                          static_cast<cudaStream_t>(cuda_stream));
}

int hdla_chunk_bwd(const HdlaDims* dims, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, const void* d_o, const float* dht, void* dq, void* dk,
                   void* dv, void* da, void* db, void* dgk, float* dh0, void* workspace, size_t workspace_bytes,
                   void* cuda_stream) {
    int rc = check_common(dims, true);
    if (rc != HDLA_OK) return rc;
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    const int phase = dims->flags & HDLA_PHASE_MASK;
    const bool needs_grads = phase == HDLA_PHASE_ALL || phase == HDLA_PHASE_POST;
    const bool param_ab = (dims->flags & HDLA_FLAG_PARAM_AB) != 0;       // `a` is beta, `da` dbeta; `b`, `db` unused
    if (!q || !k || !v || !a || (!b && !param_ab) || !gk || (phase != HDLA_PHASE_STATE && !d_o) ||
        (needs_grads && (!dq || !dk || !dv || !da || (!db && !param_ab) || !dgk)))
        return fail(HDLA_ERR_INVALID, "chunk_bwd: null tensor pointer");
    rc = check_ws(dims, workspace, workspace_bytes, 1);
    if (rc != HDLA_OK) return rc;
    if (phase != HDLA_PHASE_ALL && !tc_supported(*dims))
        return fail(HDLA_ERR_UNSUPPORTED, "phased calls need the bf16 tensor-core pipeline (bf16, chunk 64, R=2, K=V=128)");
    if (tc_supported(*dims))
        return tc_chunk_bwd(*dims, q, k, v, a, b, gk, scale, h0, d_o, dht, dq, dk, dv, da, db, dgk, dh0,
                            static_cast<unsigned char*>(workspace), static_cast<cudaStream_t>(cuda_stream));
    return simt_chunk_bwd(*dims, q, k, v, a, b, gk, scale, h0, d_o, dht, dq, dk, dv, da, db, dgk, dh0,
                          static_cast<float*>(workspace), static_cast<cudaStream_t>(cuda_stream));
}

int hdla_recurrent_fwd(const HdlaDims* dims, const void* q, const void* k, const void* v, const void* a,
                       const void* b, const void* gk, float scale, const float* h0, void* o, float* ht,
                       const int64_t* cu_seqlens, int32_t n_seqs, int32_t reverse, void* cuda_stream) {
    int rc = check_common(dims, false);
    if (rc != HDLA_OK) return rc;
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    if (!q || !k || !v || !a || !b || !gk || !o) return fail(HDLA_ERR_INVALID, "recurrent_fwd: null tensor pointer");
    return recurrent_fwd_launch(*dims, q, k, v, a, b, gk, scale, h0, o, ht, cu_seqlens, n_seqs, reverse,
                                static_cast<cudaStream_t>(cuda_stream));
}

int hdla_recurrent_read_status(int32_t* dst, void* cuda_stream) {
    if (!dst) return fail(HDLA_ERR_INVALID, "recurrent_read_status: dst is null");
    return recurrent_read_status(dst, static_cast<cudaStream_t>(cuda_stream));
}

int hdla_compose_states(const HdlaDims* dims, const float* T, const float* F, const float* S0, const float* pre,
                        const float* post, float* out, int32_t count, int64_t t_stride, int64_t f_stride,
                        int32_t reverse, void* cuda_stream) {
    int rc = check_common(dims, false);
    if (rc != HDLA_OK) return rc;
    if (dims->K != 128 || dims->V != 128)
        return fail(HDLA_ERR_UNSUPPORTED, "compose_states: K=%d V=%d (only K = V = 128)", dims->K, dims->V);
    if (count < 0 || !out || (count > 0 && (!T || !F)))
        return fail(HDLA_ERR_INVALID, "compose_states: null pointer or negative count");
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    return tc_compose_states(T, F, S0, pre, post, out, dims->B * dims->H, count, f_stride, t_stride, reverse,
                             static_cast<cudaStream_t>(cuda_stream));
}

int hdla_param_ab_fwd(const void* beta, const void* k, const void* log_f, void* a, void* b, int32_t B, int32_t T,
                      int32_t H, int32_t K, int32_t dtype, void* cuda_stream) {
    if (!beta || !k || !log_f || !a || !b) return fail(HDLA_ERR_INVALID, "param_ab_fwd: null tensor pointer");
    if (B <= 0 || T <= 0 || H <= 0 || K <= 0) return fail(HDLA_ERR_INVALID, "param_ab_fwd: non-positive dimension");
    if (dtype != HDLA_F32 && dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "dtype %d", dtype);
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    return param_ab_launch(false, beta, k, log_f, a, b, nullptr, nullptr, nullptr, B, T, H, K, dtype, dtype, 0, 0,
                           static_cast<cudaStream_t>(cuda_stream));
}

int hdla_param_ab_bwd(const void* beta, const void* k, const void* log_f, const void* da, const void* db, void* dbeta,
                      void* dk, void* dlog_f, int32_t B, int32_t T, int32_t H, int32_t K, int32_t dtype,
                      void* cuda_stream) {
    if (!beta || !k || !log_f || !da || !db || !dbeta || !dk || !dlog_f)
        return fail(HDLA_ERR_INVALID, "param_ab_bwd: null tensor pointer");
    if (B <= 0 || T <= 0 || H <= 0 || K <= 0) return fail(HDLA_ERR_INVALID, "param_ab_bwd: non-positive dimension");
    if (dtype != HDLA_F32 && dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "dtype %d", dtype);
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    return param_ab_launch(true, beta, k, log_f, const_cast<void*>(da), const_cast<void*>(db), dbeta, dk, dlog_f, B, T,
                           H, K, dtype, dtype, 0, 0, static_cast<cudaStream_t>(cuda_stream));
}

int hdla_norm_gate_fwd(const void* x, const void* gate, const void* weight, void* o, int64_t rows, int32_t D,
                       float eps, int32_t dtype, void* cuda_stream) {
    if (!x || !gate || !weight || !o) return fail(HDLA_ERR_INVALID, "norm_gate_fwd: null tensor pointer");
    if (rows <= 0 || D <= 0 || rows > 0x7fffffffLL) return fail(HDLA_ERR_INVALID, "norm_gate_fwd: bad size");
    if (dtype != HDLA_F32 && dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "dtype %d", dtype);
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    return norm_gate_launch(false, x, gate, weight, nullptr, o, nullptr, nullptr, nullptr, rows, D, eps, dtype,
                            static_cast<cudaStream_t>(cuda_stream));
}

int hdla_norm_gate_bwd(const void* x, const void* gate, const void* weight, const void* d_o, void* dx, void* dgate,
                       float* dweight, int64_t rows, int32_t D, float eps, int32_t dtype, void* cuda_stream) {
    if (!x || !gate || !weight || !d_o || !dx || !dgate || !dweight)
        return fail(HDLA_ERR_INVALID, "norm_gate_bwd: null tensor pointer");
    if (rows <= 0 || D <= 0 || rows > 0x7fffffffLL) return fail(HDLA_ERR_INVALID, "norm_gate_bwd: bad size");
    if (dtype != HDLA_F32 && dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "dtype %d", dtype);
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    return norm_gate_launch(true, x, gate, weight, d_o, nullptr, dx, dgate, dweight, rows, D, eps, dtype,
                            static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
