// extern "C" boundary of libhdla (declared in include/hdla.h): argument validation, dispatch,
// thread-local error text.  Nothing here allocates, frees or synchronises device memory.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <atomic>

#include "common.cuh"

namespace hdla {

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static int check_common(const HdlaDims* d, bool chunked) {
    if (!d) return fail(HDLA_ERR_INVALID, "dims is null");
    if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->K <= 0 || d->V <= 0 || d->R <= 0)
        return fail(HDLA_ERR_INVALID, "non-positive dimension: B=%d T=%d H=%d K=%d V=%d R=%d", d->B, d->T, d->H,
                    d->K, d->V, d->R);
    if (chunked && d->C <= 0) return fail(HDLA_ERR_INVALID, "chunk size C=%d must be positive", d->C);
    if (chunked && (d->C & (d->C - 1))) return fail(HDLA_ERR_UNSUPPORTED, "chunk size C=%d must be a power of two", d->C);
    if (d->dtype != HDLA_F32 && d->dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "dtype %d", d->dtype);
    if (d->gk_dtype != HDLA_F32 && d->gk_dtype != HDLA_BF16) return fail(HDLA_ERR_UNSUPPORTED, "gk_dtype %d", d->gk_dtype);
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

unsigned long long hdla_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

// bf16 problems the tensor-core pipeline supports use its workspace plan, everything else the fp32 one.
static size_t tc_region_bytes(const HdlaDims& d, int with_backward) {
    return tc_supported(d) ? tc_workspace_bytes(d, with_backward) : 0;
}

size_t hdla_chunk_workspace_bytes(const HdlaDims* dims, int with_backward) {
    if (check_common(dims, true) != HDLA_OK) return 0;
    const size_t simt = simt_workspace_floats(*dims, with_backward) * sizeof(float);
    if (simt == 0) return 0;
    if (tc_supported(*dims)) return tc_region_bytes(*dims, with_backward);
    return simt;
}

int hdla_debug_tc_buffer(const HdlaDims* dims, const void* workspace, const char* name, float* out,
                         void* cuda_stream) {
    int rc = check_common(dims, true);
    if (rc != HDLA_OK) return rc;
    if (!tc_supported(*dims)) return fail(HDLA_ERR_UNSUPPORTED, "no tensor-core workspace for these dims");
    if (!workspace || !name || !out) return fail(HDLA_ERR_INVALID, "debug_tc_buffer: null argument");
    return tc_debug_buffer(*dims, static_cast<const unsigned char*>(workspace), name, out,
                           static_cast<cudaStream_t>(cuda_stream));
}

int hdla_chunk_fwd(const HdlaDims* dims, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, void* o, float* ht, void* workspace,
                   size_t workspace_bytes, void* cuda_stream) {
    int rc = check_common(dims, true);
    if (rc != HDLA_OK) return rc;
    if (!q || !k || !v || !a || !b || !gk || !o) return fail(HDLA_ERR_INVALID, "chunk_fwd: null tensor pointer");
    rc = check_ws(dims, workspace, workspace_bytes, 0);
    if (rc != HDLA_OK) return rc;
    if (tc_supported(*dims))
        return tc_chunk_fwd(*dims, q, k, v, a, b, gk, scale, h0, o, ht, static_cast<unsigned char*>(workspace), true,
                            static_cast<cudaStream_t>(cuda_stream));
    return simt_chunk_fwd(*dims, q, k, v, a, b, gk, scale, h0, o, ht, static_cast<float*>(workspace), true,
                          static_cast<cudaStream_t>(cuda_stream));
}

int hdla_chunk_bwd(const HdlaDims* dims, const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0, const void* d_o, const float* dht, void* dq, void* dk,
                   void* dv, void* da, void* db, void* dgk, float* dh0, void* workspace, size_t workspace_bytes,
                   void* cuda_stream) {
    int rc = check_common(dims, true);
    if (rc != HDLA_OK) return rc;
    if (!q || !k || !v || !a || !b || !gk || !d_o || !dq || !dk || !dv || !da || !db || !dgk)
        return fail(HDLA_ERR_INVALID, "chunk_bwd: null tensor pointer");
    rc = check_ws(dims, workspace, workspace_bytes, 1);
    if (rc != HDLA_OK) return rc;
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
    if (!q || !k || !v || !a || !b || !gk || !o) return fail(HDLA_ERR_INVALID, "recurrent_fwd: null tensor pointer");
    return recurrent_fwd_launch(*dims, q, k, v, a, b, gk, scale, h0, o, ht, cu_seqlens, n_seqs, reverse,
                                static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
