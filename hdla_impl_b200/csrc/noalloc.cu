// hdla_chunk_fwd_noalloc: the chunked forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot reach an allocator at the moment they need the operator: an
// inference server that hands its plugins a fixed set of buffers and owns the rest of the device, a
// serving loop whose policy forbids any allocation once traffic has started (an allocation may
// synchronise the device or fail under memory pressure), or code that is already running where
// cudaMalloc is not permitted.  hdla_chunk_fwd() needs a caller-provided workspace; for those
// callers the workspace is instead a fixed array that lives inside the library image on every GPU
// that loads it.  Nothing else differs: the same kernels run on that array.
#include <mutex>

#include "common.cuh"

namespace {

// Scratch for one forward call.  Every device that loads the library holds these bytes until the
// process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HDLA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// In host code `g_noalloc_scratch` is only a handle, not a device address: resolve it once per
// device, with that device current.  The first resolution on a device is also the moment the CUDA
// runtime loads this library's device code there and reserves the array (nothing is allocated later).
int scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return hdla::fail(HDLA_ERR_CUDA, "noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return hdla::fail(HDLA_ERR_UNSUPPORTED, "noalloc: device index %d", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr)
            return hdla::fail(HDLA_ERR_CUDA, "noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return HDLA_OK;
}

}  // namespace

extern "C" int hdla_chunk_fwd_noalloc(const HdlaDims* dims, const void* q, const void* k, const void* v,
                                      const void* a, const void* b, const void* gk, float scale, const float* h0,
                                      void* o, float* ht, void* cuda_stream) {
    int rc = hdla::check_common(dims, true);                    // null or malformed dims: HDLA_ERR_INVALID / _UNSUPPORTED
    if (rc != HDLA_OK) return rc;
    const size_t need = hdla_chunk_workspace_bytes(dims, 0);
    if (need == 0) return HDLA_ERR_UNSUPPORTED;                 // hdla_last_error() already says why
    if (need > (size_t)HDLA_NOALLOC_SCRATCH_BYTES)
        return hdla::fail(HDLA_ERR_WORKSPACE,
                          "hdla_chunk_fwd_noalloc: this problem needs %zu bytes of scratch but the built-in scratch "
                          "holds %zu; use hdla_chunk_fwd with a caller-provided workspace",
                          need, (size_t)HDLA_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    rc = scratch_for_current_device(&scratch);
    if (rc != HDLA_OK) return rc;
    // The array keeps whatever the previous call left. The kernels overwrite everything they read
    // except the leading status block, which must start at zero.
    cudaError_t e = cudaMemsetAsync(scratch, 0, 256, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return hdla::fail(HDLA_ERR_CUDA, "noalloc: clearing the status block: %s", cudaGetErrorString(e));
    return hdla_chunk_fwd(dims, q, k, v, a, b, gk, scale, h0, o, ht, scratch, (size_t)HDLA_NOALLOC_SCRATCH_BYTES,
                          cuda_stream);
}

// The kernels report through status words at the start of their workspace (include/hdla.h); callers
// of hdla_chunk_fwd_noalloc have no workspace pointer, so this copies the words out of the array.
extern "C" int hdla_noalloc_read_status(int32_t* dst, void* cuda_stream) {
    if (!dst) return hdla::fail(HDLA_ERR_INVALID, "hdla_noalloc_read_status: dst is null");
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != HDLA_OK) return rc;
    cudaError_t e = cudaMemcpyAsync(dst, scratch, 3 * sizeof(int32_t), cudaMemcpyDefault,
                                    static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return hdla::fail(HDLA_ERR_CUDA, "noalloc: reading the status words: %s", cudaGetErrorString(e));
    return HDLA_OK;
}
