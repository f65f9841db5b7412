/*
 * hdla_debug.h -- instrumentation and test hooks of libhdla.  None of these belongs to the operator: they count
 * and time the library's kernel launches for benchmarks, expose intermediate buffers to the stage-by-stage
 * parity tests, and let a test exercise the device-side timeout path.  None has a counterpart in the reference
 * (its launches are issued by the Triton runtime and its intermediates are ordinary torch tensors).
 */
#ifndef HDLA_DEBUG_H_
#define HDLA_DEBUG_H_

#include "hdla.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Number of kernels this library has launched in the calling process so far (all threads). */
HDLA_API unsigned long long hdla_kernel_launches(void);

/* Per-kernel timing.  While enabled, every call records a CUDA event on its stream at entry and after each
 * kernel launch.  hdla_timing_report() WAITS for those events, writes one line "kernel_name launches total_ms"
 * per kernel into buf (at most size-1 characters, NUL terminated), forgets the events and returns the length of
 * the full report. */
HDLA_API void hdla_timing_enable(int on);
HDLA_API size_t hdla_timing_report(char* buf, size_t size);

/* Converts one named bf16 tile buffer of the tensor-core workspace ("Qh","Kh","Ah","Bh","Vc","Aqk","Aqb","Aak",
 * "M","W","P","U","Hs","V2","dOc","dAqk","dAqb","DV2","DE","dW","dP","dAak","dAab") to fp32 row-major
 * [B*H*NT][rows][cols] in `out` (device memory), or copies "E" / "dgl" / the "status" words. */
HDLA_API int hdla_debug_tc_buffer(const HdlaDims* dims, const void* workspace, const char* name, float* out,
                                  void* cuda_stream);

/* Launches a one-CTA kernel that waits, for at most budget_ns nanoseconds, on an mbarrier nothing ever arrives
 * at, and then records wait code 99 in status word 0 of `workspace` exactly as the pipeline's kernels do.  The
 * kernel returns normally; nothing faults.  For testing that a device-side timeout reaches the host as an
 * error and leaves the context usable. */
HDLA_API int hdla_debug_wait_timeout(void* workspace, uint64_t budget_ns, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* HDLA_DEBUG_H_ */
