// Instrumentation and test hooks (declared in include/hdla_debug.h): launch counter, optional
// per-kernel CUDA-event timing, dumps of intermediate buffers, and the wait-timeout probe.  This is
// the only translation unit of the library with process-wide mutable state.
#include <cstdio>
#include <cstring>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "../../include/hdla_debug.h"

namespace hdla {

static std::atomic<unsigned long long> g_launches{0};

// ---- optional per-kernel timing (benchmark instrumentation) -------------------------------------
// With timing on, an event is recorded on the call's stream at entry and after every launch; the
// time between consecutive events of one call is attributed to the kernel launched in between.
namespace {
struct Mark { const char* name; cudaEvent_t ev; };
std::mutex g_tmu;
bool g_timing = false;
std::vector<Mark> g_marks;
thread_local cudaStream_t g_cur_stream = nullptr;

void timing_mark(const char* name) {
    std::lock_guard<std::mutex> lock(g_tmu);
    if (!g_timing || g_marks.size() > (1u << 20)) return;
    cudaEvent_t ev;
    if (cudaEventCreate(&ev) != cudaSuccess) return;
    cudaEventRecord(ev, g_cur_stream);
    g_marks.push_back(Mark{name, ev});
}
}  // namespace

void count_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (g_timing) timing_mark(what);
}
void begin_call(cudaStream_t stream) {
    g_cur_stream = stream;
    if (g_timing) timing_mark(nullptr);
}


}  // namespace hdla

using namespace hdla;

extern "C" {

unsigned long long hdla_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

void hdla_timing_enable(int on) {
    std::lock_guard<std::mutex> lock(g_tmu);
    g_timing = on != 0;
}

size_t hdla_timing_report(char* buf, size_t size) {
    std::lock_guard<std::mutex> lock(g_tmu);
    std::map<std::string, std::pair<long long, double>> acc;
    for (size_t i = 0; i < g_marks.size(); ++i) {
        cudaEventSynchronize(g_marks[i].ev);
        if (g_marks[i].name && i > 0) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, g_marks[i - 1].ev, g_marks[i].ev) == cudaSuccess) {
                auto& e = acc[g_marks[i].name];
                e.first += 1;
                e.second += ms;
            }
        }
    }
    for (auto& m : g_marks) cudaEventDestroy(m.ev);
    g_marks.clear();
    std::string out;
    for (auto& kv : acc) {
        char line[256];
        snprintf(line, sizeof(line), "%s %lld %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        out += line;
    }
    if (buf && size) {
        const size_t n = out.size() < size - 1 ? out.size() : size - 1;
        memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return out.size();
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

int hdla_debug_wait_timeout(void* workspace, uint64_t budget_ns, void* cuda_stream) {
    if (!workspace) return fail(HDLA_ERR_INVALID, "debug_wait_timeout: workspace is null");
    begin_call(static_cast<cudaStream_t>(cuda_stream));
    return tc_wait_timeout_probe(static_cast<int*>(workspace), budget_ns, static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
