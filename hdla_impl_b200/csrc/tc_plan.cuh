// Shared declarations of the tensor-core (bf16) pipeline: tile constants, the workspace plan and
// the bounded-wait helpers.  Included by the kernel files of that pipeline only.
#pragma once
#include "tc_tiles.cuh"

namespace hdla {
namespace tc {

using namespace sm100;
using t8::Tile;

constexpr int C = 64, K = 128, V = 128, R = 2;
constexpr int CH64 = 16 * 64;      // chunks (16 B) of a [64 x 128] tile
constexpr int CH128 = 16 * 128;    // chunks of a [128 x 128] tile

// ------------------------------------------------------------------------------------------
// workspace plan (byte offsets)
// ------------------------------------------------------------------------------------------
struct TcPlan {
    int B, T, H, NT, BH;               // NT: chunks per sequence (all chunks of the packed batch with cu_seqlens);
    long long G;                       // BH: (sequence, head) pairs = scans and states;  G = tiles = H * chunks
    size_t status, Qh, Kh, Ah, Bh, Vc, E, ghat, Aqk, Aqb, Aak, Aab, M, W, P, U, Hs, V2, HT, zero;
    int nseg, seg_len;                 // two-level scan: segments per sequence, chunks per segment
    int lead_real;                     // the first segment in scan order is scanned for real in the first pass
    size_t Tseg, Fseg, Sin;            // per (b, h, segment): transition [K,K], state from zero [K,V], entering state [K,V]
    size_t dOc, dAqk, dAqb, DV2, DE, dgl, dW, dP, dAak, dAab;
    size_t dab, dab_half;              // in-operator a/b parametrisation: da then db, dab_half bytes each
    size_t total_fwd, total;
    int nseq;                          // sequences of a packed variable-length batch, 0 otherwise
    size_t chunk_tab, seq_tab;         // int2 per chunk: (first token, tokens);  int2 per sequence: (first chunk, chunks)
};

// Tokens of chunk n of the (packed) batch: from the chunk table of a variable-length batch, else uniform chunks.
__device__ __forceinline__ void chunk_tokens(const int2* chunk_tab, int n, int T, int& t0, int& valid) {
    if (chunk_tab) {
        const int2 e = chunk_tab[n];
        t0 = e.x; valid = e.y;
    } else {
        t0 = n * C; valid = min(C, T - t0);
    }
}

inline TcPlan make_tc_plan(const HdlaDims& d) {
    TcPlan p{};
    p.B = d.B; p.T = d.T; p.H = d.H;
    p.NT = (d.T + C - 1) / C;
    p.BH = d.B * d.H;
    p.nseq = 0;
    if (d.cu_seqlens && d.n_seqs > 0) {                    // packed sequences: chunks never straddle two of them
        p.nseq = d.n_seqs;
        long long nt = 0;
        for (int s_ = 0; s_ < d.n_seqs; ++s_) nt += (d.cu_seqlens[s_ + 1] - d.cu_seqlens[s_] + C - 1) / C;
        p.NT = (int)nt;
        p.BH = d.n_seqs * d.H;
    }
    p.G = (long long)d.B * d.H * p.NT;
    size_t off = 0;
    auto take = [&](size_t bytes_per_chunk) {
        size_t o = off;
        off += ((bytes_per_chunk * (size_t)p.G + 255) / 256) * 256;
        return o;
    };
    p.status = off; off += 256;
    p.chunk_tab = off; off += p.nseq ? (((size_t)p.NT * 8 + 255) / 256) * 256 : 0;
    p.seq_tab = off; off += p.nseq ? (((size_t)p.nseq * 8 + 255) / 256) * 256 : 0;
    // forward region: what the scan and the output kernel read.  The fused preparation kernel (HDLA_FLAG_FUSED_PREP)
    // keeps Aab on chip and writes Ah, Aak, M, P and the un-gating factors only for a backward pass, so with it
    // those live in the backward region; the four-kernel preparation passes them from kernel to kernel.
    // (it needs full head dims and does not form a and b itself)
    const bool fused = (d.flags & HDLA_FLAG_FUSED_PREP) != 0 && d.K == K && d.V == V && !(d.flags & HDLA_FLAG_PARAM_AB);
    p.Qh = take(16384); p.Kh = take(16384); p.Bh = take(32768); p.Vc = take(16384);
    p.E = take(K * 4);
    p.Aqk = take(8192); p.Aqb = take(16384);
    p.W = take(32768); p.U = take(32768); p.Hs = take(32768); p.V2 = take(32768);
    if (!fused) {
        p.Ah = take(32768); p.ghat = take(C * K * 2); p.Aak = take(16384); p.M = take(32768); p.P = take(32768);
        p.Aab = take(32768);
    }
    p.HT = off; off += (((size_t)p.BH * K * V * 4 + 255) / 256) * 256;
    p.zero = off; off += 32768;
    // Few (batch, head) pairs leave most SMs idle during the serial scan: cut each sequence into segments that
    // are scanned concurrently (transition + state-from-zero per segment, composed, then the real scan).
    // Two plans.  Phased calls (context parallelism) do not know the state entering the first segment, so every
    // segment needs both twins: nseg * 2 CTAs per (batch, head) in the first pass.  A complete call scans its
    // first segment for real in the first pass (from the given initial state), needs no twins for the last one,
    // and so fits more, shorter segments: 2 nseg - 3 CTAs per (batch, head).
    auto fit = [&](int nseg) {                           // -> no empty segment when NT is not a multiple
        const int len = (p.NT + nseg - 1) / nseg;
        return (p.NT + len - 1) / len;
    };
    int nseg_phased = 1;
    while (nseg_phased < 8 && 2 * p.BH * (nseg_phased * 2) <= 148 && p.NT / (nseg_phased * 2) >= 4) nseg_phased *= 2;
    nseg_phased = fit(nseg_phased);
    int nseg_all = 1;
    for (int n = 3; n <= 8; ++n)
        if (p.BH * (2 * n - 3) <= 148 && p.NT / n >= 4) nseg_all = n;
    nseg_all = fit(nseg_all);
    if (nseg_all < 3) nseg_all = 1;
    if (p.nseq) { nseg_all = 1; nseg_phased = 1; }           // sequences of different lengths: one scan per pair
    p.lead_real = (d.flags & HDLA_PHASE_MASK) == HDLA_PHASE_ALL && nseg_all > 1;
    p.nseg = (d.flags & HDLA_PHASE_MASK) == HDLA_PHASE_ALL ? nseg_all : nseg_phased;
    p.seg_len = (p.NT + p.nseg - 1) / p.nseg;
    const int nseg_max = nseg_all > nseg_phased ? nseg_all : nseg_phased;     // same offsets for both kinds of call
    const size_t slots = (size_t)p.BH * nseg_max;
    p.Tseg = off; off += nseg_max > 1 ? slots * K * K * 4 : 0;
    p.Fseg = off; off += nseg_max > 1 ? slots * K * V * 4 : 0;
    p.Sin = off; off += nseg_max > 1 ? slots * K * V * 4 : 0;
    p.total_fwd = off;
    // backward region: forward intermediates that only the backward kernels read, then the backward's own
    if (fused) {
        p.Ah = take(32768); p.ghat = take(C * K * 2); p.Aak = take(16384); p.M = take(32768); p.P = take(32768);
        p.Aab = 0;                                         // never leaves the SM
    }
    p.dOc = take(16384); p.dAqk = take(8192); p.dAqb = take(16384); p.DV2 = take(32768); p.DE = take(32768);
    p.dgl = take(K * 4); p.dW = take(32768); p.dP = take(32768); p.dAak = take(16384); p.dAab = take(32768);
    // in-operator a/b parametrisation: da and db, each [B, 2T, H, K] bf16 in the public layout, stay here for the
    // parametrisation's backward kernel
    p.dab_half = (((size_t)d.B * d.T * R * d.H * d.K * 2 + 255) / 256) * 256;
    p.dab = off; off += (d.flags & HDLA_FLAG_PARAM_AB) ? 2 * p.dab_half : 0;
    p.total = off;
    return p;
}

// The workspace starts with a 256-byte status block of int32 words written by the kernels:
//   word 0  code of a device-side wait that ran out (0 = none)
//   word 1  1 if some chunk's total log decay exceeds kMaxChunkDecay in some channel
//   word 2  the largest |total log decay of a chunk| seen, as the bit pattern of a non-negative float
constexpr int kStatusWait = 0, kStatusDecay = 1, kStatusMaxDecay = 2;

// The hat operands are scaled by up to e^{|g_last|/2}; beyond this total log decay per chunk and
// channel they leave the bf16/fp32 exponent range and the caller must use the fp32 pipeline.
constexpr float kMaxChunkDecay = 150.f;

// bounded wait on an mbarrier; records a failure in the device status word and carries on
__device__ __forceinline__ void wait_or_flag(uint64_t* bar, uint32_t parity, int* status, int code) {
    if (!mbar_wait(bar, parity)) {
        if (status) atomicExch(status, code);
    }
}

__device__ __forceinline__ void wait_idle_or_flag(uint64_t* bar, uint32_t parity, int* status, int code) {
    if (!mbar_wait_backoff(bar, parity)) {
        if (status) atomicExch(status, code);
    }
}

#ifdef HDLA_TIMELINE
// Optional tracing build (-DHDLA_TIMELINE): per-CTA time stamps of the last backward kernel's stages.
static __device__ unsigned long long g_timeline[16384 * 16];
__device__ __forceinline__ void tl_mark(long long g, int i) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (g < 16384) {
        g_timeline[g * 16 + i] = t;
        if (i == 0) {
            unsigned sm;
            asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
            g_timeline[g * 16 + 15] = sm;
        }
    }
}
#define TL(i) tl_mark(g, i)
// second trace, for the scan kernel (slot = linear CTA number)
static __device__ unsigned long long g_timeline_scan[4096 * 16];
__device__ __forceinline__ void tls_mark(int slot, int i) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (slot < 4096) g_timeline_scan[slot * 16 + i] = t;
}
#define TLS(i) do { if (threadIdx.x == 0) tls_mark((int)(blockIdx.x + gridDim.x * blockIdx.y), i); } while (0)
#else
#define TL(i)
#define TLS(i)
#endif


// Kernel launch through cudaLaunchKernelEx (errors are picked up by HDLA_CHECK_LAUNCH).  Launching the pipeline's
// kernels with programmatic stream serialisation (each kernel's prologue under the tail of the one before) was
// measured and left out: within noise at 8192 tiles, 2 % faster at 2048, 1.7 % slower at 1024.
template <typename... KArgs, typename... Args>
inline void launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace tc

// chunk_prep.cu: cumulative decay, hat operands, score matrices, inverse, Wh / u in one launch
int tc_launch_chunk_prep(const tc::TcPlan& pl, const HdlaDims& d, const void* q, const void* k, const void* v,
                         const void* a, const void* b, const void* gk, float scale, unsigned char* ws, bool save_bwd,
                         cudaStream_t st);

}  // namespace hdla
