/*
 * hdla.h -- C ABI of libhdla: the HDLA rank-R diagonal-plus-low-rank delta-rule operator for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes.  The caller owns all memory
 * (inputs, outputs and the workspace whose size hdla_chunk_workspace_bytes() reports); the
 * library never allocates, frees or synchronises, and enqueues all work on the stream it is
 * given.  Functions return 0 on success and a negative HDLA_ERR_* code otherwise; they never
 * throw, abort or trap.  hdla_last_error() returns a description of the calling thread's last
 * failure.
 *
 * Tensor layouts (dense, row-major; identical to the reference operator's,
 * HRDPLR/hrdplr.py:286-300 and HRDPLR/recurrent.py:227-241):
 *     q, k, gk : [B, T,   H, K]
 *     v, o     : [B, T,   H, V]
 *     a, b     : [B, T*R, H, K]     row t*R + r  (time major, rank minor)
 *     states   : [N, H, K, V] fp32  (N = B, or the number of sequences with cu_seqlens)
 * gk is a LOG decay (<= 0).  R is the rank of the low-rank term (2 for HDLA).
 */
#ifndef HDLA_H_
#define HDLA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HDLA_VERSION 102

#if defined(__GNUC__)
#define HDLA_API __attribute__((visibility("default")))
#else
#define HDLA_API
#endif

/* element types of q,k,v,a,b,o and their gradients (dtype) and of gk/dgk (gk_dtype) */
#define HDLA_F32  0
#define HDLA_BF16 1

/* error codes */
#define HDLA_OK                 0
#define HDLA_ERR_INVALID       -1   /* null pointer, non-positive size, inconsistent shapes      */
#define HDLA_ERR_UNSUPPORTED   -2   /* shape or dtype outside what the kernels are built for     */
#define HDLA_ERR_WORKSPACE     -3   /* workspace pointer null/misaligned or too small            */
#define HDLA_ERR_CUDA          -4   /* a CUDA runtime call or kernel launch reported an error    */

/* flags of HdlaDims.flags */
#define HDLA_FLAG_WS_HOLDS_FWD  1   /* hdla_chunk_bwd: the workspace still holds what hdla_chunk_fwd
                                       left there for the same inputs -> skip the recomputation  */
#define HDLA_FLAG_FORCE_SIMT    2   /* use the fp32 CUDA-core pipeline even for bf16 inputs       */
#define HDLA_FLAG_FUSED_PREP    4   /* bf16 tensor-core pipeline: run everything before the scan (cumulative decay,
                                       hat operands, score matrices, WY inverse, w/u) as ONE kernel per tile instead
                                       of four.  It moves 38 % fewer bytes and needs a smaller forward workspace,
                                       but runs about 5 % slower on large problems (two CTAs of four warps per SM do
                                       not hide its latencies); the workspace layout depends on it, so a forward
                                       and its backward must agree on the flag.                                   */

#define HDLA_FLAG_PARAM_AB      8   /* bf16 tensor-core pipeline: the layer's a/b parametrisation
                                       (HRDPLR/hdla_custom.py:19-43, called at :290) happens inside the operator.
                                       Argument `a` then points to beta [B,T,H] (dtype of q), `b` is ignored (may
                                       be null) and gk is the layer's log_f; the preparation kernel forms
                                         a_{t,1} = -beta k,  a_{t,2} = -beta k (e^{log_f} + s),  s = -beta sum_K e^{log_f} k^2,
                                         b_{t,1} = e^{log_f} k,  b_{t,2} = k
                                       in fp32 on the way to its operand tiles, so a and b never exist in memory.
                                       hdla_chunk_bwd with the flag writes dbeta [B,T,H] through `da`, ignores `db`,
                                       and dk and dgk (= dlog_f) contain the parametrisation's share (its backward
                                       runs as one more kernel over gradients kept in the workspace).  A forward
                                       and its backward must agree on the flag; problems outside the tensor-core
                                       pipeline report HDLA_ERR_UNSUPPORTED (use hdla_param_ab_fwd/_bwd there).   */

#define HDLA_FLAG_NORM_K       256   /* with HDLA_FLAG_PARAM_AB: k arrives un-normalised and the layer's l2_norm of k
                                       (HRDPLR/hdla_custom.py:248; k / sqrt(sum_K k^2 + 1e-5), normalizations/l2_norm.py:4)
                                       happens in the preparation kernel too; backward's dk is the gradient of the
                                       un-normalised k.                                                              */

/* Phase selector (bits 4..7 of HdlaDims.flags), for callers that split a sequence over devices
 * (context parallelism).  Only the inter-chunk scan depends on the incoming state, so a call can be cut:
 *   PHASE_ALL         the whole forward / backward (default)
 *   PHASE_PRE         forward: everything before the scan;  backward: the stage before the reverse scan
 *   PHASE_TRANSITION  forward only: ht <- product of the chunk transition matrices [B,H,K,K] (needs K == V);
 *                     the state after this call is  ht_transition * S_in + (state pass from S_in = 0),
 *                     the state gradient before it  ht_transition^T * dS_out + (state pass from dS_out = 0)
 *   PHASE_STATE       forward: ht <- state after this call's chunks from h0, nothing else written;
 *                     backward: dh0 <- state gradient entering this call's first chunk from dht
 *   PHASE_POST        forward: scan + output;  backward: reverse scan + all gradients
 * Phased calls use one workspace (sized with_backward = 1) across all phases, in the order PRE, TRANSITION,
 * STATE, POST (forward) and PRE, STATE, POST (backward): later phases reuse what earlier ones left in the
 * workspace (for long slices the scan itself is split into concurrently scanned segments whose affine maps
 * are kept there).  Backward phases need HDLA_FLAG_WS_HOLDS_FWD.  The bf16 tensor-core pipeline implements them; other problems report
 * HDLA_ERR_UNSUPPORTED. */
#define HDLA_PHASE_MASK        0xF0
#define HDLA_PHASE_ALL         0x00
#define HDLA_PHASE_PRE         0x10
#define HDLA_PHASE_TRANSITION  0x20
#define HDLA_PHASE_STATE       0x30
#define HDLA_PHASE_POST        0x40

typedef struct HdlaDims {
    int32_t B;         /* batch (sequences)                                   */
    int32_t T;         /* tokens per sequence                                 */
    int32_t H;         /* heads                                               */
    int32_t K;         /* key/query head dim                                  */
    int32_t V;         /* value head dim                                      */
    int32_t R;         /* rank of the a/b term                                */
    int32_t C;         /* chunk size as passed by the caller; the effective chunk is
                          min(C, max(next_pow2(T), 16))  (HRDPLR/hrdplr.py:42)  */
    int32_t dtype;     /* HDLA_F32 | HDLA_BF16 for q,k,v,a,b,o,do and dq..db   */
    int32_t gk_dtype;  /* HDLA_F32 | HDLA_BF16 for gk and dgk                  */
    int32_t flags;     /* HDLA_FLAG_*                                          */
    /* Variable-length batches for the chunked entry points (packed sequences, as in the reference's chunk kernels,
     * HRDPLR/fwd_triton.py:618-623 and HRDPLR/bwd_triton.py:919-924): with cu_seqlens != NULL, B must be 1, T is the
     * total number of tokens, sequence s holds tokens [cu_seqlens[s], cu_seqlens[s+1]) and has its own state, so h0 /
     * ht / dht / dh0 are [n_seqs, H, K, V].  cu_seqlens is a HOST array of n_seqs + 1 offsets (the library sizes its
     * grids from it); it only needs to live for the duration of the call.  The bf16 tensor-core pipeline implements
     * this; other problems report HDLA_ERR_UNSUPPORTED.  hdla_recurrent_fwd takes its own (device) cu_seqlens
     * argument and ignores these two fields. */
    int32_t n_seqs;    /* number of sequences, 0 without cu_seqlens            */
    int32_t reserved_; /* keep 0                                               */
    const int64_t* cu_seqlens;
} HdlaDims;

/* Library version (HDLA_VERSION of the build). */
HDLA_API int hdla_version(void);

/* Text of the calling thread's most recent error ("" if none). The pointer stays valid until
 * the same thread's next failing call. */
HDLA_API const char* hdla_last_error(void);

/* Bytes of device workspace hdla_chunk_fwd (with_backward = 0) or the pair hdla_chunk_fwd +
 * hdla_chunk_bwd (with_backward = 1) needs for these dims; 0 if the dims are unsupported (see
 * hdla_last_error).  Replaces the torch.empty(...) intermediates the reference's stage
 * wrappers allocate: HRDPLR/fwd_func.py:40-43,69-72,131-132,198,243-245,296 and
 * HRDPLR/bwd_func.py:33-36,84-86,139,181-185,238-241,300-309. */
HDLA_API size_t hdla_chunk_workspace_bytes(const HdlaDims* dims, int with_backward);

/* 1 if hdla_chunk_fwd / hdla_chunk_bwd run these dims on the bf16 tensor-core pipeline (and so write the status
 * words described below), 0 if on the fp32 CUDA-core pipeline.  No counterpart in the reference. */
HDLA_API int hdla_chunk_uses_tensor_cores(const HdlaDims* dims);

/* The first 12 bytes of a workspace used by the bf16 tensor-core pipeline are three int32 status words
 * written by the kernels:
 *   word 0  non-zero if a bounded device-side wait ran out (results invalid); the value names the wait
 *   word 1  non-zero if some chunk's total log decay |sum_chunk gk| exceeded 150 in some channel, which the
 *           bf16 pipeline cannot represent (results invalid; rerun with HDLA_FLAG_FORCE_SIMT, whose fp32
 *           pipeline has no such limit)
 *   word 2  the largest |sum_chunk gk| over all chunks and channels of the call, as the bit pattern of a float
 * Callers read them after the stream has finished the call (hdla_chunk_fwd_noalloc, which has no caller
 * workspace: hdla_noalloc_read_status).  Every device-side wait is bounded in time (2 s on the GPU's
 * nanosecond timer), so a kernel always returns. */

/* Chunked forward.  Replaces chunk_hrdplr_fwd (HRDPLR/hrdplr.py:25-99), i.e. the stage
 * sequence cumsum -> intra-chunk A matrices -> (I-Aab)^-1 and w/u -> state scan -> output.
 *   h0  : [B,H,K,V] fp32 initial state or NULL (zero state)
 *   o   : [B,T,H,V] in dims->dtype
 *   ht  : [B,H,K,V] fp32 final state or NULL
 * The workspace must be 256-byte aligned.  With a workspace sized for backward the forward
 * intermediates stay in it for hdla_chunk_bwd(HDLA_FLAG_WS_HOLDS_FWD). */
HDLA_API int hdla_chunk_fwd(const HdlaDims* dims,
                   const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0,
                   void* o, float* ht,
                   void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Chunked forward without a caller workspace: same computation and arguments as hdla_chunk_fwd,
 * but the scratch memory is a fixed array of HDLA_NOALLOC_SCRATCH_BYTES built into the library
 * (resident on every GPU that loads the library, until the process exits).  It exists for callers
 * that cannot allocate device memory when they need the operator -- plugins of a server that owns
 * the device memory, serving loops with a no-allocation policy, code running where cudaMalloc is
 * not allowed -- and performs no allocation of any kind.  It has no counterpart in the reference,
 * whose wrappers allocate their intermediates with torch.empty.
 *   - Problems whose workspace (hdla_chunk_workspace_bytes(dims, 0)) exceeds the built-in scratch are
 *     rejected with HDLA_ERR_WORKSPACE and an explanatory hdla_last_error().
 *   - The first call on each device resolves the array's device address, which also makes the CUDA runtime load
 *     this library's device code on that device and reserve the array there (it may synchronise the device or
 *     fail if the device has no room left); make that first call with the device current, before starting any
 *     stream capture and before the no-allocation regime begins.  Later calls allocate nothing.
 *   - The status words described above live in the array's first bytes; hdla_noalloc_read_status() copies them
 *     out.
 *   - All calls on a device share the one array, which keeps the previous call's contents: calls whose
 *     GPU work can overlap (different streams, different threads) race with each other.  Issue them
 *     on one stream, or order them yourself. */
#define HDLA_NOALLOC_SCRATCH_BYTES (64u << 20)
HDLA_API int hdla_chunk_fwd_noalloc(const HdlaDims* dims,
                   const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0,
                   void* o, float* ht, void* cuda_stream);

/* Enqueues on the stream a copy of the three status words that the most recent hdla_chunk_fwd_noalloc call on
 * the current device left in the built-in scratch to dst (3 x int32; device memory or pinned host memory).
 * Allocates nothing.  Like hdla_chunk_fwd_noalloc it has no counterpart in the reference. */
HDLA_API int hdla_noalloc_read_status(int32_t* dst, void* cuda_stream);

/* Chunked backward.  Replaces ChunkDPLRDeltaRuleFunction.backward (HRDPLR/hrdplr.py:146-284):
 * stages dAu, dhu (reverse state scan), dv, bwd_o, wy, intra and dgk.
 *   d_o  : [B,T,H,V] gradient of o (dims->dtype);  dht: [B,H,K,V] fp32 gradient of the final
 *          state or NULL
 *   dq,dk,dv,da,db in dims->dtype, dgk in dims->gk_dtype, shaped like their inputs
 *   dh0 : [B,H,K,V] fp32 or NULL
 * Unless HDLA_FLAG_WS_HOLDS_FWD is set the forward intermediates are recomputed first (what
 * the reference always does, HRDPLR/hrdplr.py:161-198). */
HDLA_API int hdla_chunk_bwd(const HdlaDims* dims,
                   const void* q, const void* k, const void* v, const void* a, const void* b,
                   const void* gk, float scale, const float* h0,
                   const void* d_o, const float* dht,
                   void* dq, void* dk, void* dv, void* da, void* db, void* dgk, float* dh0,
                   void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Fused recurrent forward (decode / short prefill).  Replaces
 * fused_recurrent_dplr_delta_rule_fwd (HRDPLR/recurrent.py:121-177) and its kernel (:10-119).
 *   dims->T : tokens per sequence (total tokens when cu_seqlens is given, in which case
 *             dims->B must be 1); dims->C is ignored
 *   h0      : [N,H,K,V] fp32 or NULL;  ht: [N,H,K,V] fp32 or NULL.  ht may alias h0 (in-place
 *             state update).
 *   cu_seqlens : device pointer to n_seqs+1 int64 offsets or NULL (then n_seqs is ignored)
 *   reverse : process tokens from last to first (HRDPLR/recurrent.py:64,108)
 * Needs no workspace. */
HDLA_API int hdla_recurrent_fwd(const HdlaDims* dims,
                       const void* q, const void* k, const void* v, const void* a, const void* b,
                       const void* gk, float scale, const float* h0,
                       void* o, float* ht,
                       const int64_t* cu_seqlens, int32_t n_seqs, int32_t reverse,
                       void* cuda_stream);

/* Enqueues a copy of the decode kernel's status word to dst (1 x int32; device or pinned host memory): non-zero
 * once a bounded wait for a state tile ran out in some hdla_recurrent_fwd call of this process on the current
 * device (that call's outputs are invalid and its final state was not written).  No counterpart in the
 * reference, whose kernel has no asynchronous copies to wait for. */
HDLA_API int hdla_recurrent_read_status(int32_t* dst, void* cuda_stream);

/* Composition of affine state maps, for callers that cut a sequence over devices (context parallelism; the
 * reference has no counterpart, its scan HRDPLR/fwd_triton.py:853-956 is serial over the whole sequence).
 * The state leaving a slice is affine in the state entering it, S_out = T S_in + F (T from
 * HDLA_PHASE_TRANSITION, F from HDLA_PHASE_STATE).  With the maps of `count` consecutive slices gathered in
 * local memory this computes, per (batch, head) pair bh and in fp32,
 *     forward (reverse = 0):  X = S0;  for s = 0 .. count-1:      X = T_s (X + pre_s) + F_s
 *     reverse (reverse = 1):  X = S0;  for s = count-1 .. 0:      X = T_s^T (X + pre_s) + F_s
 *     out = X + post
 * T_s of pair bh is the K x K matrix at T + (s * t_stride + bh) * K*K, F_s and pre_s the K x V matrices at
 * F / pre + (s * f_stride + bh) * K*V; S0, post, out are [B*H, K, V].  S0, pre, post may be NULL (zero);
 * count may be 0 (out = S0 + post).  dims gives B, H, K, V; only K = V = 128 is supported. */
HDLA_API int hdla_compose_states(const HdlaDims* dims, const float* T, const float* F, const float* S0,
                                 const float* pre, const float* post, float* out, int32_t count,
                                 int64_t t_stride, int64_t f_stride, int32_t reverse, void* cuda_stream);

/* a/b parametrisation of the HDLA layer, forward and backward.  Replaces parameterize_a_b
 * (HRDPLR/hdla_custom.py:19-43; as shipped that function builds a and b but has no return statement):
 *   a1 = -beta k, a2 = -beta e^{log_f} k + a1 * sum_K(k * (-beta e^{log_f} k)), b1 = e^{log_f} k, b2 = k
 *   beta [B,T,H,1], k and log_f [B,T,H,K]  ->  a, b [B, 2T, H, K] (row 2t + r), all in `dtype`.
 * Backward takes da, db and writes dbeta [B,T,H,1], dk, dlog_f. */
HDLA_API int hdla_param_ab_fwd(const void* beta, const void* k, const void* log_f, void* a, void* b,
                               int32_t B, int32_t T, int32_t H, int32_t K, int32_t dtype, void* cuda_stream);
HDLA_API int hdla_param_ab_bwd(const void* beta, const void* k, const void* log_f, const void* da, const void* db,
                               void* dbeta, void* dk, void* dlog_f,
                               int32_t B, int32_t T, int32_t H, int32_t K, int32_t dtype, void* cuda_stream);

/* Output epilogue of the layer: o = sqrt(D) * y / sqrt(sum(y^2) + eps) * weight with y = x * sigmoid(gate), per row
 * of length D.  Replaces the layer's RMSNormFusedGate call (HRDPLR/hdla_custom.py:341-345,
 * HRDPLR/normalizations/rms_norm.py:48-91).  x, gate, o, dx, dgate: [rows, D] in `dtype`; weight [D] in `dtype`;
 * dweight [D] fp32, ACCUMULATED (the caller zeroes it).  D is a multiple of 8, at most 8192 (HDLA_ERR_UNSUPPORTED
 * otherwise) and every tensor starts on a 16-byte boundary (HDLA_ERR_INVALID otherwise). */
HDLA_API int hdla_norm_gate_fwd(const void* x, const void* gate, const void* weight, void* o,
                                int64_t rows, int32_t D, float eps, int32_t dtype, void* cuda_stream);
HDLA_API int hdla_norm_gate_bwd(const void* x, const void* gate, const void* weight, const void* d_o,
                                void* dx, void* dgate, float* dweight,
                                int64_t rows, int32_t D, float eps, int32_t dtype, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* HDLA_H_ */
