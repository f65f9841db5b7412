// Kernel and launcher of the tcgen05 batched GEMM (see tc_gemm.cuh).
#include "tc_gemm.cuh"

namespace hdla {
namespace {

__global__ void __launch_bounds__(128) tc_bgemm_kernel(TcGemmP p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    uint4* sA = reinterpret_cast<uint4*>(smem_raw);
    uint4* sB = reinterpret_cast<uint4*>(smem_raw + tc::kSmemOperand);
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_base_s;

    const long long g = blockIdx.x;
    const long long bh = g / p.NT, n = g % p.NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Lp = (p.L + 15) & ~15, Np = (p.N + 15) & ~15;

    if (warp == 0) {
        sm100::tmem_alloc(&tmem_base_s, 128);
        sm100::tmem_relinquish();
    }
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        sm100::fence_mbar_init();
    }
    // operands: A as [M rows x L], B as [N rows x L] (B(l,j) -> row j)
    const void* Ab = p.A.dt == HDLA_F32
        ? static_cast<const void*>(static_cast<const float*>(p.A.p) + bh * p.A.sbh + n * p.A.sn)
        : static_cast<const void*>(static_cast<const __nv_bfloat16*>(p.A.p) + bh * p.A.sbh + n * p.A.sn);
    const void* Bb = p.B.dt == HDLA_F32
        ? static_cast<const void*>(static_cast<const float*>(p.B.p) + bh * p.B.sbh + n * p.B.sn)
        : static_cast<const void*>(static_cast<const __nv_bfloat16*>(p.B.p) + bh * p.B.sbh + n * p.B.sn);
    const int a_mn = tc::stage_operand(sA, Ab, p.A.rs, p.A.cs, p.M, p.L, Lp, p.A.dt);
    const int b_mn = tc::stage_operand(sB, Bb, p.B.cs, p.B.rs, p.N, p.L, Lp, p.B.dt);
    sm100::fence_proxy_async();
    sm100::tc_fence_before();
    __syncthreads();
    sm100::tc_fence_after();
    const uint32_t tmem = tmem_base_s;

    if (threadIdx.x == 0) {
        const uint32_t idesc = sm100::make_idesc_bf16(128, Np, a_mn, b_mn);
        const uint32_t a0 = sm100::smem_u32(sA), b0 = sm100::smem_u32(sB);
        for (int ks = 0; ks < Lp / 16; ++ks) {
            const uint64_t da = sm100::make_smem_desc(a0 + ks * 2 * tc::kLBO, tc::kLBO, tc::kSBO);
            const uint64_t db = sm100::make_smem_desc(b0 + ks * 2 * tc::kLBO, tc::kLBO, tc::kSBO);
            sm100::umma_bf16(tmem, da, db, idesc, ks > 0);
        }
        sm100::umma_commit(&bar);
    }
    if (!sm100::mbar_wait(&bar, 0)) {
        if (p.status) atomicExch(p.status, 1);
    }
    sm100::tc_fence_after();

    // epilogue: this thread owns output row r
    const int r = warp * 32 + lane;
    const long long cbase = bh * p.cbh + n * p.cn;
    const float rsc = (p.row_scale && r < p.M) ? p.row_scale[g * p.M + r] : 1.f;
    for (int c0 = 0; c0 < Np; c0 += 16) {
        uint32_t v[16];
        sm100::tmem_ld_x16(tmem + ((uint32_t)(warp * 32) << 16) + c0, v);
        sm100::tmem_wait_ld();
        if (r < p.M) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int c = c0 + j;
                if (c < p.N) {
                    bool keep = true;
                    if (p.mask == 1) keep = (r / p.ri) >= (c / p.rj);
                    else if (p.mask == 2) keep = (r / p.ri) > (c / p.rj);
                    const size_t off = (size_t)(cbase + r * p.rsC + c * p.csC);
                    float val = 0.f;
                    if (keep) {
                        val = p.alpha * __uint_as_float(v[j]) * rsc;
                        if (p.col_scale) val *= p.col_scale[g * p.N + c];
                        if (p.accumulate) val += ld_elem(p.C, off, p.cdt);
                    }
                    st_elem(p.C, off, p.cdt, val);
                }
            }
        }
    }
    sm100::tc_fence_before();
    __syncthreads();
    if (warp == 0) sm100::tmem_dealloc(tmem, 128);
}

}  // namespace

int tc_bgemm_launch(const TcGemmP& p, long long G, cudaStream_t st) {
    if (p.M > 128 || p.N > 128 || p.L > 128 || p.M < 1 || p.N < 1 || p.L < 1)
        return fail(HDLA_ERR_UNSUPPORTED, "tc gemm: M=%d N=%d L=%d outside 1..128", p.M, p.N, p.L);
    if (!((p.A.rs == 1 || p.A.cs == 1) && (p.B.rs == 1 || p.B.cs == 1)))
        return fail(HDLA_ERR_UNSUPPORTED, "tc gemm: operands need one unit stride");
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaFuncSetAttribute(tc_bgemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * tc::kSmemOperand);
        attr_dev = dev;
    }
    tc_bgemm_kernel<<<(unsigned)G, 128, 2 * tc::kSmemOperand, st>>>(p);
    HDLA_CHECK_LAUNCH("tc_bgemm_kernel");
    return HDLA_OK;
}

}  // namespace hdla
