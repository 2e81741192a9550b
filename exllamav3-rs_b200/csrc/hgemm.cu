// exl3_hgemm: dense fp16 GEMM C[m,n] = A[m,k] . B[k,n] with fp32 accumulation on tcgen05 (the reference calls cuBLAS
// here, kernels/hgemm.cu:19-78).  Both matrices are row-major, so A is a K-major operand and B an MN-major one; both
// come by tiled TMA with the 128-byte swizzle and are consumed from shared memory as they land.
//
// CTA tile 128 x 256, K step 64, two stages; the accumulator takes 256 TMEM columns, so two CTAs share an SM and one's
// epilogue overlaps the other's main loop.  Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31).  Every mbarrier wait is bounded.
#include "gemm_tc.cuh"

namespace exl3 {
namespace {

constexpr int HG_BM = 128, HG_BN = 256, HG_BK = 64, HG_STAGES = 2, HG_THREADS = 192;
constexpr int HG_A_STAGE = HG_BM * HG_BK * 2;                 // 16 KB: 128 rows of 128 bytes
constexpr int HG_B_ATOM = HG_BK * 128;                        // 8 KB: 64 k rows of 64 columns
constexpr int HG_B_STAGE = (HG_BN / 64) * HG_B_ATOM;          // 32 KB
constexpr int HG_OFF_B = HG_STAGES * HG_A_STAGE;
constexpr int HG_OFF_BAR = HG_OFF_B + HG_STAGES * HG_B_STAGE;
constexpr int HG_SMEM = HG_OFF_BAR + (2 * HG_STAGES + 1) * 8 + 16 + 1024;
// D fp32, A/B fp16, A K-major, B MN-major, N = 256, M = 128
constexpr uint32_t HG_IDESC = (1u << 4) | (1u << 16) | ((uint32_t)(HG_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

struct HgemmParams {
    void* C;
    int* status;
    int m, k, n, c_fp32;
};

__global__ void __launch_bounds__(HG_THREADS, 2) hgemm_kernel(const __grid_constant__ CUtensorMap amap,
                                                              const __grid_constant__ CUtensorMap bmap, const HgemmParams p)
{
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + HG_OFF_BAR);
    uint64_t* empty = full + HG_STAGES;
    uint64_t* acc_full = empty + HG_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    __shared__ int s_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * HG_BN, m0 = blockIdx.y * HG_BM;
    const int ksteps = p.k / HG_BK;

    if (tid == 0) {
        s_failed = 0;
        for (int i = 0; i < HG_STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            for (int ks = 0; ks < ksteps; ++ks) {
                const int s = ks % HG_STAGES;
                if (ks >= HG_STAGES && !mbar_wait_sleep(&empty[s], ((ks / HG_STAGES) - 1) & 1)) { failed = true; break; }
                mbar_expect_tx(&full[s], HG_A_STAGE + HG_B_STAGE);
                tma_load_2d(smem + s * HG_A_STAGE, &amap, ks * HG_BK, m0, &full[s]);
                #pragma unroll
                for (int a = 0; a < HG_BN / 64; ++a)        // columns past n read as zeros and are never stored
                    tma_load_2d(smem + HG_OFF_B + s * HG_B_STAGE + a * HG_B_ATOM, &bmap, n0 + a * 64, ks * HG_BK, &full[s]);
            }
        }
    } else if (warp == 1) {
        const bool leader = elect_one();
        constexpr uint32_t HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);       // SBO 1024, version 1, SWIZZLE_128B
        const uint32_t a_lo = (smem_u32(smem) >> 4) | (1u << 16);
        const uint32_t b_lo = (smem_u32(smem + HG_OFF_B) >> 4) | ((uint32_t)(HG_B_ATOM >> 4) << 16);   // LBO: next 64-column atom
        for (int ks = 0; ks < ksteps; ++ks) {
            const int s = ks % HG_STAGES;
            if (!mbar_wait_sleep_warp(&full[s], (ks / HG_STAGES) & 1)) { failed = true; break; }
            tc_fence_after();
            if (leader) {
                #pragma unroll
                for (int kk = 0; kk < HG_BK / 16; ++kk) {
                    const uint64_t ad = ((uint64_t)HI << 32) | (a_lo + s * (HG_A_STAGE >> 4) + kk * 2);          // +32 bytes
                    const uint64_t bd = ((uint64_t)HI << 32) | (b_lo + s * (HG_B_STAGE >> 4) + kk * (2048 >> 4)); // +16 k rows
                    tc_mma_f16(tmem_base, ad, bd, HG_IDESC, (ks > 0 || kk > 0) ? 1u : 0u);
                }
                tc_commit(&empty[s]);
            }
            __syncwarp();
        }
        if (!failed && leader) tc_commit(acc_full);
    } else {
        if (!mbar_wait_sleep_warp(acc_full, 0)) failed = true;
        if (!failed) {
            tc_fence_after();
            const int q = warp & 3;
            const int row = m0 + q * 32 + lane;
            const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16);
            #pragma unroll 1
            for (int c = 0; c < HG_BN / 32; ++c) {
                float v[32];
                tc_ld32(tacc + c * 32, v);
                tc_wait_ld();
                const int col = n0 + c * 32;
                if (row < p.m && col < p.n) {
                    const size_t off = (size_t)row * p.n + col;
                    #pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        if (col + e < p.n) {                  // n is a multiple of 8: a group of 8 is all in or all out
                            if (p.c_fp32) {
                                float4* dst = reinterpret_cast<float4*>((float*)p.C + off + e);
                                dst[0] = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                                dst[1] = make_float4(v[e + 4], v[e + 5], v[e + 6], v[e + 7]);
                            } else {
                                uint32_t w[4];
                                #pragma unroll
                                for (int h = 0; h < 4; ++h) {
                                    half2 x = __floats2half2_rn(v[e + 2 * h], v[e + 2 * h + 1]);
                                    w[h] = *reinterpret_cast<uint32_t*>(&x);
                                }
                                *reinterpret_cast<uint4*>((half*)p.C + off + e) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            }
        }
    }

    if (failed) s_failed = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 4);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn hgemm_encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
        else
            cudaGetLastError();
    }
    return fn;
}

}  // namespace
}  // namespace exl3

using namespace exl3;

extern "C" int exl3_hgemm(exl3_ctx* ctx, exl3_stream stream, const void* a, const void* b, void* c, int m, int k, int n, int c_fp32)
{
    EXL3_REQUIRE(ctx && a && b && c, "exl3_hgemm: null argument");
    EXL3_REQUIRE(m >= 0 && k > 0 && n > 0 && k % 64 == 0 && n % 8 == 0, "exl3_hgemm: k must be a multiple of 64 and n of 8");
    EXL3_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c), "exl3_hgemm: pointers must be 16-byte aligned");
    if (m == 0) return EXL3_OK;
    EncodeTiledFn enc = hgemm_encode_tiled();
    if (!enc) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_hgemm: cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap amap, bmap;
    {
        cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
        cuuint64_t strides[1] = {(cuuint64_t)k * 2};
        cuuint32_t box[2] = {(cuuint32_t)HG_BK, (cuuint32_t)HG_BM};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_hgemm: cuTensorMapEncodeTiled failed for A");
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)k};
        cuuint64_t strides[1] = {(cuuint64_t)n * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)HG_BK};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&bmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(b), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_hgemm: cuTensorMapEncodeTiled failed for B");
    }
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(hgemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, HG_SMEM);
        if (e != cudaSuccess) return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    HgemmParams p;
    p.C = c; p.status = ctx->status; p.m = m; p.k = k; p.n = n; p.c_fp32 = c_fp32;
    dim3 grid((n + HG_BN - 1) / HG_BN, (m + HG_BM - 1) / HG_BM);
    hgemm_kernel<<<grid, HG_THREADS, HG_SMEM, (cudaStream_t)stream>>>(amap, bmap, p);
    ctx->launches++;
    return exl3_check_launch(ctx, "exl3_hgemm");
}
