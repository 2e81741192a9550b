// exl3_mgemm: EXL3 products over a device-resident table of tensors, selected by device-resident indices - the MoE decode
// path of the reference (kernels/quant/exl3_gemm.cu:386-678, kernel kernels/quant/exl3_gemm_kernel.cuh:88-314, shim
// csrc/exl3_shim.cpp:57-75).  The routing never touches the host: one launch covers every slot, a slot whose index is
// negative is skipped, and with `weights` the slots of each token are scaled and summed into that token's row.
//
// Built on the streaming decode kernel in its table form: slot j is a run of column blocks whose codes come from
// trellis_tab[indices[j]] by plain bulk copies (the tensor is not known on the host, so there is no tensor map), whose
// activations were transformed with that tensor's input sign vector, and whose output goes to C[j].
#include "gemm_decode.cuh"

namespace {

using namespace exl3;

template <int K, int CB, int MT>
cudaError_t launch_multi(const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    constexpr int bytes = GdSmem<K, MT>::BYTES;
    static bool configured[64] = {};
    auto kern = gemm_decode_kernel<K, CB, MT, true>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GD_THREADS); cfg.dynamicSmemBytes = bytes; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    CUtensorMap none;
    memset(&none, 0, sizeof(none));
    return cudaLaunchKernelEx(&cfg, kern, none, none, none, p);
}

template <int K, int CB>
cudaError_t launch_multi_mt(int mt, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    return mt == 1 ? launch_multi<K, CB, 1>(p, grid, st) : launch_multi<K, CB, 2>(p, grid, st);
}

template <int K>
cudaError_t launch_multi_cb(int cb, int mt, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    if (cb == 0) return launch_multi_mt<K, 0>(mt, p, grid, st);
    if (cb == 1) return launch_multi_mt<K, 1>(mt, p, grid, st);
    return launch_multi_mt<K, 2>(mt, p, grid, st);
}

cudaError_t launch_multi_k(int K, int cb, int mt, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    switch (K) {
        case 1: return launch_multi_cb<1>(cb, mt, p, grid, st);
        case 2: return launch_multi_cb<2>(cb, mt, p, grid, st);
        case 3: return launch_multi_cb<3>(cb, mt, p, grid, st);
        case 4: return launch_multi_cb<4>(cb, mt, p, grid, st);
        case 5: return launch_multi_cb<5>(cb, mt, p, grid, st);
        case 6: return launch_multi_cb<6>(cb, mt, p, grid, st);
        case 7: return launch_multi_cb<7>(cb, mt, p, grid, st);
        default: return launch_multi_cb<8>(cb, mt, p, grid, st);
    }
}

// Weighted-sum reduction (kernels/quant/exl3_gemm_kernel.cuh:262-313): token t owns the `stride` consecutive slots from
// t * stride; its active slots (index >= 0) are added in slot order, in C's own precision, and the sum replaces slot t's
// rows.  Tokens go in increasing order, so row t is read (as part of group t / stride) before it is overwritten.
template <bool FP32>
__global__ void __launch_bounds__(256) mgemm_reduce_kernel(void* C, const int64_t* __restrict__ indices, long long elems_per_slot,
                                                           int stride, int num_tokens)
{
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= elems_per_slot) return;
    for (int t = 0; t < num_tokens; ++t) {
        if constexpr (FP32) {
            float* c = reinterpret_cast<float*>(C);
            float sum = 0.0f;
            for (int j = 0; j < stride; ++j)
                if (!indices || indices[t * stride + j] >= 0) sum += c[(size_t)(t * stride + j) * elems_per_slot + e];
            c[(size_t)t * elems_per_slot + e] = sum;
        } else {
            half* c = reinterpret_cast<half*>(C);
            half sum = __float2half(0.0f);
            for (int j = 0; j < stride; ++j)
                if (!indices || indices[t * stride + j] >= 0) sum = __hadd(sum, c[(size_t)(t * stride + j) * elems_per_slot + e]);
            c[(size_t)t * elems_per_slot + e] = sum;
        }
    }
}

}  // namespace

extern "C" int exl3_mgemm(exl3_ctx* ctx, exl3_stream stream, const void* A, const void* const* trellis, void* C,
                          const void* const* suh, void* A_had, const void* const* svh, const int64_t* indices,
                          const void* weights, int bszm_in, int bszm_out, int m, int k, int n, int K, int c_fp32, int mcg,
                          int mul1, int num_tokens)
{
    (void)A_had;
    EXL3_REQUIRE(ctx && A && trellis && C && suh && svh, "exl3_mgemm: null argument");
    EXL3_REQUIRE(bszm_in >= 1 && bszm_out >= 1 && m >= 0 && k > 0 && n > 0 && k % 128 == 0 && n % 128 == 0, "exl3_mgemm: bad shape");
    EXL3_REQUIRE(K >= 1 && K <= 8 && !(mcg && mul1), "exl3_mgemm: bad bits or codebook flags");
    EXL3_REQUIRE(aligned16(A) && aligned16(C), "exl3_mgemm: pointers must be 16-byte aligned");
    const int bszm = bszm_in > bszm_out ? bszm_in : bszm_out;
    EXL3_REQUIRE(bszm_in == 1 || bszm_in == bszm, "exl3_mgemm: A holds one slot or one per output slot");
    EXL3_REQUIRE(num_tokens >= 1 && bszm % num_tokens == 0, "exl3_mgemm: slots must divide evenly among the tokens");
    if (m == 0) return EXL3_OK;
    const int cb = mcg ? 1 : (mul1 ? 2 : 0);
    cudaStream_t st = (cudaStream_t)stream;
    const int blocks = bszm * (n / 128);
    EXL3_REQUIRE(blocks <= ctx->n_counters, "exl3_mgemm: too many column blocks for the context's counters");
    const int KC = (k + GD_UNIT_K - 1) / GD_UNIT_K;
    const long long total = (long long)blocks * KC;
    const int sms = ctx->num_sms;
    for (int r0 = 0; r0 < m; r0 += 16) {
        const int rows = m - r0 < 16 ? m - r0 : 16;
        const int mt = rows <= 8 ? 1 : 2;
        size_t off = 0;
        uint32_t* a_frag = (uint32_t*)exl3_ws_take(ctx, &off, (size_t)bszm * mt * k * 32);
        float* rowsum = (float*)exl3_ws_take(ctx, &off, (size_t)bszm * mt * 8 * 4);
        GemmDecodeParams p;
        memset(&p, 0, sizeof(p));
        const long long units_aligned = (long long)((blocks + sms - 1) / sms) * KC, units_even = (total + sms - 1) / sms;
        p.aligned = units_aligned <= units_even + 1 ? 1 : 0;
        const int grid = p.aligned ? (blocks < sms ? blocks : sms) : (int)(total < sms ? total : sms);
        p.partial = (float*)exl3_ws_take(ctx, &off, (size_t)grid * 2 * rows * 128 * 4);
        if (!a_frag || !rowsum || !p.partial) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "exl3_mgemm: context scratch too small");
        const half* a0 = (const half*)A + (size_t)r0 * k;
        gemm_decode_prologue_multi_kernel<<<dim3(8 * mt, bszm), 256, 0, st>>>(a0, bszm_in == 1 ? 0 : (size_t)m * k, (const half* const*)suh,
                                                                             indices, a_frag, rowsum, 8 * mt, rows, k);
        ctx->launches++;
        p.a_frag[0] = (const uint4*)a_frag; p.rowsum[0] = rowsum; p.rowsum_parts = 1;
        p.C[0] = c_fp32 ? (void*)((float*)C + (size_t)r0 * n) : (void*)((half*)C + (size_t)r0 * n);
        p.n[0] = p.n[1] = p.n[2] = n;
        p.blk_end[0] = p.blk_end[1] = p.blk_end[2] = blocks;
        p.counters = ctx->counters; p.status = ctx->status; p.m = rows; p.k = k; p.c_fp32 = c_fp32;
        p.trellis_tab = (const uint32_t* const*)trellis; p.svh_tab = (const half* const*)svh;
        p.indices = indices; p.weights = (const half*)weights; p.slots = bszm; p.c_slot_stride = (long long)m * n;
        cudaError_t e = launch_multi_k(K, cb, mt, p, grid, st);
        ctx->launches++;
        if (e != cudaSuccess) { cudaGetLastError(); return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e)); }
    }
    if (weights) {
        const long long elems = (long long)m * n;
        const int stride = bszm / num_tokens;
        if (c_fp32) mgemm_reduce_kernel<true><<<(unsigned)((elems + 255) / 256), 256, 0, st>>>(C, indices, elems, stride, num_tokens);
        else mgemm_reduce_kernel<false><<<(unsigned)((elems + 255) / 256), 256, 0, st>>>(C, indices, elems, stride, num_tokens);
        ctx->launches++;
    }
    return exl3_check_launch(ctx, "exl3_mgemm");
}
