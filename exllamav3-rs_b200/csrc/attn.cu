// exl3_bighead_attn_paged / exl3_bighead_attn_paged_q: planning, launch and split-KV combine.
#include <algorithm>
#include "attn_paged.cuh"
#include "attn_tc.cuh"
#include "attn_tc2.cuh"
#include "attn_q4.cuh"

namespace {

using namespace exl3;

// Builds the split-KV work list from the REAL sequence lengths (one CTA; bsz is small next to the KV walk).
// Each sequence gets ceil(total_k / chunk) splits per row block, with chunk sized so that the list has about
// `target_items` entries; the reference sizes its splits from the padded block-table width instead
// (kernels/attention.cu:1805), which launches empty CTAs for the short sequences of a ragged batch.
// Only sequences whose packed row count ql*G lies in (rows_lo, rows_hi] get work items; the others are left to another pass.
__global__ void __launch_bounds__(1024) attn_plan_kernel(const int32_t* __restrict__ seqlens,
                                                         const int32_t* __restrict__ cu_q, int bsz, int q_len,
                                                         int kv_append, int G, int rows_per_cta, int rows_lo, int rows_hi, int chunk_mult, int target_items,
                                                         int max_items, AttnPlan* plan, AttnItem* items, int* seq_base,
                                                         int* seq_splits, int* order, int causal, int slots, int* status)
{
    __shared__ long long s_total;
    __shared__ int s_scan[1024];
    __shared__ int s_cursor[1024];
    __shared__ int s_carry, s_chunk;
    const int tid = threadIdx.x;
    if (tid == 0) { s_total = 0; s_carry = 0; }
    __syncthreads();
    long long local = 0;
    for (int b = tid; b < bsz; b += 1024) {
        const int ql = cu_q ? cu_q[b + 1] - cu_q[b] : q_len;
        const int tk = (seqlens ? seqlens[b] : 0) + (cu_q ? ql : kv_append);
        const int pr = ql * G;
        const int rb = (pr > rows_lo && pr <= rows_hi) ? (pr + rows_per_cta - 1) / rows_per_cta : 0;
        local += (long long)tk * rb;
    }
    atomicAdd((unsigned long long*)&s_total, (unsigned long long)local);
    __syncthreads();
    // Keys per split: total work / target_items.  slots > 0 (kernels whose CTAs are whole items, target_items = two per CTA
    // slot): one item per slot instead when that already gives two or more items per slot, because every row block and
    // every sequence rounds its split count up.  Then the longest-first order balances the slots and fewer items save the
    // fixed cost of a CTA and the partials (four 256-row chunks: 125 us at one item per slot, 135 at two, 150 at three; 32
    // x 8 verify rows: 125 against 133 us), while a batch of few long items (one 256-row chunk over 32768 keys: 20 items
    // on 18 slots) keeps the finer split.
    auto chunk_for = [&](long long t) {
        long long c = (s_total + t - 1) / t;
        c = (c + chunk_mult - 1) / chunk_mult * chunk_mult;       // splits start on a key-tile boundary of the kernel
        if (c < 256) c = 256;
        if (c > (1 << 30)) c = 1 << 30;
        return (int)c;
    };
    if (slots <= 0) {
        if (tid == 0) s_chunk = chunk_for(target_items);
        __syncthreads();
    } else {
        __shared__ long long s_count;
        const int c1 = chunk_for(slots);
        if (tid == 0) s_count = 0;
        __syncthreads();
        long long cnt = 0;
        for (int b = tid; b < bsz; b += 1024) {
            const int ql = cu_q ? cu_q[b + 1] - cu_q[b] : q_len;
            const int tk = (seqlens ? seqlens[b] : 0) + (cu_q ? ql : kv_append);
            const int pr = ql * G;
            const int rb = (pr > rows_lo && pr <= rows_hi) ? (pr + rows_per_cta - 1) / rows_per_cta : 0;
            cnt += (long long)rb * (tk > 0 ? (tk + c1 - 1) / c1 : 1);
        }
        atomicAdd((unsigned long long*)&s_count, (unsigned long long)cnt);
        __syncthreads();
        if (tid == 0) s_chunk = s_count >= 2LL * slots ? c1 : chunk_for(target_items);
        __syncthreads();
    }
    const int chunk = s_chunk;
    for (int b0 = 0; b0 < bsz; b0 += 1024) {
        const int b = b0 + tid;
        int ql = 0, tk = 0, rb = 0, sp = 0;
        if (b < bsz) {
            ql = cu_q ? cu_q[b + 1] - cu_q[b] : q_len;
            tk = (seqlens ? seqlens[b] : 0) + (cu_q ? ql : kv_append);
            const int pr = ql * G;
            rb = (pr > rows_lo && pr <= rows_hi) ? (pr + rows_per_cta - 1) / rows_per_cta : 0;
            sp = (rb > 0 && tk > 0) ? (tk + chunk - 1) / chunk : 1;
        }
        const int cnt = rb * sp;
        s_scan[tid] = cnt;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {                   // inclusive Hillis-Steele scan
            int v = tid >= o ? s_scan[tid - o] : 0;
            __syncthreads();
            s_scan[tid] += v;
            __syncthreads();
        }
        const int base = s_carry + s_scan[tid] - cnt;
        if (b < bsz) {
            seq_base[b] = base;
            seq_splits[b] = sp;
            for (int j = 0; j < cnt && base + j < max_items; ++j) {
                AttnItem it; it.b = b; it.rb = j / sp; it.split = j % sp; it.pad = 0;
                items[base + j] = it;
            }
        }
        __syncthreads();
        if (tid == 1023) s_carry += s_scan[1023];
        __syncthreads();
    }
    // Launch order: longest items first (counting sort by key tiles, most first).  Items differ in length - last splits,
    // causal cuts, short sequences - and a long one started late leaves the other SMs idle at the end of the kernel
    // (four 256-row chunks: a quarter of the SM time).
    const int n_items = s_carry < max_items ? s_carry : max_items;
    s_scan[tid] = 0; s_cursor[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n_items; i += 1024) {
        const AttnItem it = items[i];
        const int ql = cu_q ? cu_q[it.b + 1] - cu_q[it.b] : q_len;
        const int tk = (seqlens ? seqlens[it.b] : 0) + (cu_q ? ql : kv_append);
        const int i_last = min(ql - 1, (it.rb * rows_per_cta + rows_per_cta - 1) / G);
        const int vis = causal > 0 ? min(tk, tk - ql + i_last + 1) : tk;
        const int k_begin = it.split * chunk;
        const int k_end = min(min(k_begin + chunk, tk), vis);
        int key = k_end > k_begin ? (k_end - k_begin + chunk_mult - 1) / chunk_mult : 0;
        key = causal >= 0 ? 1023 - min(key, 1023) : 0;          // bin 0 = longest (causal < 0: A/B switch, plan order kept)
        items[i].pad = key;
        atomicAdd(&s_scan[key], 1);
    }
    __syncthreads();
    {
        const int cnt = s_scan[tid];
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {                   // inclusive scan over the bins
            int v = tid >= o ? s_scan[tid - o] : 0;
            __syncthreads();
            s_scan[tid] += v;
            __syncthreads();
        }
        const int excl = s_scan[tid] - cnt;
        __syncthreads();
        s_scan[tid] = excl;                                    // first position of bin tid
        __syncthreads();
    }
    for (int i = tid; i < n_items; i += 1024) {
        const int key = items[i].pad;
        order[causal < 0 ? i : s_scan[key] + atomicAdd(&s_cursor[key], 1)] = i;
    }
    if (tid == 0) {
        plan->n_items = n_items;
        plan->chunk = chunk;
        // the host sizes the list from bounds on the batch; a list that does not fit would silently drop work, so it is
        // reported through the status word like a device-side wait that ran out
        if (s_carry > max_items) atomicExch(status, 3);
    }
}

// Merges the split-KV partials of one output row (b, query, head); one warp per row, lane = D/32 dims.
template <int D>
__global__ void __launch_bounds__(256) attn_combine_kernel(const AttnParams p, int rows_per_cta, int total_rows)
{
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (w >= (long long)total_rows * p.nq) return;
    const int row = (int)(w / p.nq), head = (int)(w % p.nq);
    int b;
    if (p.cu_q) {                                              // binary search: cu_q[b] <= row < cu_q[b+1]
        int lo = 0, hi = p.bsz - 1;
        while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (p.cu_q[mid] <= row) lo = mid; else hi = mid - 1; }
        b = lo;
    } else b = row / p.q_len;
    const int splits = p.seq_splits[b];
    if (splits <= 1) return;                                   // the attention kernel wrote the final value itself
    const int row_base = p.cu_q ? p.cu_q[b] : b * p.q_len;
    const int G = p.nq / p.nkv, kvh = head / G;
    const int packed = (row - row_base) * G + (head - kvh * G);
    const int rb = packed / rows_per_cta, lr = packed - rb * rows_per_cta;
    const int item0 = p.seq_base[b] + rb * splits;
    // A sequence of a small batch can have dozens of splits; walked one after the other by every lane their loads form
    // one long dependent chain (53 us per launch on 4 verify sequences).  So the lanes take the splits' maxima and sums
    // side by side, and the rows themselves are fetched four splits at a time.
    static_assert(D == 128, "a lane covers 4 dims as two 8-byte loads");
    const size_t stride = (size_t)p.nkv * rows_per_cta * (D + 2);             // floats between consecutive splits
    const float* base = p.partial + (((size_t)item0 * p.nkv + kvh) * rows_per_cta + lr) * (D + 2);
    float mm = -INFINITY;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        const int s = s0 + lane;
        if (s < splits) mm = fmaxf(mm, base[(size_t)s * stride + D]);
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    float acc[D / 32], ll = 0.f;
    #pragma unroll
    for (int e = 0; e < D / 32; ++e) acc[e] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        const int s = s0 + lane;
        float sc_l = 0.f;
        if (s < splits) {
            const float ms = base[(size_t)s * stride + D];
            sc_l = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
            ll += base[(size_t)s * stride + D + 1] * sc_l;
        }
        const int cnt = min(32, splits - s0);
        #pragma unroll 4
        for (int j = 0; j < cnt; ++j) {
            const float sc = __shfl_sync(0xffffffffu, sc_l, j);
            const float* pp = base + (size_t)(s0 + j) * stride + lane * (D / 32);
            const float2 v0 = *reinterpret_cast<const float2*>(pp), v1 = *reinterpret_cast<const float2*>(pp + 2);
            acc[0] += v0.x * sc; acc[1] += v0.y * sc; acc[2] += v1.x * sc; acc[3] += v1.y * sc;
        }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
    const float inv = ll > 0.f ? 1.0f / ll : 0.f;
    half* op = p.o + ((size_t)row * p.nq + head) * D + lane * (D / 32);
    #pragma unroll
    for (int e = 0; e < D / 32; e += 2) *reinterpret_cast<uint32_t*>(op + e) = pack_h2(acc[e] * inv, acc[e + 1] * inv);
}

template <int D, int WM, int WN, int QB>
cudaError_t launch_attn(const AttnParams& p, dim3 grid, cudaStream_t st)
{
    constexpr int bytes = AttnSmem<D, QB>::BYTES;
    auto kern = attn_paged_kernel<D, WM, WN, QB>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kern<<<grid, AT_THREADS, bytes, st>>>(p);
    return cudaPeekAtLastError();
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn attn_encode_tiled()
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

// tcgen05 attention: one CTA per work item and kv head; K/V tiles come through 4-D tensor maps of the pools
cudaError_t launch_attn_tc(exl3_ctx* ctx, const AttnParams& p, int max_items, cudaStream_t st)
{
    EncodeTiledFn enc = attn_encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap maps[2];
    const void* pools[2] = {p.kc, p.vc};
    for (int i = 0; i < 2; ++i) {
        cuuint64_t dims[4] = {(cuuint64_t)ATC_D, (cuuint64_t)p.nkv, 256, (cuuint64_t)p.pages};
        cuuint64_t strides[3] = {(cuuint64_t)ATC_D * 2, (cuuint64_t)p.nkv * ATC_D * 2, (cuuint64_t)256 * p.nkv * ATC_D * 2};
        cuuint32_t box[4] = {64, 1, (cuuint32_t)ATC_TN, 1};           // 128 tokens of one page, one 64-wide d block
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(pools[i]), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    (void)ctx;
    attn_tc_kernel<<<dim3((unsigned)max_items * p.nkv), ATC_THREADS, ATC_SMEM, st>>>(maps[0], maps[1], p);
    return cudaPeekAtLastError();
}

cudaError_t launch_attn_tc2(exl3_ctx* ctx, const AttnParams& p, int max_items, cudaStream_t st)
{
    EncodeTiledFn enc = attn_encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap maps[2];
    const void* pools[2] = {p.kc, p.vc};
    for (int i = 0; i < 2; ++i) {
        cuuint64_t dims[4] = {(cuuint64_t)ATC_D, (cuuint64_t)p.nkv, 256, (cuuint64_t)p.pages};
        cuuint64_t strides[3] = {(cuuint64_t)ATC_D * 2, (cuuint64_t)p.nkv * ATC_D * 2, (cuuint64_t)256 * p.nkv * ATC_D * 2};
        cuuint32_t box[4] = {64, 1, (cuuint32_t)ATC_TN, 1};           // 128 tokens of one page, one 64-wide d block
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(pools[i]), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    static bool configured[64] = {};
    static const int tune_h = getenv("EXL3_TUNE_TC_H") ? atoi(getenv("EXL3_TUNE_TC_H")) : 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc2_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_tc2_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    (void)ctx;
    if (tune_h == 4) attn_tc2_kernel<4><<<dim3((unsigned)max_items * p.nkv), a2_threads(4), A2_SMEM, st>>>(maps[0], maps[1], p);
    else attn_tc2_kernel<2><<<dim3((unsigned)max_items * p.nkv), a2_threads(2), A2_SMEM, st>>>(maps[0], maps[1], p);
    return cudaPeekAtLastError();
}

// decode-class kernel over 4-bit pools: tensor maps over the code planes ([tokens][nkv * 16] words) and the scale planes
// ([tokens][nkv * 4] halves, copied in 16-byte pairs of heads)
cudaError_t launch_attn_q4(const AttnParams& p, dim3 grid, cudaStream_t st)
{
    EncodeTiledFn enc = attn_encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap maps[4];
    const void* planes[4] = {p.qk, p.qv, p.sk, p.sv};
    const cuuint64_t tokens = (cuuint64_t)p.pages * EXL3_PAGE;
    for (int i = 0; i < 4; ++i) {
        const bool codes = i < 2;
        cuuint64_t dims[2] = {(cuuint64_t)p.nkv * (codes ? 16 : 4), tokens};
        cuuint64_t strides[1] = {(cuuint64_t)p.nkv * (codes ? 64 : 8)};
        cuuint32_t box[2] = {codes ? 16u : 8u, (cuuint32_t)AQ_TK};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&maps[i], codes ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(planes[i]),
                dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_q4_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AQ_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    attn_q4_decode_kernel<<<grid, AQ_THREADS, AQ_SMEM, st>>>(maps[0], maps[1], maps[2], maps[3], p);
    return cudaPeekAtLastError();
}

bool q4_decode_kernel_applies(const AttnParams& p, bool quant);

// One pass = plan + attention + combine over the sequences whose packed row count lies in (rows_lo, rows_hi].
int attn_pass(exl3_ctx* ctx, cudaStream_t st, AttnParams p, int total_rows, int max_rows, int rows_lo, int rows_hi,
              bool decode_shape, bool quant, size_t* ws_off)
{
    const int D = 128;
    const int G = p.nq / p.nkv;
    const bool q4 = quant && p.k_bits == 4 && p.v_bits == 4;       // the common cache format has its own, smaller staging
    // long class on fp16 pools: tcgen05 kernel (256-row items) unless the context was switched to the mma.sync kernels
    // (its row maximum is taken on the raw scores, which needs a positive scale)
    // (sequences with 17..128 packed rows - speculative verify - stay on it too: on 32 sequences x 8 query rows x 5 heads
    // the 64-row mma.sync kernel measured 228 us against 224 us, at 16 and 24 query rows 373 / 383 us against 233 / 241 us)
    const bool use_tc = !decode_shape && !quant && ctx->mma_attn != 0 && p.scale_log2 > 0.f && !p.contig_kv;
    // two arrangements of the tcgen05 kernel: 128-row items with two softmax threads per row (default), 256-row items
    static const bool tc_256 = getenv("EXL3_B200_ATTN_TC256") != nullptr;
    const int rows_per_cta = decode_shape ? 16 : (use_tc ? (tc_256 ? ATC_CTA_ROWS : A2_ROWS) : 64);
    const int rb_max = (max_rows + rows_per_cta - 1) / rows_per_cta;
    // resident CTAs per SM over all kv heads: about 3 for the mma.sync kernels, 1 for the tcgen05 kernel (all of TMEM)
    // (rounded down: one CTA more than fits would run alone in a second wave after all the others have finished)
    // 4-bit pools, decode class: the kernel that builds the K operand from the codes (its scale copies are 16 bytes wide =
    // two heads, so the kv head count must be even and the planes 16-byte aligned)
    const bool use_q4 = decode_shape && q4_decode_kernel_applies(p, quant);
    int per_sm = 1;
    if (use_q4) per_sm = 3;
    else if (!use_tc) {
        // CTAs of the mma.sync kernel that fit on an SM (bounded by shared memory: stages x 34.8 KB for fp16 pools)
        const size_t smem = quant ? (q4 ? AttnSmem<128, 4>::BYTES : AttnSmem<128, 8>::BYTES) : AttnSmem<128, 0>::BYTES;
        per_sm = std::max(1, std::min(q4 ? 4 : 3, (int)((227 * 1024) / (smem + 1024))));
    }
    const int grid_x = std::max(1, ctx->num_sms * per_sm / p.nkv);
    // tcgen05 kernels: two items per CTA slot: more items shorten the tail of the last wave but every extra KV split costs
    // a partial per kv head written and read back (128-row kernel on 4 x 256 query rows: 154 / 168 / 171 / 188 / 205 us at
    // 2 / 3 / 4 / 6 / 8 per slot).
    // mma.sync kernels (units handed out dynamically, 8 KB partials): see below.
    static const int tc_items = getenv("EXL3_TUNE_TC_ITEMS") ? atoi(getenv("EXL3_TUNE_TC_ITEMS")) : 0;
    // With the units handed out longest first, fewer and longer items win on the mma.sync kernels too (64 decode
    // sequences at 1 / 2 / 3 / 4 items per slot: fp16 pools 242 / 234 / 237 / 242 us, 4-bit pools 195 / 202 / 209 / 212 us;
    // the 4-sequence verify step 21.5 / 22.0 / 22.6 / 23.2 ms; 8-bit pools on the generic kernel 532 / 548 / 550 us at 2 / 3 /
    // 4): two, and one for the 4-bit kernel.
    static const int dec_items = getenv("EXL3_TUNE_DEC_ITEMS") ? atoi(getenv("EXL3_TUNE_DEC_ITEMS")) : 0;
    const int target_items = grid_x * (use_tc ? (tc_items ? tc_items : 2) : (dec_items ? dec_items : (use_q4 ? 1 : 2)));
    // items <= target + sum of row blocks (every (sequence, row block) rounds its split count up once); the row blocks are
    // bounded by bsz * rb_max and, usually much tighter for ragged batches, by total_rows * G / rows_per_cta + bsz
    const long long rb_sum = std::min((long long)p.bsz * rb_max, ((long long)total_rows * G + rows_per_cta - 1) / rows_per_cta + p.bsz);
    const int max_items = target_items + (int)std::min(rb_sum, (long long)(1 << 24)) + 1;

    // The work list depends on the batch's lengths, not on the layer: inside exl3_step_forward it is built by the first
    // layer's call into the context's slot for this class and reused by the other layers.
    const int cls = decode_shape ? 0 : 1;
    const size_t list_bytes = 256 + (((size_t)max_items * sizeof(AttnItem) + 255) & ~(size_t)255) + 2 * (((size_t)p.bsz * 4 + 255) & ~(size_t)255) +
                              (((size_t)max_items * 4 + 255) & ~(size_t)255);
    const bool keep = ctx->plan_keep && list_bytes <= ctx->plan_slot_bytes;
    size_t off = *ws_off;                                // scratch of an earlier pass that may still be running
    AttnPlan* plan; AttnItem* items; int* seq_base; int* seq_splits; int* order;
    if (keep) {
        uint8_t* slot = ctx->plan_slots + cls * ctx->plan_slot_bytes;
        plan = (AttnPlan*)slot;
        items = (AttnItem*)(slot + 256);
        seq_base = (int*)(slot + 256 + (((size_t)max_items * sizeof(AttnItem) + 255) & ~(size_t)255));
        seq_splits = (int*)((uint8_t*)seq_base + (((size_t)p.bsz * 4 + 255) & ~(size_t)255));
        order = (int*)((uint8_t*)seq_splits + (((size_t)p.bsz * 4 + 255) & ~(size_t)255));
    } else {
        plan = (AttnPlan*)exl3_ws_take(ctx, &off, sizeof(AttnPlan));
        items = (AttnItem*)exl3_ws_take(ctx, &off, (size_t)max_items * sizeof(AttnItem));
        seq_base = (int*)exl3_ws_take(ctx, &off, (size_t)p.bsz * 4);
        seq_splits = (int*)exl3_ws_take(ctx, &off, (size_t)p.bsz * 4);
        order = (int*)exl3_ws_take(ctx, &off, (size_t)max_items * 4);
    }
    float* partial = (float*)exl3_ws_take(ctx, &off, (size_t)max_items * p.nkv * rows_per_cta * (D + 2) * 4);
    if (!plan || !items || !seq_base || !seq_splits || !order || !partial)
        return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "attention: context scratch too small for the split-KV partials");
    p.plan = plan; p.items = items; p.seq_base = seq_base; p.seq_splits = seq_splits; p.order = order; p.partial = partial;
    p.status = ctx->status;
    *ws_off = off;

    static const bool no_lpt = getenv("EXL3_TUNE_NO_LPT") != nullptr;
    if (!(keep && ctx->plan_valid[cls])) {
        attn_plan_kernel<<<1, 1024, 0, st>>>(p.seqlens, p.cu_q, p.bsz, p.q_len, p.kv_append, G, rows_per_cta, rows_lo, rows_hi,
                                              use_tc ? ATC_TN : AT_TK, target_items, max_items, plan, items, seq_base, seq_splits, order, no_lpt ? -1 : (p.causal ? 1 : 0),
                                              (use_tc && !tc_items) ? grid_x : 0, ctx->status);
        ctx->launches++;
        if (keep) ctx->plan_valid[cls] = 1;
    }
    dim3 grid(grid_x, p.nkv);
    cudaError_t e;
    if (!use_tc && cudaMemsetAsync(&plan->next, 0, sizeof(int), st) != cudaSuccess)      // the persistent kernel's work counter
        return exl3_fail(ctx, EXL3_ERR_CUDA, "attention: cudaMemsetAsync failed");
    if (use_tc) e = tc_256 ? launch_attn_tc(ctx, p, max_items, st) : launch_attn_tc2(ctx, p, max_items, st);
    else if (use_q4) e = launch_attn_q4(p, grid, st);
    else if (q4)    e = decode_shape ? launch_attn<128, 1, 4, 4>(p, grid, st) : launch_attn<128, 4, 1, 4>(p, grid, st);
    else if (quant) e = decode_shape ? launch_attn<128, 1, 4, 8>(p, grid, st) : launch_attn<128, 4, 1, 8>(p, grid, st);
    else            e = decode_shape ? launch_attn<128, 1, 4, 0>(p, grid, st) : launch_attn<128, 4, 1, 0>(p, grid, st);
    ctx->launches++;
    if (e != cudaSuccess) { cudaGetLastError(); return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e)); }
    const long long warps = (long long)total_rows * p.nq;
    attn_combine_kernel<128><<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(p, rows_per_cta, total_rows);
    ctx->launches++;
    return exl3_check_launch(ctx, "attention");
}

// Sequences with at most 16 packed (query, head) rows (decode, short verify) take the kernel that spreads the keys of a
// tile over the four warps; longer ones (verify with many heads, prefill chunks) the one with a 16-row tile per warp.
// A ragged batch that holds both kinds runs one pass for each.
// true when attn_pass will take the 4-bit decode-class kernel for these pools
bool q4_decode_kernel_applies(const AttnParams& p, bool quant)
{
    static const bool no_q4 = getenv("EXL3_B200_NO_Q4_ATTN") != nullptr;
    return quant && p.k_bits == 4 && p.v_bits == 4 && !no_q4 && p.nkv % 2 == 0 && aligned16(p.qk) && aligned16(p.qv) &&
           aligned16(p.sk) && aligned16(p.sv);
}

int attn_impl(exl3_ctx* ctx, cudaStream_t st, AttnParams p, int total_rows, int max_q_len, bool quant)
{
    const int G = p.nq / p.nkv;
    const int max_rows = max_q_len * G;
    size_t off = 0;
    // Decode class = sequences with at most 16 packed rows.  Over 4-bit pools it also takes up to 48 rows (speculative
    // verify: 8 query rows x 5 heads) as row blocks of 16 that each walk the codes again: the kernel that builds its
    // operands from the codes is that much cheaper per key than the generic one (4 verify sequences: 90 us per layer there).
    // (Sending the decode rows of a ragged fp16 batch through the tcgen05 kernel as well, as items of 128 rows with 5 in
    // use, was measured on the benchmark step: the attention stage takes the same 28.0 ms of the step's 83.)
    const int dec_rows = q4_decode_kernel_applies(p, quant) ? 48 : 16;
    if (max_rows <= dec_rows) return attn_pass(ctx, st, p, total_rows, max_rows, 0, dec_rows, true, quant, &off);
    if (!p.cu_q) return attn_pass(ctx, st, p, total_rows, max_rows, 0, 1 << 30, false, quant, &off);
    // Ragged batch with both classes: the decode-class pass (bound by HBM) is issued on the context's second stream and
    // the long-class pass (bound by the tensor core and the MUFU) on the caller's; they touch disjoint sequences and
    // output rows, and each has its own scratch.  Fork and join by events, which also works while the caller's stream
    // is being captured.  What the second stream buys is the tail of one pass filling with the other's first CTAs: a
    // tcgen05 CTA takes a whole SM, so the bulk of the two passes runs one after the other (per layer of the benchmark
    // step the attention stage takes the sum of the two kernels' times).
    if (cudaEventRecord(ctx->ev_fork, st) != cudaSuccess || cudaStreamWaitEvent(ctx->aux_stream, ctx->ev_fork, 0) != cudaSuccess)
        return exl3_fail(ctx, EXL3_ERR_CUDA, "attention: stream fork failed");
    int rc = attn_pass(ctx, ctx->aux_stream, p, total_rows, dec_rows, 0, dec_rows, true, quant, &off);
    int rc2 = rc == EXL3_OK ? attn_pass(ctx, st, p, total_rows, max_rows, dec_rows, 1 << 30, false, quant, &off) : rc;
    // always join, also after an error, so that a capture in progress stays well-formed
    if (cudaEventRecord(ctx->ev_join, ctx->aux_stream) != cudaSuccess || cudaStreamWaitEvent(st, ctx->ev_join, 0) != cudaSuccess)
        return exl3_fail(ctx, EXL3_ERR_CUDA, "attention: stream join failed");
    return rc != EXL3_OK ? rc : rc2;
}

int check_common(exl3_ctx* ctx, const void* q, const void* o, const int32_t* bt, const int32_t* sl, int bsz, int q_len,
                 int kv_append, int nq, int nkv, int hd, int pages, int pps)
{
    EXL3_REQUIRE(ctx && q && o && bt && sl, "attention: null argument");
    EXL3_REQUIRE(bsz >= 0 && q_len >= 0 && kv_append >= 0 && nq > 0 && nkv > 0 && pages > 0 && pps > 0, "attention: bad shape");
    EXL3_REQUIRE(nq % nkv == 0, "attention: n_q_heads must be a multiple of n_kv_heads");
    EXL3_REQUIRE(nq / nkv <= 16, "attention: GQA ratio above 16");
    if (hd != 128) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "attention: head_dim must be 128");
    EXL3_REQUIRE(nkv <= 65535, "attention: too many kv heads");
    EXL3_REQUIRE(aligned16(q) && aligned16(o), "attention: pointers must be 16-byte aligned");
    return EXL3_OK;
}

}  // namespace

extern "C" int exl3_bighead_attn_paged(exl3_ctx* ctx, exl3_stream stream, const void* q, const void* k, const void* v,
                                       void* k_cache, void* v_cache, const int32_t* block_table,
                                       const int32_t* cache_seqlens, const int32_t* cu_q, void* o, int bsz, int q_len,
                                       int kv_append, int nq, int nkv, int hd, int pages, int pages_per_seq,
                                       int kv_chunk_size, int causal, float sm_scale)
{
    (void)kv_chunk_size;
    int rc = check_common(ctx, q, o, block_table, cache_seqlens, bsz, q_len, kv_append, nq, nkv, hd, pages, pages_per_seq);
    if (rc) return rc;
    EXL3_REQUIRE(k_cache && v_cache && aligned16(k_cache) && aligned16(v_cache), "attention: bad cache pointers");
    if (bsz == 0 || q_len == 0) return EXL3_OK;
    const int append = cu_q ? q_len : kv_append;
    if (append > 0) {
        EXL3_REQUIRE(k && v, "attention: kv_append > 0 needs k and v");
        rc = exl3_paged_kv_cache_update(ctx, stream, k, v, k_cache, v_cache, block_table, cache_seqlens, cu_q, bsz, append,
                                        nkv, hd, pages, pages_per_seq);
        if (rc) return rc;
    }
    AttnParams p;
    memset(&p, 0, sizeof(p));
    p.q = (const half*)q; p.o = (half*)o; p.kc = (const half*)k_cache; p.vc = (const half*)v_cache;
    p.block_table = block_table; p.seqlens = cache_seqlens; p.cu_q = cu_q;
    p.bsz = bsz; p.q_len = q_len; p.kv_append = kv_append; p.nq = nq; p.nkv = nkv; p.pps = pages_per_seq; p.pages = pages;
    p.causal = causal;
    p.scale_log2 = (sm_scale == 0.0f ? rsqrtf((float)hd) : sm_scale) * 1.4426950408889634f;
    const int total_rows = cu_q ? kv_append : bsz * q_len;
    return attn_impl(ctx, (cudaStream_t)stream, p, total_rows, q_len, false);
}

extern "C" int exl3_bighead_attn_paged_q(exl3_ctx* ctx, exl3_stream stream, const void* q, const void* k,
                                         const void* v, void* qk, void* sk, void* qv, void* sv,
                                         const int32_t* block_table, const int32_t* cache_seqlens, const int32_t* cu_q,
                                         void* o, int bsz, int q_len, int kv_append, int nq, int nkv, int hd, int pages,
                                         int pages_per_seq, int k_bits, int v_bits, int kv_chunk_size, int causal,
                                         float sm_scale, float compand_a)
{
    (void)kv_chunk_size;
    int rc = check_common(ctx, q, o, block_table, cache_seqlens, bsz, q_len, kv_append, nq, nkv, hd, pages, pages_per_seq);
    if (rc) return rc;
    EXL3_REQUIRE(qk && sk && qv && sv, "attention: null quantised pool");
    EXL3_REQUIRE(k_bits >= 2 && k_bits <= 8 && v_bits >= 2 && v_bits <= 8, "attention: bits must be 2..8");
    if (compand_a > 0.0f) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "attention: compand_a > 0 is not supported");
    if (bsz == 0 || q_len == 0) return EXL3_OK;
    const int append = cu_q ? q_len : kv_append;
    if (append > 0) {
        EXL3_REQUIRE(k && v, "attention: kv_append > 0 needs k and v");
        rc = exl3_quant_cache_paged(ctx, stream, k, qk, sk, v, qv, sv, cache_seqlens, block_table, cu_q, bsz, append,
                                    nkv * hd, pages, pages_per_seq, k_bits, v_bits, EXL3_PAGE, 0.0f, 1);
        if (rc) return rc;
    }
    AttnParams p;
    memset(&p, 0, sizeof(p));
    p.q = (const half*)q; p.o = (half*)o;
    p.qk = (const uint32_t*)qk; p.sk = (const half*)sk; p.qv = (const uint32_t*)qv; p.sv = (const half*)sv;
    p.block_table = block_table; p.seqlens = cache_seqlens; p.cu_q = cu_q;
    p.bsz = bsz; p.q_len = q_len; p.kv_append = kv_append; p.nq = nq; p.nkv = nkv; p.pps = pages_per_seq; p.pages = pages;
    p.causal = causal; p.k_bits = k_bits; p.v_bits = v_bits;
    p.scale_log2 = (sm_scale == 0.0f ? rsqrtf((float)hd) : sm_scale) * 1.4426950408889634f;
    const int total_rows = cu_q ? kv_append : bsz * q_len;
    return attn_impl(ctx, (cudaStream_t)stream, p, total_rows, q_len, true);
}

// Attention over plain tensors: q, o [bsz, q_len, nq, hd], k, v [bsz, kv_len, nkv, hd], no cache and no block table
// (kernels/attention.cu:2292-2437).  A causal query i sees keys <= kv_len - q_len + i (:1476).  Runs the mma.sync kernels
// with the key index taken straight from the sequence's base; kv_chunk_size is accepted and ignored (the split size comes
// from the work list).
extern "C" int exl3_bighead_attn(exl3_ctx* ctx, exl3_stream stream, const void* q, const void* k, const void* v, void* o,
                                 int bsz, int q_len, int kv_len, int nq, int nkv, int hd, int kv_chunk_size, int causal,
                                 float sm_scale)
{
    EXL3_REQUIRE(ctx && q && k && v && o, "attention: null argument");
    EXL3_REQUIRE(bsz >= 0 && q_len >= 0 && kv_len >= 0 && nq > 0 && nkv > 0, "attention: bad shape");
    EXL3_REQUIRE(kv_chunk_size > 0, "attention: kv_chunk_size must be positive");
    EXL3_REQUIRE(nq % nkv == 0, "attention: n_q_heads must be a multiple of n_kv_heads");
    EXL3_REQUIRE(nq / nkv <= 16, "attention: GQA ratio above 16");
    if (hd != 128) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "attention: head_dim must be 128");
    EXL3_REQUIRE(nkv <= 65535, "attention: too many kv heads");
    EXL3_REQUIRE(aligned16(q) && aligned16(o) && aligned16(k) && aligned16(v), "attention: pointers must be 16-byte aligned");
    if (bsz == 0 || q_len == 0) return EXL3_OK;
    if (kv_len == 0)                                      // nothing to attend to: the reference writes zeros (l = 0)
        return cudaMemsetAsync(o, 0, (size_t)bsz * q_len * nq * hd * 2, (cudaStream_t)stream) == cudaSuccess
                   ? EXL3_OK : exl3_fail(ctx, EXL3_ERR_CUDA, "attention: cudaMemsetAsync failed");
    AttnParams p;
    memset(&p, 0, sizeof(p));
    p.q = (const half*)q; p.o = (half*)o; p.kc = (const half*)k; p.vc = (const half*)v;
    p.bsz = bsz; p.q_len = q_len; p.kv_append = kv_len; p.contig_kv = kv_len; p.nq = nq; p.nkv = nkv; p.pps = 1; p.pages = 1;
    p.causal = causal;
    p.scale_log2 = (sm_scale == 0.0f ? rsqrtf((float)hd) : sm_scale) * 1.4426950408889634f;
    // the work lists kept across the layers of a step belong to the paged batch: plan afresh
    const int keep = ctx->plan_keep;
    ctx->plan_keep = 0;
    const int rc = attn_impl(ctx, (cudaStream_t)stream, p, bsz * q_len, q_len, false);
    ctx->plan_keep = keep;
    return rc;
}
